"""Compiles the CUDA sources under ``csrc/`` for sm_100a, one shared library per
source file, and loads them with ctypes.

Nothing is compiled at import.  A kernel module is built the first time it is
asked for (``module("norm")``), so a model compiles what it needs and no more;
``build_all`` compiles everything.  Libraries land in ``csrc/_build`` inside
the package, or, when that folder cannot be written, in a per-user folder under
the system's temporary directory.  A library is reused only while the hash of
its source, of the shared header and of the compiler flags is unchanged.

There is no fallback: if a library is missing and cannot be compiled, the call
raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
NVCC_FLAGS += os.environ.get("GROUT_B200_NVCC_FLAGS", "").split()   # e.g. -DNAME for experiments

_LOCK = threading.Lock()
_LOADED: Dict[str, ctypes.CDLL] = {}


class KernelBuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[grout_b200] {msg}", file=sys.stderr, flush=True)


def sources() -> List[str]:
    return sorted(f[:-3] for f in os.listdir(CSRC) if f.endswith(".cu"))


def _nvcc() -> str:
    cands = []
    if os.environ.get("CUDA_HOME"):
        cands.append(os.path.join(os.environ["CUDA_HOME"], "bin", "nvcc"))
    cands.append(shutil.which("nvcc") or "")
    cands.append("/usr/local/cuda/bin/nvcc")
    for c in cands:
        if c and os.path.exists(c):
            return c
    raise KernelBuildError("nvcc not found (looked at $CUDA_HOME/bin, PATH, /usr/local/cuda/bin); "
                           "the CUDA kernels cannot be compiled and there is no fallback")


def _writable(d: str) -> bool:
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


_BUILD_DIR = None


def build_dir() -> str:
    global _BUILD_DIR
    if _BUILD_DIR is None:
        d = os.environ.get("GROUT_B200_BUILD_DIR") or os.path.join(CSRC, "_build")
        if not _writable(d):
            d = os.path.join(tempfile.gettempdir(), f"grout_b200_build_{os.getuid()}")
            if not _writable(d):
                raise KernelBuildError(f"no writable folder for compiled kernels (tried {d})")
        _BUILD_DIR = d
    return _BUILD_DIR


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in [name + ".cu"] + sorted(x for x in os.listdir(CSRC) if x.endswith((".cuh", ".h"))):
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    return h.hexdigest()


def _lib_path(name: str) -> str:
    return os.path.join(build_dir(), f"libgb_{name}.so")


def is_built(name: str) -> bool:
    so, stamp = _lib_path(name), _lib_path(name) + ".stamp"
    if not (os.path.exists(so) and os.path.exists(stamp)):
        return False
    with open(stamp) as fh:
        return fh.read().strip() == _digest(name)


def compile_module(name: str) -> str:
    """Compiles ``csrc/<name>.cu`` if its library is absent or stale; returns the path."""
    src = os.path.join(CSRC, name + ".cu")
    if not os.path.exists(src):
        raise KernelBuildError(f"no kernel source {src}")
    so = _lib_path(name)
    if is_built(name):
        return so
    nvcc = _nvcc()
    tmp = f"{so}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-o", tmp, src]
    _log(f"compiling {name}.cu for sm_100a ...")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _log(f"... still compiling {name}.cu ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed for {name}.cu:\n{out.decode(errors='replace')}")
    os.replace(tmp, so)
    with open(so + ".stamp", "w") as fh:
        fh.write(_digest(name))
    _log(f"compiled {name}.cu in {time.time() - t0:.1f} s")
    return so


def compile_modules(names: Iterable[str]) -> None:
    """Compiles several modules side by side."""
    todo = [n for n in dict.fromkeys(names) if not is_built(n)]
    if not todo:
        return
    with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as ex:
        list(ex.map(compile_module, todo))


def build_all() -> None:
    compile_modules(sources())


def module(name: str) -> ctypes.CDLL:
    """The loaded library of ``csrc/<name>.cu`` (compiled first if need be)."""
    lib = _LOADED.get(name)
    if lib is not None:
        return lib
    with _LOCK:
        lib = _LOADED.get(name)
        if lib is None:
            path = compile_module(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            _LOADED[name] = lib
    return lib


def loaded_modules() -> List[str]:
    return sorted(_LOADED)
