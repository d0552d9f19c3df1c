"""Reading and writing the safetensors container.

Layout: 8 bytes little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": ...}``
and the raw little-endian tensor data.  A model folder holds either one
``model.safetensors`` or shards named by ``model.safetensors.index.json``'s
``weight_map`` (the reference accepts only the latter, src/loader.rs:26-50).

Files are memory-mapped; a tensor is a view of the map until it is copied to
the device, so a checkpoint larger than host memory still loads.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    file: str
    begin: int        # absolute byte offset in the file
    end: int


class SafetensorsFile:
    """One memory-mapped safetensors file."""

    def __init__(self, path: str):
        self.path = path
        self._fh = open(path, "rb")
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        base = 8 + hlen
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            dt = _DTYPES.get(info.get("dtype"))
            if dt is None:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype "
                                       f"{info.get('dtype')!r}")
            b, e = info["data_offsets"]
            shape = tuple(int(s) for s in info["shape"])
            n = 1
            for s in shape:
                n *= s
            if e - b != n * torch.empty((), dtype=dt).element_size() or base + e > size:
                raise SafetensorsError(f"{path}: tensor '{name}' has inconsistent offsets")
            self.entries[name] = TensorEntry(name, dt, shape, path, base + b, base + e)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the map (read-only: copy before writing)."""
        e = self.entries[name]
        n = 1
        for s in e.shape:
            n *= s
        if n == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            flat = torch.frombuffer(self._map, dtype=e.dtype, count=n, offset=e.begin)
        return flat.reshape(e.shape)

    def close(self):
        # views may still be alive; the map is closed by the garbage collector then
        try:
            self._fh.close()
        except Exception:
            pass


class Checkpoint:
    """All tensors of a model folder, by name, over one or many files."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self.files: Dict[str, SafetensorsFile] = {}
        self.where: Dict[str, str] = {}
        if os.path.exists(index):
            with open(index, "r", encoding="utf-8") as fh:
                try:
                    weight_map = json.load(fh)["weight_map"]
                except (json.JSONDecodeError, KeyError) as e:
                    raise SafetensorsError(f"{index}: cannot read weight_map ({e})") from None
            for shard in sorted(set(weight_map.values())):
                path = os.path.join(model_dir, shard)
                if not os.path.exists(path):
                    raise SafetensorsError(f"{index} names shard '{shard}', which is missing")
                self.files[shard] = SafetensorsFile(path)
            for shard, f in self.files.items():
                for name in f.entries:
                    self.where[name] = shard
        elif os.path.exists(single):
            self.files["model.safetensors"] = SafetensorsFile(single)
            self.where = {n: "model.safetensors" for n in self.files["model.safetensors"].entries}
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor "
                                   f"model.safetensors.index.json found")

    def names(self) -> List[str]:
        return sorted(self.where)

    def entry(self, name: str) -> TensorEntry:
        return self.files[self.where[name]].entries[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self.files[self.where[name]].tensor(name)


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Dict[str, str] | None = None) -> None:
    """Writes tensors in the order given.  The iterable is walked twice (sizes,
    then data) unless it is a list, so pass a list or a re-iterable."""
    items = list(tensors)
    header, offset = {}, 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for _name, t in items:
            c = t.detach().contiguous().cpu()
            fh.write(c.reshape(-1).view(torch.uint8).numpy().tobytes() if c.numel() else b"")
    os.replace(tmp, path)
