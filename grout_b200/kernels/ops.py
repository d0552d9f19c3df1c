"""Typed, checked entry points of the CUDA kernels.

Each function takes torch CUDA tensors, checks dtype, shape and contiguity,
and launches the kernel on torch's current stream.  Nothing here computes: a
tensor that is not on the GPU, or a size a kernel does not take, raises.
"""
from __future__ import annotations

import ctypes
import functools
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Tuple

import torch

from .build import module

_P, _I, _F, _L = c_void_p, c_int, c_float, c_longlong
_CODES = {"p": _P, "i": _I, "f": _F, "l": _L}
_FUNCS = {}


class KernelError(RuntimeError):
    pass


_OWN_ERRORS = {-1: "the kernel refused its arguments (bad size or pointer)",
               -2: "no kernel for this combination of sizes and types",
               -3: "size beyond the kernel's stated maximum"}


def _fn(mod: str, name: str, sig: str):
    key = (mod, name)
    f = _FUNCS.get(key)
    if f is None:
        f = getattr(module(mod), name)
        f.argtypes = [_CODES[c] for c in sig]
        f.restype = c_int
        _FUNCS[key] = f
    return f


_LAUNCHES = 0


def launch_count() -> int:
    """Kernel launches made through this module so far (a decode-attention call
    with more than one split counts its merge kernel too)."""
    return _LAUNCHES


class OpProfile:
    """Per-operation device times of steps that are launched one by one (not
    replayed from a graph): CUDA events around every call of this module, with
    the bytes each call has to move and the flops it has to do, so that the
    report can set every kernel against the machine's peaks.  (The reference's
    per-op totals: src/model.rs:1139-1142, 1183-1207, filled at 4370-4379.)"""

    def __init__(self, hbm_gbs: Optional[float] = None, tflops: Optional[float] = None,
                 lead_us: int = 80):
        """``lead_us``: how long the device is kept busy in front of every timed
        call (a timer kernel), so that the call and its events are queued by the
        time the device gets to them and the interval is the kernel's own; 0
        for none."""
        self.hbm_gbs, self.tflops, self.lead_us = hbm_gbs, tflops, int(lead_us)
        self.records = []          # (name, start event, end event, bytes, flops); the last two may be callables

    def add(self, name, a, b, nbytes, flops) -> None:
        self.records.append((name, a, b, nbytes, flops))

    def totals(self):
        """name -> [calls, ms, bytes, flops], after waiting for the device."""
        torch.cuda.synchronize()
        out = {}
        for name, a, b, nbytes, flops in self.records:
            r = out.setdefault(name, [0, 0.0, 0.0, 0.0])
            r[0] += 1
            r[1] += a.elapsed_time(b)
            r[2] += float(nbytes() if callable(nbytes) else nbytes)
            r[3] += float(flops() if callable(flops) else flops)
        return out

    def report(self) -> str:
        rows = sorted(self.totals().items(), key=lambda kv: -kv[1][1])
        whole = sum(r[1] for _n, r in rows) or 1.0
        head = ("op profile (an event pair around every call, each kernel alone on the device; steps are "
                "not replayed from graphs)\n")
        head += f"  {'op':<22}{'calls':>7}{'total_ms':>10}{'avg_us':>9}{'share':>7}{'GB/s':>9}{'TFLOP/s':>9}"
        if self.hbm_gbs or self.tflops:
            head += f"{'of hbm':>8}{'of mma':>8}"
        lines = [head]
        for name, (calls, ms, nbytes, flops) in rows:
            gbs = nbytes / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
            tfs = flops / (ms * 1e-3) / 1e12 if ms > 0 else 0.0
            line = (f"  {name:<22}{calls:>7}{ms:>10.3f}{ms / calls * 1e3:>9.2f}{ms / whole:>7.1%}"
                    f"{gbs:>9.0f}{tfs:>9.1f}")
            if self.hbm_gbs or self.tflops:
                line += f"{(gbs / self.hbm_gbs if self.hbm_gbs else 0):>8.2f}"
                line += f"{(tfs / self.tflops if self.tflops else 0):>8.2f}"
            lines.append(line)
        return "\n".join(lines)


_PROFILE: Optional[OpProfile] = None


def set_profile(profile: Optional[OpProfile]) -> None:
    """Turns the per-operation profile on (an ``OpProfile``) or off (None)."""
    global _PROFILE
    _PROFILE = profile


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if isinstance(t, torch.Tensor))


def _profiled(name: str, cost):
    """Decorator: with a profile on, brackets the call with events and notes
    ``cost(result, *args, **kw) -> (bytes, flops)``."""
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*args, **kw):
            prof = _PROFILE
            if prof is None:
                return fn(*args, **kw)
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            if prof.lead_us:
                _fn("elementwise", "gb_delay_ns", "lp")(prof.lead_us * 1000, _stream())
            a.record()
            out = fn(*args, **kw)
            b.record()
            nbytes, flops = cost(out, *args, **kw)
            prof.add(name, a, b, nbytes, flops)
            return out
        return wrapper
    return deco


def _cost_io(out, *args, **kw):
    """What goes in and what comes out, each once."""
    outs = out if isinstance(out, (tuple, list)) else (out,)
    return _nbytes(*args, *kw.values(), *outs), 0


def _cost_gemm(out, x, w, *args, **kw):
    M, K = x.shape
    N = w.shape[0]
    return _nbytes(x, w, out), 2.0 * M * N * K


def _cost_attention(out, q, k_pages, *args, **kw):
    """Keys and values of the live sequences once, q in, the result out; flops of
    the two products over the keys every query row sees (lengths are on the
    device: they are read when the report is made)."""
    nq, D = q.shape[1], q.shape[2]
    nkv, item = k_pages.shape[1], k_pages.element_size()
    kv_len, slots, cu_q, window = kw.get("kv_len"), kw.get("slots"), kw.get("cu_q"), kw.get("window")
    if kv_len is None:
        return _nbytes(q, out), 0
    live = (slots >= 0)
    lens = torch.where(live, kv_len, torch.zeros_like(kv_len)).double()
    if cu_q is not None:
        rows = torch.where(live, cu_q[1:] - cu_q[:-1], torch.zeros_like(kv_len)).double()
    else:
        rows = live.double()
    pairs = rows * (lens - rows) + rows * (rows + 1) / 2        # (query, visible key) pairs, causal
    if window:
        pairs = torch.minimum(pairs, rows * float(window))
        lens = torch.minimum(lens, rows + float(window))
    kv_bytes = (lens.sum() * (2 * nkv * D * item))
    pair_sum = pairs.sum()
    base = _nbytes(q, out)
    return (lambda: base + float(kv_bytes.item())), (lambda: 4.0 * nq * D * float(pair_sum.item()))


def _cost_qk_prepare(out, qkv, nq, nkv, D):
    """The projection in, q out, and k and v out (to their pages or to a tensor)."""
    q = out[0]
    kv_bytes = q.shape[0] * 2 * nkv * D * q.element_size()
    return _nbytes(qkv, q) + kv_bytes, 0


LAUNCH_LOG: Optional[list] = None     # when a list: one label per kernel launched, in order


def _check(rc: int, what: str, kernels: int = 1, detail: str = "") -> None:
    global _LAUNCHES
    if rc == 0:
        _LAUNCHES += kernels
        if LAUNCH_LOG is not None and kernels > 0:
            LAUNCH_LOG.extend([what + detail] + [what + " (second kernel)"] * (kernels - 1))
        return
    if rc in _OWN_ERRORS:
        raise KernelError(f"{what}: {_OWN_ERRORS[rc]}")
    raise KernelError(f"{what}: CUDA error {rc} at launch ({_cuda_error_name(rc)})")


def _cuda_error_name(rc: int) -> str:
    try:
        return str(torch.cuda.cudart().cudaGetErrorString(torch.cuda.cudart().cudaError(rc)))
    except Exception:
        return "cudaError_t value"


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _suffix(dtype: torch.dtype) -> str:
    if dtype == torch.float32:
        return "f32"
    if dtype == torch.bfloat16:
        return "bf16"
    raise KernelError(f"kernels take float32 or bfloat16 activations, not {dtype}")


def _need(t: Optional[torch.Tensor], name: str, dtype=None, ndim=None) -> None:
    if t is None:
        raise KernelError(f"{name} is missing")
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: there is no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, found {tuple(t.shape)}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


# ---------------------------------------------------------------- embedding
@_profiled("embed", lambda out, table, ids: (_nbytes(ids, out, out), 0))
def embed(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    _need(table, "embedding table", ndim=2)
    _need(ids, "token ids", torch.int32, 1)
    V, H = table.shape
    out = torch.empty((ids.shape[0], H), dtype=table.dtype, device=table.device)
    sfx = _suffix(table.dtype)
    _check(_fn("embed", f"gb_embed_{sfx}", "pppiiip")(
        table.data_ptr(), ids.data_ptr(), out.data_ptr(), ids.shape[0], H, V, _stream()), "embed")
    return out


# ---------------------------------------------------------------- norm
@_profiled("add_rmsnorm", _cost_io)
def add_rmsnorm(res_in: Optional[torch.Tensor], delta: Optional[torch.Tensor],
                weight: torch.Tensor, eps: float, *, dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None, write_res: bool = True
                ) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
    """(res_in + delta) in 32-bit -> (residual, normed).  Without ``rows`` the
    residual is updated in place when ``res_in`` is given.  ``delta`` may also be
    a stack of 32-bit partial sums [S, T, N] (what a split-K product leaves): they
    are added in order."""
    parts = None
    if delta is not None and delta.dim() == 3:
        _need(delta, "partial sums", torch.float32, 3)
        parts, delta = delta, None
    src = res_in if res_in is not None else (delta if delta is not None else
                                             (parts[0] if parts is not None else None))
    if src is None:
        raise KernelError("add_rmsnorm needs a residual or a delta")
    if res_in is not None:
        _need(res_in, "residual", torch.float32, 2)
    if delta is not None:
        _need(delta, "delta", dtype, 2)
        if res_in is not None and delta.shape != res_in.shape:
            raise KernelError(f"residual {tuple(res_in.shape)} and delta {tuple(delta.shape)} differ")
    if parts is not None and res_in is not None and tuple(parts.shape[1:]) != tuple(res_in.shape):
        raise KernelError(f"residual {tuple(res_in.shape)} and partial sums {tuple(parts.shape)} differ")
    _need(weight, "norm weight", ndim=1)
    N = src.shape[1]
    if weight.shape[0] != N:
        raise KernelError(f"norm weight has {weight.shape[0]} elements for rows of {N}")
    w_is_f32 = weight.dtype == torch.float32
    if not w_is_f32 and weight.dtype != dtype:
        raise KernelError(f"norm weight must be float32 or {dtype}, found {weight.dtype}")
    if rows is not None:
        _need(rows, "row list", torch.int32, 1)
        n_rows = rows.shape[0]
    else:
        n_rows = src.shape[0]
    res_out = None
    if write_res:
        if rows is None and res_in is not None:
            res_out = res_in
        else:
            res_out = torch.empty((n_rows, N), dtype=torch.float32, device=src.device)
    y = torch.empty((n_rows, N), dtype=dtype, device=src.device)
    sfx = _suffix(dtype)
    _check(_fn("norm", f"gb_add_rmsnorm_{sfx}", "pppilppifppiip")(
        _ptr(res_in), _ptr(delta), _ptr(parts), 0 if parts is None else parts.shape[0],
        0 if parts is None else parts.stride(0), _ptr(rows), weight.data_ptr(), int(w_is_f32),
        float(eps), _ptr(res_out), y.data_ptr(), n_rows, N, _stream()), "add_rmsnorm")
    return res_out, y


# ---------------------------------------------------------------- q/k preparation
class _QkPrepareArgs(ctypes.Structure):
    _fields_ = [("qkv", _P), ("q_w", _P), ("k_w", _P), ("inv_freq", _P), ("token_seq", _P),
                ("token_pos", _P), ("slots", _P), ("block_table", _P), ("q_out", _P),
                ("kv_out", _P), ("k_pages", _P), ("v_pages", _P), ("eps", _F),
                ("n_tokens", _I), ("nq", _I), ("nkv", _I), ("D", _I), ("rot_dim", _I),
                ("max_pages", _I), ("page", _I), ("qkv_parts", _P), ("n_parts", _I),
                ("part_stride", _L)]


@_profiled("qk_prepare", lambda out, qkv, nq, nkv, D, **k: _cost_qk_prepare(out, qkv, nq, nkv, D))
def qk_prepare(qkv: torch.Tensor, nq: int, nkv: int, D: int, *, q_w=None, k_w=None,
               eps: float = 0.0, inv_freq=None, rot_dim: int = 0, token_seq, token_pos, slots,
               block_table=None, k_pages=None, v_pages=None, page: int = 0,
               want_kv_out: bool = False):
    """Returns (q [T, nq, D], kv_out or None); writes k, v into the pages when given.
    ``qkv`` may be a stack of 32-bit partial sums [S, T, width] of the projection
    (bf16 engines only): they are added in order."""
    parts = None
    if qkv.dim() == 3:
        _need(qkv, "qkv partial sums", torch.float32, 3)
        if k_pages is not None and k_pages.dtype != torch.bfloat16:
            raise KernelError("partial sums of qkv are taken with a bfloat16 cache only")
        parts, dt = qkv, torch.bfloat16
    else:
        _need(qkv, "qkv", ndim=2)
        dt = qkv.dtype
    T = qkv.shape[-2]
    if qkv.shape[-1] != (nq + 2 * nkv) * D:
        raise KernelError(f"qkv has {qkv.shape[-1]} columns, expected (nq + 2 nkv) * D = "
                          f"{(nq + 2 * nkv) * D}")
    w_is_f32 = int(dt == torch.float32)      # without norm weights: whatever the entry point takes
    for w, nm in ((q_w, "q norm weight"), (k_w, "k norm weight")):
        if w is not None:
            _need(w, nm, ndim=1)
            if w.shape[0] != D:
                raise KernelError(f"{nm} has {w.shape[0]} elements for head_dim {D}")
            w_is_f32 = int(w.dtype == torch.float32)
    if q_w is not None and k_w is not None and q_w.dtype != k_w.dtype:
        raise KernelError("q and k norm weights must have one dtype")
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] * 2 != rot_dim:
            raise KernelError("inv_freq must hold rot_dim / 2 entries")
    _need(token_pos, "token_pos", torch.int32, 1)
    _need(token_seq, "token_seq", torch.int32, 1)
    _need(slots, "slots", torch.int32, 1)
    q = torch.empty((T, nq, D), dtype=dt, device=qkv.device)
    kv_out = torch.empty((T, 2 * nkv, D), dtype=dt, device=qkv.device) if want_kv_out else None
    a = _QkPrepareArgs()
    a.qkv, a.q_w, a.k_w, a.inv_freq = (None if parts is not None else qkv.data_ptr()), _ptr(q_w), \
        _ptr(k_w), _ptr(inv_freq)
    if parts is not None:
        a.qkv_parts, a.n_parts, a.part_stride = parts.data_ptr(), parts.shape[0], parts.stride(0)
    a.token_seq, a.token_pos, a.slots = token_seq.data_ptr(), token_pos.data_ptr(), slots.data_ptr()
    a.q_out, a.kv_out = q.data_ptr(), _ptr(kv_out)
    a.eps, a.n_tokens, a.nq, a.nkv, a.D, a.rot_dim = float(eps), T, nq, nkv, D, int(rot_dim)
    if k_pages is not None:
        _need(k_pages, "k pages", dt, 4)
        _need(v_pages, "v pages", dt, 4)
        _need(block_table, "block table", torch.int32, 2)
        if tuple(k_pages.shape[1:]) != (nkv, page, D) or v_pages.shape != k_pages.shape:
            raise KernelError(f"pages are {tuple(k_pages.shape)}, expected [*, {nkv}, {page}, {D}]")
        a.block_table, a.k_pages, a.v_pages = block_table.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr()
        a.max_pages, a.page = block_table.shape[1], page
    sfx = _suffix(dt)
    f = _fn("qk_prepare", f"gb_qk_prepare_{sfx}", "pip")
    _check(f(ctypes.addressof(a), w_is_f32, _stream()), "qk_prepare")
    return q, kv_out


@_profiled("kv_write", lambda out, kv, *a, **k: (2 * _nbytes(kv), 0))
def kv_write(kv: torch.Tensor, nkv: int, D: int, *, token_seq, token_pos, slots, block_table,
             k_pages, v_pages, page: int) -> None:
    _need(kv, "kv rows", ndim=3)
    if tuple(kv.shape[1:]) != (2 * nkv, D):
        raise KernelError(f"kv rows are {tuple(kv.shape)}, expected [T, {2 * nkv}, {D}]")
    _need(k_pages, "k pages", kv.dtype, 4)
    _need(v_pages, "v pages", kv.dtype, 4)
    _need(block_table, "block table", torch.int32, 2)
    sfx = _suffix(kv.dtype)
    _check(_fn("qk_prepare", f"gb_kv_write_{sfx}", "pppppppiiiiip")(
        kv.data_ptr(), token_seq.data_ptr(), token_pos.data_ptr(), slots.data_ptr(),
        block_table.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), kv.shape[0], nkv, D,
        block_table.shape[1], page, _stream()), "kv_write")


# ---------------------------------------------------------------- attention
def _attn_common(q, k_pages, v_pages, block_table, token_seq, token_pos, slots, page):
    _need(q, "q", ndim=3)
    T, nq, D = q.shape
    _need(k_pages, "k pages", q.dtype, 4)
    _need(v_pages, "v pages", q.dtype, 4)
    nkv = k_pages.shape[1]
    if tuple(k_pages.shape[1:]) != (nkv, page, D) or v_pages.shape != k_pages.shape:
        raise KernelError(f"pages are {tuple(k_pages.shape)}, expected [*, nkv, {page}, {D}]")
    if nq % nkv:
        raise KernelError(f"{nq} query heads cannot share {nkv} kv heads")
    _need(block_table, "block table", torch.int32, 2)
    _need(token_seq, "token_seq", torch.int32, 1)
    _need(token_pos, "token_pos", torch.int32, 1)
    _need(slots, "slots", torch.int32, 1)
    return T, nq, nkv, D


@_profiled("attn_generic", lambda out, q, *a, **k: (_nbytes(q, out), 0))
def attn_generic(q, k_pages, v_pages, block_table, *, token_seq, token_pos, slots, page: int,
                 scale: float, window: Optional[int] = None) -> torch.Tensor:
    T, nq, nkv, D = _attn_common(q, k_pages, v_pages, block_table, token_seq, token_pos, slots, page)
    out = torch.empty_like(q)
    sfx = _suffix(q.dtype)
    _check(_fn("attn_generic", f"gb_attn_generic_{sfx}", "ppppippppiiiiifip")(
        q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], token_seq.data_ptr(), token_pos.data_ptr(), slots.data_ptr(),
        out.data_ptr(), T, nq, nkv, D, page, float(scale), int(window or 0), _stream()),
        "attn_generic")
    return out


# ---------------------------------------------------------------- matrix products
@_profiled("gemm_f32", _cost_gemm)
def gemm_f32(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """a [M, K] . w [N, K]^T in true 32-bit on the CUDA cores."""
    _need(a, "activations", torch.float32, 2)
    _need(w, "weight", torch.float32, 2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"weight is {tuple(w.shape)} for activations of width {K}")
    c = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _check(_fn("gemm_f32", "gb_gemm_nt_f32", "pppiiiiiip")(
        a.data_ptr(), w.data_ptr(), c.data_ptr(), M, N, K, K, K, N, _stream()), "gemm_f32")
    return c


# ---------------------------------------------------------------- elementwise
@_profiled("silu_mul", _cost_io)
def silu_mul(gate_up: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """silu(gate) * up.  ``interleave`` 0: gate in the first half of the columns,
    up in the second; g > 0: groups of g gate columns followed by their g up columns."""
    _need(gate_up, "gate|up", ndim=2)
    T, two_i = gate_up.shape
    if two_i % 2 or (interleave and two_i % (2 * interleave)):
        raise KernelError("gate|up must have an even number of columns (of whole groups)")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    sfx = _suffix(gate_up.dtype)
    _check(_fn("elementwise", f"gb_silu_mul_{sfx}", "ppiiip")(
        gate_up.data_ptr(), out.data_ptr(), T, two_i // 2, int(interleave), _stream()), "silu_mul")
    return out


@_profiled("cast", lambda out, x, dtype: ((0, 0) if out is x else (_nbytes(x, out), 0)))
def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _need(x, "tensor")
    if x.dtype == dtype:
        return x
    pair = {(torch.float32, torch.bfloat16): "gb_cast_f32_to_bf16",
            (torch.bfloat16, torch.float32): "gb_cast_bf16_to_f32"}.get((x.dtype, dtype))
    if pair is None:
        raise KernelError(f"no conversion kernel from {x.dtype} to {dtype}")
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _check(_fn("elementwise", pair, "pplp")(x.data_ptr(), out.data_ptr(), x.numel(), _stream()),
           "cast")
    return out


@_profiled("library_mm", _cost_gemm)
def library_mm(x: torch.Tensor, w: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """x [M, K] . w [N, K]^T by the library's matrix product (cuBLAS through
    torch.mm): the prompt products for which the reference calls a library too
    (src/cublas.rs:287-307).  It is here so that the profile sees it."""
    _need(x, "activations", torch.bfloat16, 2)
    _need(w, "weight", torch.bfloat16, 2)
    if out_dtype == torch.float32:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    return torch.mm(x, w.t())


SKINNY_MAX_ROWS = 64


class _SkinnyArgs(ctypes.Structure):
    _fields_ = [("x", _P), ("W", _P), ("y", _P), ("scratch", _P), ("counters", _P), ("M", _I),
                ("N", _I), ("K", _I)]


class _Workspace:
    """Scratch of the kernels that split a sum over blocks, one per device:
    32-bit partial tiles and arrival counters.  The counters are zero between
    launches (the kernels leave them so).  Launches that share it must be ordered
    on one stream, which every step of this library is."""

    def __init__(self):
        self.scratch = None
        self.counters = None
        self._kept = []     # outgrown buffers stay alive: captured graphs still point at them

    def get(self, device, n_floats: int, n_counters: int):
        if self.scratch is None or self.scratch.numel() < n_floats:
            self._kept.append(self.scratch)
            self.scratch = torch.empty(max(n_floats, 1 << 22), dtype=torch.float32, device=device)
        if self.counters is None or self.counters.numel() < n_counters:
            self._kept.append(self.counters)
            self.counters = torch.zeros(max(n_counters, 1 << 16), dtype=torch.int32, device=device)
        return self.scratch, self.counters


_WORKSPACES = {}
_SKINNY_PLANS = {}


def skinny_plan(M: int, N: int, K: int, out_f32: bool, silu: bool):
    """(blocks, scratch floats, counters) of the decode product for this shape:
    as many blocks as the GPU holds at once, each streaming an equal share of the
    weights; it depends on N, K and M's bucket (<= 8, 16, 32, 64) only."""
    bucket = 8 if M <= 8 else 16 if M <= 16 else 32 if M <= 32 else 64
    key = (bucket, N, K, bool(out_f32), bool(silu), torch.cuda.current_device())
    plan = _SKINNY_PLANS.get(key)
    if plan is None:
        out = (c_int * 3)()
        _check(_fn("gemm_skinny_bf16", "gb_gemm_skinny_plan", "iiiiip")(
            bucket, N, K, int(out_f32), int(silu), ctypes.addressof(out)), "gemm_skinny_plan", 0)
        plan = _SKINNY_PLANS[key] = (out[0], out[1], out[2])
    return plan


@_profiled("gemm_skinny_bf16", _cost_gemm)
def gemm_skinny_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype=torch.bfloat16,
                     silu_mul: bool = False) -> torch.Tensor:
    """x [M <= 64, K] . w [N, K]^T, bf16 in, 32-bit accumulate; the decode-time
    linear.  With ``silu_mul`` the rows of ``w`` are gate and up rows interleaved
    in groups of 8 and the result is silu(gate) * up, [M, N / 2]."""
    _need(x, "activations", torch.bfloat16, 2)
    _need(w, "weight", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"weight is {tuple(w.shape)} for activations of width {K}")
    if M > SKINNY_MAX_ROWS:
        raise KernelError(f"gemm_skinny_bf16 takes at most {SKINNY_MAX_ROWS} rows, got {M}")
    if K % 8:
        raise KernelError(f"gemm_skinny_bf16 needs an inner size that is a multiple of 8, got {K}")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"output must be bfloat16 or float32, not {out_dtype}")
    if silu_mul and N % 16:
        raise KernelError(f"the interleaved gate|up product needs N to be a multiple of 16, got {N}")
    y = torch.empty((M, N // 2 if silu_mul else N), dtype=out_dtype, device=x.device)
    if M == 0:
        return y
    with torch.cuda.device(x.device):
        _blocks, n_floats, n_counters = skinny_plan(M, N, K, out_dtype == torch.float32, silu_mul)
        ws = _WORKSPACES.setdefault(x.device.index or 0, _Workspace())
        scratch, counters = ws.get(x.device, n_floats, n_counters)
        a = _SkinnyArgs()
        a.x, a.W, a.y = x.data_ptr(), w.data_ptr(), y.data_ptr()
        a.scratch, a.counters = scratch.data_ptr(), counters.data_ptr()
        a.M, a.N, a.K = M, N, K
        _check(_fn("gemm_skinny_bf16", "gb_gemm_skinny_bf16", "piip")(
            ctypes.addressof(a), int(out_dtype == torch.float32), int(silu_mul), _stream()),
            "gemm_skinny_bf16")
    return y


# ---------------------------------------------------------------- tcgen05 matrix product
class _TcArgs(ctypes.Structure):
    _fields_ = [("out", _P), ("scratch", _P), ("counters", _P), ("error", _P), ("rowsA", _I),
                ("rowsB", _I), ("K", _I), ("ld", _I), ("transpose_out", _I), ("out_f32", _I),
                ("silu", _I), ("dep_b", _I), ("stamps", _P), ("split_k", _I)]


_TC_PLANS = {}
_TC_ERRORS = {}
_TC_ERROR_NAMES = {111: "a role of the tcgen05 attention kernel waited 2 s on a barrier",
                   101: "the MMA warp waited 2 s for a stage that never arrived",
                   102: "the TMA producer waited 2 s for a stage that was never released",
                   103: "the epilogue waited 2 s for an accumulator that was never finished",
                   104: "the MMA warp waited 2 s for an accumulator that was never drained",
                   121: "the pair product's MMA lane waited 2 s for a stage that never arrived",
                   122: "the pair product's producer waited 2 s for a stage that was never released",
                   123: "the pair product's epilogue waited 2 s for an accumulator that was never finished",
                   124: "the pair product's MMA lane waited 2 s for an accumulator that was never drained"}


def _tc_error_flag(device) -> torch.Tensor:
    i = torch.device(device).index or 0
    if i not in _TC_ERRORS:
        _TC_ERRORS[i] = torch.zeros(1, dtype=torch.int32, device=device)
    return _TC_ERRORS[i]


def check_kernel_errors() -> None:
    """Reads the flags that kernels with bounded waits set when a wait expires
    (this synchronises with the device); raises if any is set."""
    for i, flag in _TC_ERRORS.items():
        code = int(flag.item())
        if code:
            flag.zero_()
            raise KernelError(f"tensor-memory kernel on cuda:{i}: {_TC_ERROR_NAMES.get(code, code)}")


def tc_wait_selftest(device, limit_us: int = 1000) -> int:
    """Runs the give-up path of the tensor-memory kernels by itself: one block
    whose first role waits ``limit_us`` on a barrier nobody arrives at, records its
    code in the device's error flag and raises the block's abort flag, which ends
    the second role's (long) wait.  Nothing is in flight and nothing else waits.
    Returns how many roles left (2); ``check_kernel_errors`` then raises."""
    dev = torch.device(device)
    left = torch.zeros(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _check(_fn("gemm_tc", "gb_tc_wait_selftest", "plpp")(
            _tc_error_flag(dev).data_ptr(), int(limit_us) * 1000, left.data_ptr(), _stream()),
            "tc_wait_selftest")
    return int(left.item())


@_profiled("gemm_tc_bf16", _cost_gemm)
def gemm_tc_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype=torch.bfloat16,
                 swap: Optional[bool] = None, silu_mul: bool = False,
                 stamps: Optional[torch.Tensor] = None, split_out: bool = False) -> torch.Tensor:
    """x [M, K] . w [N, K]^T on the tcgen05 tensor cores (TMA-fed, accumulator in
    tensor memory).  ``swap``: put the weight rows on the 128-row side of the MMA
    and the activation rows on the narrow side (the layout for few rows); by
    default chosen when M <= 64.  ``silu_mul`` (with swap): the rows of ``w`` are
    gate and up rows interleaved in groups of 8 and the result is
    silu(gate) * up, [M, N / 2].  ``split_out`` (with swap): when the product has
    too few tiles to fill the GPU, K is cut S ways and the S 32-bit partial
    products are returned as [S, M, N] for the consumer to add (its norm or q/k
    preparation does so in the kernel it runs anyway); otherwise the result is the
    ordinary [M, N]."""
    _need(x, "activations", torch.bfloat16, 2)
    _need(w, "weight", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"weight is {tuple(w.shape)} for activations of width {K}")
    if K % 8:
        raise KernelError(f"gemm_tc_bf16 needs an inner size that is a multiple of 8, got {K}")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"output must be bfloat16 or float32, not {out_dtype}")
    swap = (M <= 64) if swap is None else bool(swap)
    if silu_mul and (not swap or N % 16):
        raise KernelError("the interleaved gate|up epilogue needs the swapped layout and N % 16 == 0")
    n_out = N // 2 if silu_mul else N
    y = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    if M == 0:
        return y
    A, B = (w, x) if swap else (x, w)
    with torch.cuda.device(x.device):
        key = (A.shape[0], B.shape[0], K, torch.cuda.current_device())
        plan = _TC_PLANS.get(key)
        if plan is None:
            out = (c_int * 5)()
            _check(_fn("gemm_tc", "gb_gemm_tc_plan", "iiip")(
                A.shape[0], B.shape[0], K, ctypes.addressof(out)), "gemm_tc_plan", 0)
            plan = _TC_PLANS[key] = (out[0], out[1], out[2], out[3], out[4])
        split = plan[4] if (split_out and swap and not silu_mul) else 0
        if split:
            y = torch.empty((split, M, N), dtype=torch.float32, device=x.device)
        ws = _WORKSPACES.setdefault(x.device.index or 0, _Workspace())
        scratch, counters = ws.get(x.device, plan[2], plan[3])
        a = _TcArgs()
        a.out, a.scratch, a.counters = y.data_ptr(), scratch.data_ptr(), counters.data_ptr()
        a.error = _tc_error_flag(x.device).data_ptr()
        a.rowsA, a.rowsB, a.K, a.ld = A.shape[0], B.shape[0], K, n_out
        a.transpose_out, a.out_f32 = int(swap), int(out_dtype == torch.float32 or bool(split))
        a.split_k = split
        a.silu, a.dep_b = int(silu_mul), int(swap)      # the activations are another kernel's output
        a.stamps = _ptr(stamps)     # int64 [blocks, 8]: phase times of every block, for tuning
        _check(_fn("gemm_tc", "gb_gemm_tc_bf16", "pppp")(
            A.data_ptr(), B.data_ptr(), ctypes.addressof(a), _stream()), "gemm_tc_bf16",
            detail=f" {N}x{K}" + (" silu" if silu_mul else "") + (f" split {split}" if split else ""))
    return y


class _Tc2Args(ctypes.Structure):
    _fields_ = [("out", _P), ("error", _P), ("M", _I), ("N", _I), ("K", _I), ("ld", _I),
                ("out_f32", _I), ("silu", _I), ("bn", _I)]


_TC_ERROR_NAMES.update({121: "the pair product's MMA lane waited 2 s for a stage that never arrived",
                        122: "the pair product's loads waited 2 s for a stage that was never released",
                        123: "the pair product's epilogue waited 2 s for an accumulator",
                        124: "the pair product's MMA lane waited 2 s for an accumulator to be drained"})


def gemm_tc2_takes(n_out: int, out_dtype) -> bool:
    """Whether the pair product can store rows of ``n_out`` columns (16 bytes at a time)."""
    return (n_out * (4 if out_dtype == torch.float32 else 2)) % 16 == 0


def gemm_tc2_pays(M: int, N: int, device, fused_silu: bool) -> bool:
    """Whether the pair product is at least as fast as the library's for this shape.
    It is for the gate|up product with its fused SiLU when the rounds of tiles it runs
    are mostly full: the useful share M N / (whole rounds x pairs x 256 x 256) is at
    least 3/4.  Measured (us, pair / library product plus SiLU kernel; N 19,456, K 2,560):
    384 rows (share 0.51) 52 / 39, 512 (0.69) 53 / 51, 768 (0.77) 68 / 69, 1,024 (0.82)
    84 / 85, 2,048 (0.91) 149 / 162; N 51,200, K 5,120: 128 rows (0.45) 109 / 106, 256
    (0.90) 115 / 133, 384 (0.68) 193 / 165, 2,048 (0.98) 722 / 821.  A product without an
    epilogue to fuse never pays: 6,144 x 2,560 at 2,048 rows 47.0 / 46.2, 10,240 x 5,120
    172.7 / 157.2, and the library is ahead at every smaller row count."""
    if not fused_silu:
        return False
    pairs = max(1, _sm_count(device) // 2)
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    whole_rounds = (tiles + pairs - 1) // pairs
    return 4 * M * N >= 3 * whole_rounds * pairs * 256 * 256


@_profiled("gemm_tc2_bf16", _cost_gemm)
def gemm_tc2_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype=torch.bfloat16,
                  silu_mul: bool = False, tile_cols: int = 0) -> torch.Tensor:
    """x [M, K] . w [N, K]^T for many rows on pairs of SMs (tcgen05.mma.cta_group::2,
    tiles of 256 rows and ``tile_cols`` columns: a multiple of 16 up to 256, by
    default chosen by the kernel's launcher for the shape).  ``silu_mul``: the rows of ``w`` are gate and up rows
    interleaved in groups of 8 and the result is silu(gate) * up, [M, N / 2]."""
    _need(x, "activations", torch.bfloat16, 2)
    _need(w, "weight", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"weight is {tuple(w.shape)} for activations of width {K}")
    if K % 8:
        raise KernelError(f"gemm_tc2_bf16 needs an inner size that is a multiple of 8, got {K}")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"output must be bfloat16 or float32, not {out_dtype}")
    if silu_mul and (N % 16 or out_dtype != torch.bfloat16):
        raise KernelError("the interleaved gate|up epilogue needs N % 16 == 0 and a bfloat16 output")
    n_out = N // 2 if silu_mul else N
    if (n_out * (4 if out_dtype == torch.float32 else 2)) % 16:
        raise KernelError(f"gemm_tc2_bf16 stores 16 bytes at a time: {n_out} output columns do not allow it")
    y = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    if M == 0:
        return y
    a = _Tc2Args()
    a.out, a.error = y.data_ptr(), _tc_error_flag(x.device).data_ptr()
    a.M, a.N, a.K, a.ld = M, N, K, n_out
    a.out_f32, a.silu, a.bn = int(out_dtype == torch.float32), int(silu_mul), int(tile_cols)
    with torch.cuda.device(x.device):
        _check(_fn("gemm_tc2", "gb_gemm_tc2_bf16", "pppp")(
            x.data_ptr(), w.data_ptr(), ctypes.addressof(a), _stream()), "gemm_tc2_bf16")
    return y


# ---------------------------------------------------------------- fast bf16 attention
class _PrefillArgs(ctypes.Structure):
    _fields_ = [("q", _P), ("k_pages", _P), ("v_pages", _P), ("block_table", _P), ("cu_q", _P),
                ("slots", _P), ("kv_len", _P), ("out", _P), ("n_seqs", _I), ("nq", _I),
                ("nkv", _I), ("max_pages", _I), ("window", _I), ("n_qblocks", _I),
                ("scale_log2", _F)]


class _DecodeArgs(ctypes.Structure):
    _fields_ = [("q", _P), ("k_pages", _P), ("v_pages", _P), ("block_table", _P), ("slots", _P),
                ("kv_len", _P), ("out", _P), ("part_o", _P), ("part_ml", _P), ("n_seqs", _I),
                ("nq", _I), ("nkv", _I), ("max_pages", _I), ("page", _I), ("window", _I),
                ("n_splits", _I), ("scale_log2", _F)]


_LOG2E = 1.4426950408889634
PREFILL_ROWS = 64          # query rows per block of the prefill kernel
PREFILL_ATTENTION = "tc"      # "tc": tcgen05 where the shape allows; "mma": the mma.sync kernel


def fast_attention_modules(D: int, nq: int, nkv: int, page: int = 64) -> Tuple[str, ...]:
    """The tensor-core attention sources that heads of this shape can reach (a model
    compiles what it needs and no more)."""
    mods: Tuple[str, ...] = ()
    if fast_attention_takes(D, nq, nkv, page):
        mods += ("attn_prefill_bf16", "attn_decode_bf16")
        if attn_prefill_tc_takes(D, nq, nkv, page):
            mods += ("attn_prefill_tc",)
        if attn_decode_tma_takes(D, nq, nkv, page):
            mods += ("attn_decode_tma",)
    return mods
_SM_COUNT = {}


def _sm_count(device) -> int:
    i = torch.device(device).index or 0
    if i not in _SM_COUNT:
        _SM_COUNT[i] = torch.cuda.get_device_properties(i).multi_processor_count
    return _SM_COUNT[i]


def fast_attention_takes(D: int, nq: int, nkv: int, page: int) -> bool:
    """Shapes the tensor-core kernels accept; others go to the plain kernel."""
    return D % 16 == 0 and 16 <= D <= 128 and page == 64 and nq % nkv == 0 and nq // nkv <= 16


def _q_blocks(q_lens, n_qblocks, rows: int, T: int, n_seqs: int) -> int:
    """Blocks of ``rows`` query rows: counted from the host's copy of the
    sequences' row counts, or taken as given (an upper bound; the kernels find each
    block's sequence on the device and blocks beyond the real count do nothing)."""
    if q_lens:
        if sum(q_lens) != T or len(q_lens) != n_seqs:
            raise KernelError("q_lens do not describe the step's rows")
        return sum((n + rows - 1) // rows for n in q_lens)
    if n_qblocks is None:
        return T // rows + n_seqs
    return int(n_qblocks)


@_profiled("attn_prefill_bf16", _cost_attention)
def attn_prefill_bf16(q, k_pages, v_pages, block_table, *, cu_q, slots, kv_len, q_lens=(),
                      page: int, scale: float, window: Optional[int] = None,
                      n_qblocks: Optional[int] = None) -> torch.Tensor:
    """Causal attention of whole prompts (or their continuation) on the tensor
    cores.  The grid is sized from ``q_lens``, the host's copy of the sequences'
    row counts, or, without them, from ``n_qblocks`` (an upper bound of the
    64-row blocks; by default the most the rows and sequences can make)."""
    T, nq, D = q.shape
    _need(q, "q", torch.bfloat16, 3)
    _need(k_pages, "k pages", torch.bfloat16, 4)
    _need(v_pages, "v pages", torch.bfloat16, 4)
    nkv = k_pages.shape[1]
    if tuple(k_pages.shape[1:]) != (nkv, page, D) or v_pages.shape != k_pages.shape:
        raise KernelError(f"pages are {tuple(k_pages.shape)}, expected [*, nkv, {page}, {D}]")
    for t, nm in ((block_table, "block table"), (cu_q, "cu_q"), (slots, "slots"), (kv_len, "kv_len")):
        _need(t, nm, torch.int32)
    n_seqs = slots.shape[0]
    if cu_q.shape[0] != n_seqs + 1 or kv_len.shape[0] != n_seqs:
        raise KernelError("cu_q, slots and kv_len do not describe one list of sequences")
    out = torch.empty_like(q)
    a = _PrefillArgs()
    a.q, a.k_pages, a.v_pages, a.block_table = q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr()
    a.cu_q, a.slots, a.kv_len, a.out = cu_q.data_ptr(), slots.data_ptr(), kv_len.data_ptr(), out.data_ptr()
    a.n_seqs, a.nq, a.nkv, a.max_pages = n_seqs, nq, nkv, block_table.shape[1]
    a.window = int(window or 0)
    a.n_qblocks = _q_blocks(q_lens, n_qblocks, PREFILL_ROWS, T, n_seqs)
    a.scale_log2 = float(scale) * _LOG2E
    _check(_fn("attn_prefill_bf16", "gb_attn_prefill_bf16", "piip")(
        ctypes.addressof(a), D, page, _stream()), "attn_prefill_bf16")
    return out


class _AttnTcArgs(ctypes.Structure):
    _fields_ = [("block_table", _P), ("cu_q", _P), ("slots", _P), ("kv_len", _P), ("out", _P),
                ("error", _P), ("n_seqs", _I), ("nq", _I), ("nkv", _I), ("max_pages", _I),
                ("window", _I), ("n_qblocks", _I), ("scale_log2", _F)]


PREFILL_TC_ROWS = 0        # query rows per block of the tcgen05 prefill kernel: 128, 256 or 0 = by size


def prefill_tc_rows(blocks_of_256: int, nq: int, device) -> int:
    """256 rows a block (two query blocks that share their key tiles, one block
    an SM) unless that leaves most SMs without a block; then 128 (half-size
    blocks, two an SM).  Measured on 32 heads of 128: 512 tokens 21.8 us with 128
    rows against 25.7 us with 256; from 1,024 tokens on 256 rows are faster."""
    if PREFILL_TC_ROWS:
        return PREFILL_TC_ROWS
    return 256 if 5 * blocks_of_256 * nq >= 3 * _sm_count(device) else 128


def attn_prefill_tc_takes(D: int, nq: int, nkv: int, page: int) -> bool:
    return D in (64, 128) and page == 64 and nq % nkv == 0


@_profiled("attn_prefill_tc", _cost_attention)
def attn_prefill_tc(q, k_pages, v_pages, block_table, *, cu_q, slots, kv_len, q_lens=(),
                    page: int, scale: float, window: Optional[int] = None,
                    rows_per_block: int = 0, n_qblocks: Optional[int] = None) -> torch.Tensor:
    """Causal attention of whole prompts (or their continuation) with both
    products on the tcgen05 tensor cores.  Pages must hold finite values in the
    rows beyond a sequence's length (the cache zero-fills its pages).  The grid is
    sized from ``q_lens`` (the host's copy of the row counts) or, without them,
    from ``n_qblocks``, an upper bound of the blocks of ``rows_per_block`` rows."""
    _need(q, "q", torch.bfloat16, 3)
    T, nq, D = q.shape
    _need(k_pages, "k pages", torch.bfloat16, 4)
    _need(v_pages, "v pages", torch.bfloat16, 4)
    nkv = k_pages.shape[1]
    if tuple(k_pages.shape[1:]) != (nkv, page, D) or v_pages.shape != k_pages.shape:
        raise KernelError(f"pages are {tuple(k_pages.shape)}, expected [*, nkv, {page}, {D}]")
    for t, nm in ((block_table, "block table"), (cu_q, "cu_q"), (slots, "slots"), (kv_len, "kv_len")):
        _need(t, nm, torch.int32)
    n_seqs = slots.shape[0]
    if cu_q.shape[0] != n_seqs + 1 or kv_len.shape[0] != n_seqs:
        raise KernelError("cu_q, slots and kv_len do not describe one list of sequences")
    out = torch.empty_like(q)
    a = _AttnTcArgs()
    a.block_table, a.cu_q, a.slots, a.kv_len = (block_table.data_ptr(), cu_q.data_ptr(),
                                                slots.data_ptr(), kv_len.data_ptr())
    a.out, a.error = out.data_ptr(), _tc_error_flag(q.device).data_ptr()
    a.n_seqs, a.nq, a.nkv, a.max_pages = n_seqs, nq, nkv, block_table.shape[1]
    a.window = int(window or 0)
    rows = int(rows_per_block) if rows_per_block else \
        prefill_tc_rows(_q_blocks(q_lens, None, 256, T, n_seqs), nq, q.device)
    a.n_qblocks = _q_blocks(q_lens, n_qblocks, rows, T, n_seqs)
    a.scale_log2 = float(scale) * _LOG2E
    _check(_fn("attn_prefill_tc", "gb_attn_prefill_tc", "ppppiliiip")(
        q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), ctypes.addressof(a), T,
        k_pages.shape[0], D, page, rows, _stream()), "attn_prefill_tc")
    return out


DECODE_SPLITS_OVERRIDE: Optional[int] = None      # for experiments


def decode_splits(n_seqs: int, nkv: int, max_kv_len: int, device) -> int:
    """How many ways the keys of a sequence are split.  Blocks run in waves of
    three per SM; with S splits a block streams 1/S of a sequence's 32-key tiles
    plus a fixed cost of about three tiles (query load, merge, partial store), so
    the step costs waves(S) * (tiles / S + 3).  The smallest S within 3 % of the
    cheapest is taken, with at least 256 keys a split."""
    if DECODE_SPLITS_OVERRIDE:
        return DECODE_SPLITS_OVERRIDE
    slots = 3 * _sm_count(device)
    pairs = max(1, n_seqs * nkv)
    tiles = max(1, (max_kv_len + 31) // 32)
    most = max(1, min(64, (max_kv_len + 255) // 256))
    cost = {s: ((pairs * s + slots - 1) // slots) * (tiles / s + 3.0) for s in range(1, most + 1)}
    best = min(cost.values())
    return min(s for s, c in cost.items() if c <= 1.03 * best)


@_profiled("attn_decode_bf16", _cost_attention)
def attn_decode_bf16(q, k_pages, v_pages, block_table, *, slots, kv_len, page: int, scale: float,
                     max_kv_len: int, window: Optional[int] = None,
                     n_splits: Optional[int] = None) -> torch.Tensor:
    """Attention of one new token per sequence over its cached keys (split-K)."""
    _need(q, "q", torch.bfloat16, 3)
    B, nq, D = q.shape
    _need(k_pages, "k pages", torch.bfloat16, 4)
    _need(v_pages, "v pages", torch.bfloat16, 4)
    nkv = k_pages.shape[1]
    if tuple(k_pages.shape[1:]) != (nkv, page, D) or v_pages.shape != k_pages.shape:
        raise KernelError(f"pages are {tuple(k_pages.shape)}, expected [*, nkv, {page}, {D}]")
    for t, nm in ((block_table, "block table"), (slots, "slots"), (kv_len, "kv_len")):
        _need(t, nm, torch.int32)
    if slots.shape[0] != B or kv_len.shape[0] != B:
        raise KernelError("one slot and one length per query row are needed")
    ns = int(n_splits) if n_splits else decode_splits(B, nkv, max_kv_len, q.device)
    out = torch.empty_like(q)
    part_o = part_ml = None
    if ns > 1:
        # scratch of the split: 32-bit partials of every (sequence, head, split)
        ws = _WORKSPACES.setdefault(q.device.index or 0, _Workspace())
        scratch, _counters = ws.get(q.device, B * nq * ns * (D + 2), 1)
        part_o = scratch[:B * nq * ns * D]
        part_ml = scratch[B * nq * ns * D:B * nq * ns * (D + 2)]
    a = _DecodeArgs()
    a.q, a.k_pages, a.v_pages, a.block_table = q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr()
    a.slots, a.kv_len, a.out = slots.data_ptr(), kv_len.data_ptr(), out.data_ptr()
    a.part_o, a.part_ml = _ptr(part_o), _ptr(part_ml)
    a.n_seqs, a.nq, a.nkv, a.max_pages, a.page = B, nq, nkv, block_table.shape[1], page
    a.window, a.n_splits, a.scale_log2 = int(window or 0), ns, float(scale) * _LOG2E
    _check(_fn("attn_decode_bf16", "gb_attn_decode_bf16", "pip")(
        ctypes.addressof(a), D, _stream()), "attn_decode_bf16", 2 if ns > 1 else 1)
    return out


class _DecodeTmaArgs(ctypes.Structure):
    _fields_ = [("q", _P), ("block_table", _P), ("slots", _P), ("kv_len", _P), ("out", _P),
                ("part_o", _P), ("part_ml", _P), ("counters", _P), ("error", _P), ("n_seqs", _I),
                ("nq", _I), ("nkv", _I), ("max_pages", _I), ("window", _I), ("n_splits", _I),
                ("scale_log2", _F), ("stamps", _P)]


DECODE_TMA_STAMPS: Optional[torch.Tensor] = None      # int64 [blocks, 12] for tuning, or None
_TC_ERROR_NAMES[131] = "a role of the decode attention kernel waited 2 s on a barrier"
# Which decode attention runs: "auto" takes the TMA kernel where the shape allows and the
# step has at least DECODE_TMA_PAIRS (sequence, kv head) pairs, with two stages (three blocks
# an SM) below DECODE_TMA_DEEP_PAIRS pairs and three stages (two blocks an SM) from there
# on, and the cp.async kernel for fewer pairs; "tma" and "mma" force one.  Measured inside
# the decode step at 32 query and 8 kv heads of 128 with 2,100 keys a sequence (ms a step,
# cp.async / TMA with two stages / with three): 1 sequence 2.38 / 2.50 / 2.48, 4 sequences
# 2.57 / 2.57 / 2.55, 8 sequences 2.74 / 2.72 / 2.78, 16 sequences 3.19 / 3.10 / 3.18, 32
# sequences 4.35 / 4.27 / 4.04, 64 sequences 6.41 / 6.22 / 5.99.  Timed by itself, one call
# after the other, the TMA kernel is the faster or the equal at every size (16.8 against
# 17.9 us at 8 sequences, 86 against 97 at 64); inside a step of very few sequences, where
# a short kernel comes before it, its longer start (descriptor fetch, barrier set-up, the
# hand-over from the loading lane) shows.
DECODE_ATTENTION = "auto"
DECODE_TMA_PAIRS = 64
DECODE_TMA_DEEP_PAIRS = 256
DECODE_TMA_STAGES = 0         # tiles of a block in shared memory (0: by the number of pairs)
_ATTN_COUNTERS = {}


def attn_decode_tma_takes(D: int, nq: int, nkv: int, page: int) -> bool:
    return D in (64, 128) and page == 64 and nq % nkv == 0 and nq // nkv <= 16


def decode_tma_splits(n_seqs: int, nkv: int, max_kv_len: int, device, per_sm: int = 2) -> int:
    """How many ways the keys of a sequence are split for the TMA kernel: blocks
    run in waves of ``per_sm`` per SM; with S splits a block streams 1/S of a
    sequence's 64-key tiles plus a fixed cost of about six tiles (descriptor and
    block-table loads before the first copy, the partial store and the combining
    at the end), so the step costs waves(S) * (tiles / S + 6).  The smallest S
    within 3 % of the cheapest is taken, with at least 256 keys a split.
    Measured (us, 32 query and 8 kv heads of 128): 8 sequences of 2,049 keys 16.8
    with the 4 splits this picks (19.8 with 2, 21.7 with 8); 64 sequences 86.3 with
    1 (99.4 with 2); one sequence 9.1 with 8 or 9 (17.7 with 2)."""
    if DECODE_SPLITS_OVERRIDE:
        return DECODE_SPLITS_OVERRIDE
    places = per_sm * _sm_count(device)
    pairs = max(1, n_seqs * nkv)
    tiles = max(1, (max_kv_len + 63) // 64)
    most = max(1, min(64, (max_kv_len + 255) // 256))
    cost = {s: ((pairs * s + places - 1) // places) * (-(-tiles // s) + 6.0) for s in range(1, most + 1)}
    best = min(cost.values())
    return min(s for s, c in cost.items() if c <= 1.03 * best)


@_profiled("attn_decode_tma", _cost_attention)
def attn_decode_tma(q, k_pages, v_pages, block_table, *, slots, kv_len, page: int, scale: float,
                    max_kv_len: int, window: Optional[int] = None,
                    n_splits: Optional[int] = None, stages: int = 0) -> torch.Tensor:
    """Attention of one new token per sequence over its cached keys, the tiles
    brought in by TMA and the splits combined by the block that finishes last (one
    launch).  Heads of 64 or 128, pages of 64 tokens."""
    _need(q, "q", torch.bfloat16, 3)
    B, nq, D = q.shape
    _need(k_pages, "k pages", torch.bfloat16, 4)
    _need(v_pages, "v pages", torch.bfloat16, 4)
    nkv = k_pages.shape[1]
    if tuple(k_pages.shape[1:]) != (nkv, page, D) or v_pages.shape != k_pages.shape:
        raise KernelError(f"pages are {tuple(k_pages.shape)}, expected [*, nkv, {page}, {D}]")
    for t, nm in ((block_table, "block table"), (slots, "slots"), (kv_len, "kv_len")):
        _need(t, nm, torch.int32)
    if slots.shape[0] != B or kv_len.shape[0] != B:
        raise KernelError("one slot and one length per query row are needed")
    stages = int(stages or DECODE_TMA_STAGES) or (2 if B * nkv < DECODE_TMA_DEEP_PAIRS else 3)
    per_sm = {2: 3, 3: 2, 4: 1}.get(stages, 2) if D == 128 else 3
    ns = int(n_splits) if n_splits else decode_tma_splits(B, nkv, max_kv_len, q.device, per_sm)
    out = torch.empty_like(q)
    a = _DecodeTmaArgs()
    if ns > 1:
        ws = _WORKSPACES.setdefault(q.device.index or 0, _Workspace())
        scratch, _c = ws.get(q.device, B * nq * ns * (D + 2), 1)
        dev = q.device.index or 0
        counters = _ATTN_COUNTERS.get(dev)
        if counters is None or counters.numel() < B * nkv:
            counters = _ATTN_COUNTERS[dev] = torch.zeros(max(B * nkv, 1 << 16), dtype=torch.int32,
                                                         device=q.device)
        a.part_o, a.part_ml = scratch.data_ptr(), scratch[B * nq * ns * D:].data_ptr()
        a.counters = counters.data_ptr()
    a.q, a.block_table, a.slots = q.data_ptr(), block_table.data_ptr(), slots.data_ptr()
    a.kv_len, a.out, a.error = kv_len.data_ptr(), out.data_ptr(), _tc_error_flag(q.device).data_ptr()
    a.n_seqs, a.nq, a.nkv, a.max_pages = B, nq, nkv, block_table.shape[1]
    a.window, a.n_splits, a.scale_log2 = int(window or 0), ns, float(scale) * _LOG2E
    a.stamps = _ptr(DECODE_TMA_STAMPS)
    with torch.cuda.device(q.device):
        _check(_fn("attn_decode_tma", "gb_attn_decode_tma", "pplpiiip")(
            k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0], ctypes.addressof(a), D, page,
            stages, _stream()), "attn_decode_tma")
    return out


# ---------------------------------------------------------------- attention dispatch
def attention(q, k_pages, v_pages, block_table, *, step, page: int, scale: float,
              window: Optional[int] = None) -> torch.Tensor:
    """Attention of the step's queries over their sequences' cached keys.
    32-bit tensors take the plain 32-bit kernel; bfloat16 takes the tensor-core
    kernels where they accept the shape and the plain kernel elsewhere."""
    _T, nq, D = q.shape
    if q.dtype == torch.bfloat16 and fast_attention_takes(D, nq, k_pages.shape[1], page):
        nkv = k_pages.shape[1]
        if step.decode and attn_decode_tma_takes(D, nq, nkv, page) and (
                DECODE_ATTENTION == "tma" or
                (DECODE_ATTENTION == "auto" and step.n_seqs * nkv >= DECODE_TMA_PAIRS)):
            return attn_decode_tma(q, k_pages, v_pages, block_table, slots=step.slots,
                                   kv_len=step.kv_len, page=page, scale=scale,
                                   max_kv_len=step.max_kv_len, window=window)
        if step.decode:
            return attn_decode_bf16(q, k_pages, v_pages, block_table, slots=step.slots,
                                    kv_len=step.kv_len, page=page, scale=scale,
                                    max_kv_len=step.max_kv_len, window=window)
        # the grid comes from the host's copy of the lengths; a captured step has
        # none, and the kernels then take the most blocks its rows can make
        if PREFILL_ATTENTION == "tc" and attn_prefill_tc_takes(D, nq, k_pages.shape[1], page):
            return attn_prefill_tc(q, k_pages, v_pages, block_table, cu_q=step.cu_q,
                                   slots=step.slots, kv_len=step.kv_len, q_lens=step.q_lens,
                                   page=page, scale=scale, window=window)
        return attn_prefill_bf16(q, k_pages, v_pages, block_table, cu_q=step.cu_q,
                                 slots=step.slots, kv_len=step.kv_len, q_lens=step.q_lens,
                                 page=page, scale=scale, window=window)
    return attn_generic(q, k_pages, v_pages, block_table, token_seq=step.token_seq,
                        token_pos=step.token_pos, slots=step.slots, page=page, scale=scale,
                        window=window)


# ---------------------------------------------------------------- sampling
@_profiled("argmax", lambda out, logits: (_nbytes(logits), 0))
def argmax(logits: torch.Tensor) -> torch.Tensor:
    """First maximum of every row of 32-bit logits -> int32 [rows]."""
    _need(logits, "logits", torch.float32, 2)
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    scratch = torch.empty((logits.shape[0], 64), dtype=torch.float32, device=logits.device)
    _check(_fn("sample", "gb_argmax_f32", "piippp")(
        logits.data_ptr(), logits.shape[0], logits.shape[1], out.data_ptr(), scratch.data_ptr(),
        _stream()), "argmax", 2)
    return out


@_profiled("sample", lambda out, logits, *a: (_nbytes(logits), 0))
def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """One token per row from temperature / top-k / top-p sampling with the
    uniform draw ``u[row]``; a temperature <= 1e-5 means argmax."""
    _need(logits, "logits", torch.float32, 2)
    n = logits.shape[0]
    for t, nm, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                      (top_p, "top_p", torch.float32), (u, "u", torch.float32)):
        _need(t, nm, dt, 1)
        if t.shape[0] != n:
            raise KernelError(f"{nm} has {t.shape[0]} entries for {n} rows")
    out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(_fn("sample", "gb_sample_f32", "piipppppp")(
        logits.data_ptr(), n, logits.shape[1], temperature.data_ptr(), top_k.data_ptr(),
        top_p.data_ptr(), u.data_ptr(), out.data_ptr(), _stream()), "sample")
    return out
