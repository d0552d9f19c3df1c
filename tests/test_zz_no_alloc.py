"""The entry point for callers that cannot allocate device memory
(csrc/gemm_skinny_noalloc.h), called through its exported C symbol.

It keeps its split-K scratch in static device arrays inside the library, so it
can be used where no allocator may be called.  The check is against the
library's ordinary entry point for the same product, on two calls in a row,
since all calls share that scratch and the second must not see the first's
leftovers.  The file is named to be collected last."""
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _symbol():
    from grout_b200.kernels.build import module
    fn = module("gemm_skinny_bf16").gb_gemm_skinny_bf16_noalloc
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    fn.restype = c_int
    return fn


def _call(fn, x, w, out_dtype):
    y = torch.full((x.shape[0], w.shape[0]), float("nan"), dtype=out_dtype, device=x.device)
    rc = fn(x.data_ptr(), w.data_ptr(), y.data_ptr(), x.shape[0], w.shape[0], x.shape[1],
            int(out_dtype == torch.float32), torch.cuda.current_stream().cuda_stream)
    return rc, y


@pytest.mark.parametrize("M,N,K", [(8, 2560, 9728), (1, 6144, 2560), (16, 2560, 4096), (5, 200, 264)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_matches_the_allocating_entry_point_twice_in_a_row(M, N, K, out_dtype):
    from grout_b200.kernels import ops
    fn = _symbol()
    g = torch.Generator().manual_seed(1000 + M + N)
    with torch.cuda.device(DEV):
        for call in range(2):
            x = torch.randn((M, K), generator=g).to(torch.bfloat16).to(DEV)
            w = (torch.randn((N, K), generator=g) * 0.05).to(torch.bfloat16).to(DEV)
            want = ops.gemm_skinny_bf16(x, w, out_dtype)
            rc, got = _call(fn, x, w, out_dtype)
            assert rc == 0, (call, rc)
            torch.cuda.synchronize()
            # the same kernel with the same split: the sums are the same sums
            assert torch.equal(got, want), (call, (got.float() - want.float()).abs().max().item())
            ref = x.double().cpu() @ w.double().cpu().T
            tol = 2e-5 * K ** 0.5 + (2.0 ** -7 if out_dtype == torch.bfloat16 else 0.0)
            assert torch.allclose(got.double().cpu(), ref, atol=tol, rtol=2.0 ** -7)


def test_refuses_what_does_not_fit_its_scratch():
    fn = _symbol()
    with torch.cuda.device(DEV):
        x = torch.zeros((64, 9728), dtype=torch.bfloat16, device=DEV)
        w = torch.zeros((2560, 9728), dtype=torch.bfloat16, device=DEV)
        rc, y = _call(fn, x, w, torch.float32)
        assert rc == -3                                   # GB_ERR_TOO_LARGE
        assert bool(torch.isnan(y).all())                 # nothing was launched
        rc, _ = _call(fn, x[:, :100].contiguous(), w[:, :100].contiguous(), torch.float32)
        assert rc == -2                                   # inner size not a multiple of 8
