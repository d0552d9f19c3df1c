"""The tcgen05 matrix product alone against a 64-bit product, in both
orientations, at sizes with ragged edges, and with tiles shared between blocks."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16)


def _check(M, N, K, out_dtype, swap, seed=0):
    from grout_b200.kernels import ops
    x, w = _rand((M, K), 50 + seed), _rand((N, K), 51 + seed, 0.05)
    got = ops.gemm_tc_bf16(x.to(DEV), w.to(DEV), out_dtype, swap=swap)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    want = x.double() @ w.double().T
    e = 2.0 ** -8 if out_dtype == torch.bfloat16 else 0.0
    assert got.shape == (M, N) and got.dtype == out_dtype
    err = (got.double().cpu() - want).abs()
    bound = 2e-5 * math.sqrt(K) + 2 * e + 2 * e * want.abs()
    assert bool((err <= bound).all()), (M, N, K, swap, err.max().item())


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (300, 200, 264), (2048, 512, 2560),
                                   (70, 1000, 96), (513, 130, 4096),
                                   # 160 and 190 tiles on 148 SMs: leftover tiles cut over K
                                   (1280, 4096, 520), (1200, 4800, 1032)])
def test_prefill_orientation(M, N, K, out_dtype):
    _check(M, N, K, out_dtype, swap=False)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 2560, 9728), (16, 6144, 2560), (33, 200, 264),
                                   (64, 2560, 4096), (5, 19456, 2560),
                                   # a few more tiles than SMs, wide tiles: the tiles beyond one
                                   # per block are cut over K and taken first
                                   (64, 19456, 2560), (40, 20000, 520), (100, 21000, 1032)])
def test_decode_orientation(M, N, K, out_dtype):
    _check(M, N, K, out_dtype, swap=True)


def test_twice_in_a_row_and_row_independence():
    """Shared tiles leave their counters at zero; a row's result does not depend
    on the rows beside it when the layout is the same."""
    from grout_b200.kernels import ops
    x, w = _rand((16, 4096), 60).to(DEV), _rand((2560, 4096), 61, 0.05).to(DEV)
    a = ops.gemm_tc_bf16(x, w, torch.float32)
    b = ops.gemm_tc_bf16(x, w, torch.float32)
    one = ops.gemm_tc_bf16(x[9:10].contiguous(), w, torch.float32)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    assert torch.equal(a, b)
    assert torch.equal(a[9:10], one)
    # the same with leftover tiles shared out before every block's own tile
    x, w = _rand((48, 520), 62).to(DEV), _rand((20000, 520), 63, 0.05).to(DEV)
    a = ops.gemm_tc_bf16(x, w, torch.float32, swap=True)
    b = ops.gemm_tc_bf16(x, w, torch.float32, swap=True)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    assert torch.equal(a, b)


@pytest.mark.parametrize("M", [1, 8, 17, 33, 40, 64])
@pytest.mark.parametrize("I,K", [(152, 96), (9728, 2560), (24, 4096), (1000, 264),
                                 # 400 tiles: several whole tiles per block at 32 and 64 columns
                                 (25600, 512)])
def test_silu_epilogue(M, I, K):
    """Gate and up rows interleaved in groups of 8; the kernel returns silu(gate) * up."""
    from grout_b200.kernels import ops
    x = _rand((M, K), 70)
    gate, up = _rand((I, K), 71, 0.05), _rand((I, K), 72, 0.05)
    w = torch.stack([gate.view(-1, 8, K), up.view(-1, 8, K)], 1).reshape(2 * I, K).contiguous()
    got = ops.gemm_tc_bf16(x.to(DEV), w.to(DEV), torch.bfloat16, swap=True, silu_mul=True).cpu()
    ops.check_kernel_errors()
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    want = g / (1 + torch.exp(-g)) * u
    assert got.shape == (M, I)
    assert torch.allclose(got.double(), want, atol=2e-4, rtol=3 * 2.0 ** -8)


@pytest.mark.parametrize("M,N,K", [(8, 2560, 4096), (1, 6144, 2560), (64, 2560, 9728), (16, 128, 512)])
def test_split_out_partials_sum_to_the_product(M, N, K):
    """With few tiles the product may leave its split-K reduction to its consumer."""
    from grout_b200.kernels import ops
    x, w = _rand((M, K), 80), _rand((N, K), 81, 0.05)
    got = ops.gemm_tc_bf16(x.to(DEV), w.to(DEV), torch.bfloat16, swap=True, split_out=True)
    ops.check_kernel_errors()
    assert got.dtype == torch.float32 and got.dim() == 3 and got.shape[1:] == (M, N)
    assert got.shape[0] >= 2
    want = x.double() @ w.double().T
    assert torch.allclose(got.double().sum(0).cpu(), want, atol=2e-5 * math.sqrt(K), rtol=1e-5)
    # a product with many tiles keeps its own reduction
    big = ops.gemm_tc_bf16(x.to(DEV)[:, :256].contiguous(), _rand((19456, 256), 82, 0.05).to(DEV),
                           torch.bfloat16, swap=True, split_out=True)
    assert big.dim() == 2


# ---- the product on pairs of SMs (tcgen05.mma.cta_group::2)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K,cols", [(256, 256, 64, 0), (128, 256, 512, 256), (300, 200, 264, 48),
                                        (2048, 512, 2560, 0), (70, 1000, 96, 144), (513, 136, 4096, 0),
                                        (1, 8, 8, 0), (2100, 2560, 2560, 0), (600, 1000, 520, 240)])
def test_pair_product(M, N, K, cols, out_dtype):
    from grout_b200.kernels import ops
    x, w = _rand((M, K), 60), _rand((N, K), 61, 0.05)
    got = ops.gemm_tc2_bf16(x.to(DEV), w.to(DEV), out_dtype, tile_cols=cols)
    again = ops.gemm_tc2_bf16(x.to(DEV), w.to(DEV), out_dtype, tile_cols=cols)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    want = x.double() @ w.double().T
    e = 2.0 ** -8 if out_dtype == torch.bfloat16 else 0.0
    assert got.shape == (M, N) and got.dtype == out_dtype
    err = (got.double().cpu() - want).abs()
    bound = 2e-5 * math.sqrt(K) + 2 * e + 2 * e * want.abs()
    assert bool((err <= bound).all()), (M, N, K, err.max().item())
    assert torch.equal(got, again)


@pytest.mark.parametrize("M", [65, 300, 2048])
@pytest.mark.parametrize("I,K", [(152, 96), (9728, 2560), (24, 4096)])
def test_pair_product_silu_epilogue(M, I, K):
    from grout_b200.kernels import ops
    x = _rand((M, K), 62)
    g, u = _rand((I, K), 63, 0.05), _rand((I, K), 64, 0.05)
    fused = torch.stack([g.view(-1, 8, K), u.view(-1, 8, K)], dim=1).reshape(2 * I, K)
    got = ops.gemm_tc2_bf16(x.to(DEV), fused.to(DEV), torch.bfloat16, silu_mul=True)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    gd, ud = x.double() @ g.double().T, x.double() @ u.double().T
    want = gd / (1 + torch.exp(-gd)) * ud
    assert got.shape == (M, I)
    err = (got.double().cpu() - want).abs()
    bound = 8e-5 * math.sqrt(K) + 2.0 ** -7 * want.abs() + 1e-3
    assert bool((err <= bound).all()), (M, I, K, err.max().item())


def test_pair_product_refuses_what_it_cannot_store():
    from grout_b200.kernels import ops
    x, w = _rand((4, 64), 65), _rand((12, 64), 66)           # 12 bf16 columns: 24 bytes a row
    with pytest.raises(ops.KernelError):
        ops.gemm_tc2_bf16(x.to(DEV), w.to(DEV))
