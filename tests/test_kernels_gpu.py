"""Each kernel alone against a plain 64-bit computation of the same operation,
at sizes other than the tiny models' (odd widths, head sizes in steps of 16,
many groups, scattered pages)."""
import math

import pytest
import torch

from plain import qwen3 as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _ops():
    from grout_b200.kernels import ops
    return ops


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def _eps(dtype):
    return 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -22


@pytest.mark.parametrize("dtype", list(DT))
def test_embed(dtype):
    dt = DT[dtype]
    table = _rand((1000, 72), dt, 1)
    ids = torch.tensor([0, 999, 5, 5, 317], dtype=torch.int32)
    got = _ops().embed(table.to(DEV), ids.to(DEV)).cpu()
    assert torch.equal(got, table[ids.long()])
    # a width that is no multiple of 16 bytes takes the scalar path
    table = _rand((50, 7), dt, 2)
    got = _ops().embed(table.to(DEV), ids[:3].clamp(max=49).to(DEV)).cpu()
    assert torch.equal(got, table[ids[:3].clamp(max=49).long()])


@pytest.mark.parametrize("w32", [False, True])
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("N", [200, 2560, 5000])
def test_add_rmsnorm(dtype, N, w32):
    dt = DT[dtype]
    if dtype == "float32" and not w32:
        pytest.skip("32-bit activations take 32-bit weights")
    rows = 9
    res = _rand((rows, N), torch.float32, 3)
    delta = _rand((rows, N), dt, 4)
    w = (1 + 0.1 * _rand((N,), torch.float32, 5)).to(torch.float32 if w32 else dt)
    eps = 1e-5
    want_res = res.double() + delta.double()
    want_y = plain.rms_norm(want_res, w, eps)
    r = res.clone().to(DEV)
    res_out, y = _ops().add_rmsnorm(r, delta.to(DEV), w.to(DEV), eps, dtype=dt)
    assert res_out.data_ptr() == r.data_ptr()
    assert torch.allclose(res_out.cpu().double(), want_res, atol=1e-6, rtol=1e-6)
    assert torch.allclose(y.cpu().double(), want_y, atol=4 * _eps(dt), rtol=2 * _eps(dt))
    # gathered rows, first-layer form (no residual yet) and plain norm
    idx = torch.tensor([8, 0, 3], dtype=torch.int32)
    res2, y2 = _ops().add_rmsnorm(res.to(DEV), delta.to(DEV), w.to(DEV), eps, dtype=dt,
                                  rows=idx.to(DEV))
    assert torch.allclose(res2.cpu().double(), want_res[idx.long()], atol=1e-6, rtol=1e-6)
    assert torch.allclose(y2.cpu().double(), want_y[idx.long()], atol=4 * _eps(dt), rtol=2 * _eps(dt))
    res3, y3 = _ops().add_rmsnorm(None, delta.to(DEV), w.to(DEV), eps, dtype=dt)
    assert torch.equal(res3.cpu(), delta.float())
    assert torch.allclose(y3.cpu().double(), plain.rms_norm(delta.double(), w, eps),
                          atol=4 * _eps(dt), rtol=2 * _eps(dt))


class Paged:
    """Sequences laid out in scattered pages, with the dense copies for the oracle."""

    def __init__(self, lens, nkv, D, dtype, seed, page=64, spare=5, fill=float("nan")):
        g = torch.Generator().manual_seed(seed)
        self.page, self.nkv, self.D = page, nkv, D
        n_need = sum((n + page - 1) // page for n in lens)
        n_pages = n_need + spare
        perm = torch.randperm(n_pages, generator=g).tolist()
        self.max_pages = max((n + page - 1) // page for n in lens) + 1
        # slots are scattered too: sequence i lives in slot slot_of[i]
        self.n_slots = len(lens) + 2
        self.slot_of = torch.randperm(self.n_slots, generator=g).tolist()[:len(lens)]
        self.table = torch.zeros((self.n_slots, self.max_pages), dtype=torch.int32)
        self.k_pages = torch.full((n_pages, nkv, page, D), fill).to(dtype)
        self.v_pages = torch.full((n_pages, nkv, page, D), fill).to(dtype)
        self.k, self.v = [], []
        for i, n in enumerate(lens):
            k = (torch.randn((n, nkv, D), generator=g)).to(dtype)
            v = (torch.randn((n, nkv, D), generator=g)).to(dtype)
            self.k.append(k)
            self.v.append(v)
            for p in range((n + page - 1) // page):
                pg = perm.pop()
                self.table[self.slot_of[i], p] = pg
                m = min(page, n - p * page)
                self.k_pages[pg, :, :m] = k[p * page:p * page + m].transpose(0, 1)
                self.v_pages[pg, :, :m] = v[p * page:p * page + m].transpose(0, 1)

    def store(self, i, pos, k_row, v_row):
        pg = int(self.table[self.slot_of[i], pos // self.page])
        self.k_pages[pg, :, pos % self.page] = k_row
        self.v_pages[pg, :, pos % self.page] = v_row


def _attn_oracle(q, k, v, pos, scale, window):
    """q [nq, D] at absolute position pos over keys k, v [n, nkv, D]."""
    nq, D = q.shape
    nkv = k.shape[1]
    out = torch.empty(nq, D, dtype=torch.float64)
    lo = 0 if window is None else max(0, pos - window + 1)
    for h in range(nq):
        kh, vh = k[lo:pos + 1, h // (nq // nkv)].double(), v[lo:pos + 1, h // (nq // nkv)].double()
        s = (kh @ q[h].double()) * scale
        p = torch.softmax(s, 0)
        out[h] = p @ vh
    return out


@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("nq,nkv,D", [(6, 2, 48), (8, 1, 128), (3, 3, 16)])
def test_attn_generic(dtype, nq, nkv, D, window):
    dt = DT[dtype]
    lens = [1, 130, 200, 64]
    pc = Paged(lens, nkv, D, dt, 7)
    # queries: every sequence's last position, plus inner positions of sequence 2
    places = [(0, 0), (1, 129), (2, 199), (3, 63), (2, 0), (2, 63), (2, 64), (2, 127), (2, 128)]
    q = _rand((len(places), nq, D), dt, 8)
    scale = 1.0 / math.sqrt(D)
    # the far key among hundreds: scale one query and one early key so that its
    # score stands out; the output must then be that key's value
    far_q, far_seq, far_key = 2, 2, 3
    if window is None:
        q[far_q] = 0
        q[far_q, :, 0] = 30.0
        pc.k[far_seq][:, :, 0] = 0
        pc.k[far_seq][far_key, :, 0] = 30.0
        pc.store(far_seq, far_key, pc.k[far_seq][far_key], pc.v[far_seq][far_key])
        for j in range(lens[far_seq]):
            pc.store(far_seq, j, pc.k[far_seq][j], pc.v[far_seq][j])
    slots = torch.tensor(pc.slot_of, dtype=torch.int32)
    token_seq = torch.tensor([s for s, _ in places], dtype=torch.int32)
    token_pos = torch.tensor([p for _, p in places], dtype=torch.int32)
    got = _ops().attn_generic(q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV),
                              token_seq=token_seq.to(DEV), token_pos=token_pos.to(DEV),
                              slots=slots.to(DEV), page=64, scale=scale, window=window).cpu()
    for r, (s, p) in enumerate(places):
        want = _attn_oracle(q[r], pc.k[s], pc.v[s], p, scale, window)
        assert torch.allclose(got[r].double(), want, atol=6 * _eps(dt), rtol=4 * _eps(dt)), (r, s, p)
    if window is None:
        h = 0
        want = pc.v[far_seq][far_key, 0].double()
        assert torch.allclose(got[far_q, h].double(), want, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("nq,nkv,D,rot", [(6, 2, 48, 48), (4, 4, 64, 32), (8, 1, 128, 128),
                                          (3, 3, 64, 64), (2, 1, 256, 256), (4, 2, 128, 64)])
def test_qk_prepare(dtype, nq, nkv, D, rot):
    dt = DT[dtype]
    theta, eps = 50000.0, 1e-5
    lens = [3, 70]
    pc = Paged(lens, nkv, D, dt, 11)
    # tokens: the last two of sequence 0 and three of sequence 1 across a page edge
    places = [(0, 1), (0, 2), (1, 63), (1, 64), (1, 69)]
    T = len(places)
    qkv = _rand((T, (nq + 2 * nkv) * D), dt, 12)
    q_w = (1 + 0.1 * _rand((D,), torch.float32, 13)).to(dt)
    k_w = (1 + 0.1 * _rand((D,), torch.float32, 14)).to(dt)
    inv = torch.from_numpy(plain.rope_inv_freq(rot, theta))
    pos = [p for _, p in places]
    x = qkv.double().view(T, nq + 2 * nkv, D)
    qn = plain.rms_norm(x[:, :nq], q_w, eps)
    kn = plain.rms_norm(x[:, nq:nq + nkv], k_w, eps)
    cos, sin = plain.rope_cos_sin(pos, rot, theta)
    want_q = torch.cat([plain.apply_rope(qn[..., :rot], cos, sin), qn[..., rot:]], -1)
    want_k = torch.cat([plain.apply_rope(kn[..., :rot], cos, sin), kn[..., rot:]], -1)
    want_v = x[:, nq + nkv:]
    kp, vp = pc.k_pages.to(DEV), pc.v_pages.to(DEV)
    before_k = kp.clone()
    q, kv = _ops().qk_prepare(
        qkv.to(DEV), nq, nkv, D, q_w=q_w.to(DEV), k_w=k_w.to(DEV), eps=eps, inv_freq=inv.to(DEV),
        rot_dim=rot, token_seq=torch.tensor([s for s, _ in places], dtype=torch.int32, device=DEV),
        token_pos=torch.tensor(pos, dtype=torch.int32, device=DEV),
        slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV),
        block_table=pc.table.to(DEV), k_pages=kp, v_pages=vp, page=64, want_kv_out=True)
    tol = dict(atol=6 * _eps(dt), rtol=4 * _eps(dt))
    assert torch.allclose(q.cpu().double(), want_q, **tol)
    assert torch.allclose(kv.cpu().double()[:, :nkv], want_k, **tol)
    assert torch.equal(kv.cpu()[:, nkv:], qkv.view(T, -1, D)[:, nq + nkv:])
    touched = torch.zeros(kp.shape[0], kp.shape[2], dtype=torch.bool)
    for r, (s, p) in enumerate(places):
        pg = int(pc.table[pc.slot_of[s], p // 64])
        touched[pg, p % 64] = True
        assert torch.allclose(kp[pg, :, p % 64].cpu().double(), want_k[r], **tol)
        assert torch.allclose(vp[pg, :, p % 64].cpu().double(), want_v[r], **tol)
    # nothing else in the cache was written
    same = (kp.cpu().view(torch.int16 if dt == torch.bfloat16 else torch.int32) ==
            before_k.cpu().view(torch.int16 if dt == torch.bfloat16 else torch.int32)).all(-1).all(1)
    assert bool(same[~touched].all())


@pytest.mark.parametrize("w32", [False, True])
@pytest.mark.parametrize("nq,nkv,D", [(6, 2, 64), (5, 1, 128), (3, 3, 256), (7, 2, 48)])
def test_qk_prepare_of_a_prompt(nq, nkv, D, w32):
    """Many tokens at once (the path of a prompt, which takes 16 bytes a lane where
    the sizes allow): 150 tokens of one sequence from position 37 on, over page edges."""
    dt = torch.bfloat16
    theta, eps = 10000.0, 1e-6
    start, T = 37, 150
    pc = Paged([start + T], nkv, D, dt, 18)
    qkv = _rand((T, (nq + 2 * nkv) * D), dt, 19)
    wdt = torch.float32 if w32 else dt
    q_w = (1 + 0.1 * _rand((D,), torch.float32, 20)).to(wdt)
    k_w = (1 + 0.1 * _rand((D,), torch.float32, 21)).to(wdt)
    inv = torch.from_numpy(plain.rope_inv_freq(D, theta))
    pos = list(range(start, start + T))
    x = qkv.double().view(T, nq + 2 * nkv, D)
    cos, sin = plain.rope_cos_sin(pos, D, theta)
    want_q = plain.apply_rope(plain.rms_norm(x[:, :nq], q_w, eps), cos, sin)
    want_k = plain.apply_rope(plain.rms_norm(x[:, nq:nq + nkv], k_w, eps), cos, sin)
    kp, vp = pc.k_pages.to(DEV), pc.v_pages.to(DEV)
    q, kv = _ops().qk_prepare(
        qkv.to(DEV), nq, nkv, D, q_w=q_w.to(DEV), k_w=k_w.to(DEV), eps=eps, inv_freq=inv.to(DEV),
        rot_dim=D, token_seq=torch.zeros(T, dtype=torch.int32, device=DEV),
        token_pos=torch.tensor(pos, dtype=torch.int32, device=DEV),
        slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV),
        block_table=pc.table.to(DEV), k_pages=kp, v_pages=vp, page=64, want_kv_out=True)
    tol = dict(atol=6 * _eps(dt), rtol=4 * _eps(dt))
    assert torch.allclose(q.cpu().double(), want_q, **tol)
    assert torch.allclose(kv.cpu().double()[:, :nkv], want_k, **tol)
    assert torch.equal(kv.cpu()[:, nkv:], qkv.view(T, -1, D)[:, nq + nkv:])
    for r in (0, 26, 27, 90, 91, T - 1):                      # 37 + 27 = 64: the first page edge
        p = pos[r]
        pg = int(pc.table[pc.slot_of[0], p // 64])
        assert torch.allclose(kp[pg, :, p % 64].cpu().double(), want_k[r], **tol)
        assert torch.equal(vp[pg, :, p % 64].cpu(), qkv.view(T, -1, D)[r, nq + nkv:])


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("D", [48, 64])
def test_qk_prepare_without_norm_and_rotation_copies(dtype, D):
    """No norm weights and no rotation (an attention without q/k norm whose
    position encoding is applied elsewhere): heads pass through unchanged, keys
    and values come back dense and nothing is stored when no pages are given."""
    dt = DT[dtype]
    nq, nkv, T = 5, 1, 7
    qkv = _rand((T, (nq + 2 * nkv) * D), dt, 17)
    z = torch.zeros(T, dtype=torch.int32, device=DEV)
    q, kv = _ops().qk_prepare(qkv.to(DEV), nq, nkv, D, token_seq=z, token_pos=z,
                              slots=torch.zeros(1, dtype=torch.int32, device=DEV), want_kv_out=True)
    x = qkv.view(T, nq + 2 * nkv, D)
    assert torch.equal(q.cpu(), x[:, :nq]) and torch.equal(kv.cpu(), x[:, nq:])


def test_qk_prepare_skips_padding_rows():
    nq, nkv, D = 4, 2, 32
    pc = Paged([5], nkv, D, torch.bfloat16, 15)
    kp, vp = pc.k_pages.to(DEV), pc.v_pages.to(DEV)
    before = kp.clone().view(torch.int16)
    qkv = _rand((1, (nq + 2 * nkv) * D), torch.bfloat16, 16).to(DEV)
    _ops().qk_prepare(qkv, nq, nkv, D, token_seq=torch.zeros(1, dtype=torch.int32, device=DEV),
                      token_pos=torch.zeros(1, dtype=torch.int32, device=DEV),
                      slots=torch.tensor([-1], dtype=torch.int32, device=DEV),
                      block_table=pc.table.to(DEV), k_pages=kp, v_pages=vp, page=64)
    assert torch.equal(kp.view(torch.int16), before)


@pytest.mark.parametrize("M,N,K", [(1, 130, 100), (70, 65, 17), (129, 200, 333)])
def test_gemm_f32(M, N, K):
    a, w = _rand((M, K), torch.float32, 20), _rand((N, K), torch.float32, 21)
    got = _ops().gemm_f32(a.to(DEV), w.to(DEV)).cpu()
    want = a.double() @ w.double().T
    assert torch.allclose(got.double(), want, atol=1e-5 * math.sqrt(K), rtol=1e-5)


def test_gemm_f32_row_independent():
    """A row's result does not depend on the rows beside it (bitwise)."""
    a, w = _rand((70, 96), torch.float32, 22), _rand((50, 96), torch.float32, 23)
    full = _ops().gemm_f32(a.to(DEV), w.to(DEV)).cpu()
    one = _ops().gemm_f32(a[33:34].contiguous().to(DEV), w.to(DEV)).cpu()
    assert torch.equal(full[33:34], one)


@pytest.mark.parametrize("out", ["bfloat16", "float32"])
@pytest.mark.parametrize("M", [1, 5, 8, 13, 16, 27, 33, 64])
@pytest.mark.parametrize("N,K", [(200, 264), (77, 2560), (2560, 96)])
def test_gemm_skinny_bf16(M, N, K, out):
    x, w = _rand((M, K), torch.bfloat16, 24), _rand((N, K), torch.bfloat16, 25, 0.05)
    got = _ops().gemm_skinny_bf16(x.to(DEV), w.to(DEV), DT[out]).cpu()
    want = x.double() @ w.double().T
    e = _eps(DT[out])
    assert torch.allclose(got.double(), want, atol=2e-5 * math.sqrt(K) + 2 * e, rtol=2 * e)


@pytest.mark.parametrize("M,N,K", [(8, 2560, 9728), (3, 160, 4096), (40, 2560, 4096), (16, 6144, 2560)])
def test_gemm_skinny_split_k(M, N, K):
    """Shapes whose tiles are shared by several blocks (partials in scratch, the
    block that arrives last sums them); called twice, since the arrival counters
    must be left at zero."""
    ops = _ops()
    blocks, n_floats, n_counters = ops.skinny_plan(M, N, K, True, False)
    rows = 16 if M <= 16 else 32
    assert blocks > (N + rows - 1) // rows and n_floats > 0
    x, w = _rand((M, K), torch.bfloat16, 32), _rand((N, K), torch.bfloat16, 33, 0.05)
    want = x.double() @ w.double().T
    first = ops.gemm_skinny_bf16(x.to(DEV), w.to(DEV), torch.float32).cpu()
    second = ops.gemm_skinny_bf16(x.to(DEV), w.to(DEV), torch.float32).cpu()
    assert torch.equal(first, second)
    assert torch.allclose(first.double(), want, atol=2e-5 * math.sqrt(K), rtol=1e-5)


@pytest.mark.parametrize("M", [1, 8, 11, 33, 64])
@pytest.mark.parametrize("I,K", [(152, 96), (9728, 2560), (24, 4096)])
def test_gemm_skinny_silu_epilogue(M, I, K):
    """Gate and up rows interleaved in groups of 8; the kernel returns silu(gate) * up."""
    x = _rand((M, K), torch.bfloat16, 34)
    gate, up = _rand((I, K), torch.bfloat16, 35, 0.05), _rand((I, K), torch.bfloat16, 36, 0.05)
    w = torch.stack([gate.view(-1, 8, K), up.view(-1, 8, K)], 1).reshape(2 * I, K).contiguous()
    got = _ops().gemm_skinny_bf16(x.to(DEV), w.to(DEV), torch.bfloat16, silu_mul=True).cpu()
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    want = g / (1 + torch.exp(-g)) * u
    assert got.shape == (M, I)
    assert torch.allclose(got.double(), want, atol=2e-4 + 2 * _eps(torch.bfloat16) * 0,
                          rtol=3 * _eps(torch.bfloat16))
    # the stand-alone kernel on the same interleaved layout agrees
    raw = _ops().gemm_skinny_bf16(x.to(DEV), w.to(DEV), torch.float32)
    two = _ops().silu_mul(raw, 8).cpu()
    # 32-bit sums over K, then the product of two such values
    assert torch.allclose(two.double(), want, atol=8e-5 * math.sqrt(K), rtol=1e-5)


def test_gemm_skinny_row_independent():
    x, w = _rand((16, 512), torch.bfloat16, 26), _rand((300, 512), torch.bfloat16, 27)
    full = _ops().gemm_skinny_bf16(x.to(DEV), w.to(DEV), torch.float32).cpu()
    one = _ops().gemm_skinny_bf16(x[9:10].contiguous().to(DEV), w.to(DEV), torch.float32).cpu()
    assert torch.equal(full[9:10], one)


def test_gemm_skinny_refuses():
    ops = _ops()
    x, w = _rand((2, 100), torch.bfloat16, 28).to(DEV), _rand((8, 100), torch.bfloat16, 29).to(DEV)
    with pytest.raises(ops.KernelError):
        ops.gemm_skinny_bf16(x, w)            # inner size not a multiple of 8
    with pytest.raises(ops.KernelError):
        ops.gemm_skinny_bf16(torch.zeros((65, 96), dtype=torch.bfloat16, device=DEV),
                             torch.zeros((8, 96), dtype=torch.bfloat16, device=DEV))
    with pytest.raises(ops.KernelError):
        ops.gemm_skinny_bf16(x.cpu(), w.cpu())   # no CPU path


@pytest.mark.parametrize("dtype", list(DT))
def test_silu_mul_and_cast(dtype):
    dt = DT[dtype]
    gu = _rand((7, 2 * 301), dt, 30, 3.0)
    got = _ops().silu_mul(gu.to(DEV)).cpu()
    g, u = gu.double()[:, :301], gu.double()[:, 301:]
    want = g / (1 + torch.exp(-g)) * u
    assert torch.allclose(got.double(), want, atol=2 * _eps(dt), rtol=2 * _eps(dt))
    # widths in whole runs of 8 take the 16-byte path (bf16), plain and interleaved
    for I, group in ((304, 0), (304, 8), (9728, 8)):
        gu = _rand((5, 2 * I), dt, 32 + I + group, 3.0)
        got = _ops().silu_mul(gu.to(DEV), group).cpu()
        if group:
            v = gu.double().view(5, -1, 2, group)
            g, u = v[:, :, 0].reshape(5, I), v[:, :, 1].reshape(5, I)
        else:
            g, u = gu.double()[:, :I], gu.double()[:, I:]
        want = g / (1 + torch.exp(-g)) * u
        assert torch.allclose(got.double(), want, atol=2 * _eps(dt), rtol=2 * _eps(dt)), (I, group)
    x = _rand((1000,), torch.float32, 31)
    assert torch.equal(_ops().cast(x.to(DEV), torch.bfloat16).cpu(), x.to(torch.bfloat16))
    assert torch.equal(_ops().cast(x.to(torch.bfloat16).to(DEV), torch.float32).cpu(),
                       x.to(torch.bfloat16).float())


# ------------------------------------------------------------------ tensor-core attention
FAST_TOL = dict(atol=6e-3, rtol=1e-2)   # probabilities and outputs are rounded to bf16


@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("nq,nkv,D", [(6, 2, 48), (8, 1, 128), (3, 3, 16), (16, 4, 64)])
def test_attn_prefill_bf16(nq, nkv, D, window):
    dt = torch.bfloat16
    # (tokens already held, tokens of this step): fresh prompts and continued ones
    plan = [(0, 1), (0, 130), (37, 100), (64, 64), (0, 200), (5, 63)]
    lens = [s + n for s, n in plan]
    pc = Paged(lens, nkv, D, dt, 40)
    q_lens = [n for _, n in plan]
    T = sum(q_lens)
    q = _rand((T, nq, D), dt, 41)
    scale = 1.0 / math.sqrt(D)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    if window is None:
        # the far key: the last row of the 200-token prompt looks at key 3 only
        seq, key, row = 4, 3, cu[4] + 199
        q[row] = 0
        q[row, :, 0] = 30.0
        pc.k[seq][:, :, 0] = 0
        pc.k[seq][key, :, 0] = 30.0
        for j in range(lens[seq]):
            pc.store(seq, j, pc.k[seq][j], pc.v[seq][j])
    got = _ops().attn_prefill_bf16(
        q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV),
        cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
        slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV),
        kv_len=torch.tensor(lens, dtype=torch.int32, device=DEV), q_lens=tuple(q_lens), page=64,
        scale=scale, window=window).cpu()
    assert not torch.isnan(got.float()).any()
    for s, (start, n) in enumerate(plan):
        for i in ([0, n // 2, n - 1] if n > 2 else range(n)):
            want = _attn_oracle(q[cu[s] + i], pc.k[s], pc.v[s], start + i, scale, window)
            assert torch.allclose(got[cu[s] + i].double(), want, **FAST_TOL), (s, i)
    # every row of one long sequence
    s, (start, n) = 2, plan[2]
    for i in range(n):
        want = _attn_oracle(q[cu[s] + i], pc.k[s], pc.v[s], start + i, scale, window)
        assert torch.allclose(got[cu[s] + i].double(), want, **FAST_TOL), (s, i)
    if window is None:
        assert torch.allclose(got[cu[4] + 199, 0].double(), pc.v[4][3, 0].double(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("n_splits", [1, 3, 11, None])     # 11: more partials than the merge requests at once
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("nq,nkv,D", [(6, 2, 48), (8, 1, 128), (3, 3, 16), (32, 8, 128), (16, 1, 32)])
def test_attn_decode_bf16(nq, nkv, D, window, n_splits):
    dt = torch.bfloat16
    lens = [1, 130, 200, 64, 33, 65]
    pc = Paged(lens, nkv, D, dt, 42)
    B = len(lens) + 1                               # one padding row at the end
    q = _rand((B, nq, D), dt, 43)
    scale = 1.0 / math.sqrt(D)
    if window is None:
        q[2] = 0
        q[2, :, 0] = 30.0
        pc.k[2][:, :, 0] = 0
        pc.k[2][5, :, 0] = 30.0
        for j in range(lens[2]):
            pc.store(2, j, pc.k[2][j], pc.v[2][j])
    got = _ops().attn_decode_bf16(
        q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV),
        slots=torch.tensor(pc.slot_of + [-1], dtype=torch.int32, device=DEV),
        kv_len=torch.tensor(lens + [7], dtype=torch.int32, device=DEV), page=64, scale=scale,
        max_kv_len=256, window=window, n_splits=n_splits).cpu()
    assert not torch.isnan(got.float()).any()
    for s, n in enumerate(lens):
        want = _attn_oracle(q[s], pc.k[s], pc.v[s], n - 1, scale, window)
        assert torch.allclose(got[s].double(), want, **FAST_TOL), (s, n)
    assert bool((got[B - 1] == 0).all())            # the padding row
    if window is None:
        assert torch.allclose(got[2, 0].double(), pc.v[2][5, 0].double(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("stages", [2, 3, 4])
@pytest.mark.parametrize("n_splits", [1, 3, 11, None])     # 11: more partials than the merge requests at once
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("nq,nkv,D", [(8, 1, 128), (32, 8, 128), (6, 2, 64), (16, 1, 64)])
def test_attn_decode_tma(nq, nkv, D, window, n_splits, stages):
    """The decode attention whose tiles come by TMA and whose splits are combined by the
    block that finishes last.  Rows of a page beyond a sequence's length hold NaN here:
    the kernel masks them as keys and zeroes them as values.  Two launches in a row:
    the second finds the arrival counters as the first left them (zero)."""
    ops = _ops()
    dt = torch.bfloat16
    lens = [1, 130, 200, 64, 33, 65, 128, 129]
    pc = Paged(lens, nkv, D, dt, 42)
    B = len(lens) + 1                               # one padding row at the end
    q = _rand((B, nq, D), dt, 43)
    scale = 1.0 / math.sqrt(D)
    if window is None:
        q[2] = 0
        q[2, :, 0] = 30.0
        pc.k[2][:, :, 0] = 0
        pc.k[2][5, :, 0] = 30.0
        for j in range(lens[2]):
            pc.store(2, j, pc.k[2][j], pc.v[2][j])
    args = (q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV))
    kw = dict(slots=torch.tensor(pc.slot_of + [-1], dtype=torch.int32, device=DEV),
              kv_len=torch.tensor(lens + [7], dtype=torch.int32, device=DEV), page=64, scale=scale,
              max_kv_len=256, window=window, n_splits=n_splits, stages=stages)
    first = ops.attn_decode_tma(*args, **kw).cpu()
    got = ops.attn_decode_tma(*args, **kw).cpu()
    ops.check_kernel_errors()
    assert torch.equal(first, got)
    assert not torch.isnan(got.float()).any()
    for s, n in enumerate(lens):
        want = _attn_oracle(q[s], pc.k[s], pc.v[s], n - 1, scale, window)
        assert torch.allclose(got[s].double(), want, **FAST_TOL), (s, n)
    assert bool((got[B - 1] == 0).all())            # the padding row
    if window is None:
        assert torch.allclose(got[2, 0].double(), pc.v[2][5, 0].double(), atol=1e-2, rtol=1e-2)
    # the kernel without TMA gives the same within rounding
    other = ops.attn_decode_bf16(*args, **{k: v for k, v in kw.items() if k != "stages"}).cpu()
    assert torch.allclose(got.float(), other.float(), **FAST_TOL)


@pytest.mark.parametrize("n_splits", [1, 2, 5, None])
def test_attn_decode_tma_long_sequences(n_splits):
    """Long sequences, so that the ring of stages goes round many times; one query looks
    at a single far key, whose value must come back."""
    ops = _ops()
    dt = torch.bfloat16
    nq, nkv, D = 8, 2, 128
    lens = [1500, 700, 33, 2049]
    pc = Paged(lens, nkv, D, dt, 48)
    q = _rand((len(lens), nq, D), dt, 49)
    scale = 1.0 / math.sqrt(D)
    q[0] = 0
    q[0, :, 0] = 30.0
    pc.k[0][:, :, 0] = 0
    pc.k[0][777, :, 0] = 30.0
    for j in range(lens[0]):
        pc.store(0, j, pc.k[0][j], pc.v[0][j])
    got = ops.attn_decode_tma(
        q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV),
        slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV),
        kv_len=torch.tensor(lens, dtype=torch.int32, device=DEV), page=64, scale=scale,
        max_kv_len=2112, n_splits=n_splits).cpu()
    ops.check_kernel_errors()
    for s, n in enumerate(lens):
        want = _attn_oracle(q[s], pc.k[s], pc.v[s], n - 1, scale, None)
        assert torch.allclose(got[s].double(), want, **FAST_TOL), (s, n)
    assert torch.allclose(got[0, 0].double(), pc.v[0][777, 0].double(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("n_splits", [1, 2, 5])
def test_attn_decode_many_tiles_per_warp(n_splits):
    """Long sequences, so that each warp refills its key and value buffers many times (its
    copies of keys and of values are committed and waited for separately).  One query looks
    at a single far key, whose value must come back."""
    dt = torch.bfloat16
    nq, nkv, D = 8, 2, 128
    lens = [1500, 700, 33]
    pc = Paged(lens, nkv, D, dt, 48)
    q = _rand((len(lens), nq, D), dt, 49)
    scale = 1.0 / math.sqrt(D)
    q[0] = 0
    q[0, :, 0] = 30.0
    pc.k[0][:, :, 0] = 0
    pc.k[0][777, :, 0] = 30.0
    for j in range(lens[0]):
        pc.store(0, j, pc.k[0][j], pc.v[0][j])
    got = _ops().attn_decode_bf16(
        q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV),
        slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV),
        kv_len=torch.tensor(lens, dtype=torch.int32, device=DEV), page=64, scale=scale,
        max_kv_len=1536, n_splits=n_splits).cpu()
    for s, n in enumerate(lens):
        want = _attn_oracle(q[s], pc.k[s], pc.v[s], n - 1, scale, None)
        assert torch.allclose(got[s].double(), want, **FAST_TOL), (s, n)
    assert torch.allclose(got[0, 0].double(), pc.v[0][777, 0].double(), atol=1e-2, rtol=1e-2)


def test_fast_attention_refuses_what_it_cannot_do():
    ops = _ops()
    assert ops.fast_attention_takes(128, 32, 8, 64)
    assert not ops.fast_attention_takes(40, 4, 2, 64)       # head size not in steps of 16
    assert not ops.fast_attention_takes(256, 4, 2, 64)
    assert not ops.fast_attention_takes(64, 34, 2, 64)      # 17 heads per group
    pc = Paged([5], 2, 40, torch.bfloat16, 44)
    q = _rand((1, 4, 40), torch.bfloat16, 45).to(DEV)
    with pytest.raises(ops.KernelError):
        ops.attn_decode_bf16(q, pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV),
                             slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV),
                             kv_len=torch.tensor([5], dtype=torch.int32, device=DEV), page=64,
                             scale=1.0, max_kv_len=64)


@pytest.mark.parametrize("rows_per_block", [128, 256])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("nq,nkv,D", [(8, 1, 128), (6, 2, 64), (16, 4, 128)])
def test_attn_prefill_tc(nq, nkv, D, window, rows_per_block):
    """Both products on the tcgen05 tensor cores.  Rows beyond a sequence's length
    hold large finite values here (the cache zero-fills; NaN there is excluded by
    the kernel's contract)."""
    ops = _ops()
    dt = torch.bfloat16
    plan = [(0, 1), (0, 130), (37, 100), (64, 64), (0, 300), (5, 63), (100, 200)]
    lens = [s + n for s, n in plan]
    pc = Paged(lens, nkv, D, dt, 46, fill=300.0)
    q_lens = [n for _, n in plan]
    T = sum(q_lens)
    q = _rand((T, nq, D), dt, 47)
    scale = 1.0 / math.sqrt(D)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    if window is None:
        seq, key, row = 4, 3, cu[4] + 299
        q[row] = 0
        q[row, :, 0] = 30.0
        pc.k[seq][:, :, 0] = 0
        pc.k[seq][key, :, 0] = 30.0
        for j in range(lens[seq]):
            pc.store(seq, j, pc.k[seq][j], pc.v[seq][j])
    got = ops.attn_prefill_tc(
        q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV),
        cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
        slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV),
        kv_len=torch.tensor(lens, dtype=torch.int32, device=DEV), q_lens=tuple(q_lens), page=64,
        scale=scale, window=window, rows_per_block=rows_per_block).cpu()
    ops.check_kernel_errors()
    assert not torch.isnan(got.float()).any()
    for s, (start, n) in enumerate(plan):
        for i in sorted(set([0, n // 2, n - 1, min(n - 1, 63), min(n - 1, 64), min(n - 1, 127), min(n - 1, 128)])):
            want = _attn_oracle(q[cu[s] + i], pc.k[s], pc.v[s], start + i, scale, window)
            assert torch.allclose(got[cu[s] + i].double(), want, **FAST_TOL), (s, i)
    s, (start, n) = 2, plan[2]
    for i in range(n):
        want = _attn_oracle(q[cu[s] + i], pc.k[s], pc.v[s], start + i, scale, window)
        assert torch.allclose(got[cu[s] + i].double(), want, **FAST_TOL), (s, i)
    if window is None:
        assert torch.allclose(got[cu[4] + 299, 0].double(), pc.v[4][3, 0].double(), atol=1e-2, rtol=1e-2)


def _plant_window_edge(q, row, pc, seq, pos, window):
    """Makes query ``row`` (at position ``pos`` of sequence ``seq``) look along one
    axis only, and gives two keys a component there: the key just outside its
    window (pos - window) the largest, the key just inside (pos - window + 1) the
    second largest, every other key of the sequence none.  With the window right
    the output is the inner key's value; one key too many and it is the outer
    key's value; one too few and it is a blend of all of them."""
    q[row] = 0
    q[row, :, 0] = 30.0
    pc.k[seq][pos - window, :, 0] = 30.0
    pc.k[seq][pos - window + 1, :, 0] = 20.0


def _clear_axis(pc, seq):
    pc.k[seq][:, :, 0] = 0


def _restore(pc, seq):
    for j in range(pc.k[seq].shape[0]):
        pc.store(seq, j, pc.k[seq][j], pc.v[seq][j])


@pytest.mark.parametrize("kernel", ["decode-1", "decode-3", "tma-decode-1", "tma-decode-3", "mma",
                                    "tc-128", "tc-256"])
@pytest.mark.parametrize("nq,nkv,D", [(8, 2, 128), (6, 3, 64)])
def test_the_window_edge_to_the_key(kernel, nq, nkv, D):
    """The tensor-core attention kernels at a window's edge, with keys planted so that
    an edge off by one in either direction changes the output entirely: edges that fall
    on a page boundary (the outer key the last of page 0, the inner the first of
    page 1), inside a page, and in a continued prompt."""
    ops = _ops()
    dt, W = torch.bfloat16, 70
    scale = 1.0 / math.sqrt(D)
    if "decode" in kernel:
        # the one query of each sequence sits at its last position
        lens = [W + 64, W + 81, 3 * 64 + 5, W + 1]
        pc = Paged(lens, nkv, D, dt, 60)
        q = _rand((len(lens), nq, D), dt, 61)
        planted = []
        for s, n in enumerate(lens):
            _clear_axis(pc, s)
            _plant_window_edge(q, s, pc, s, n - 1, W)
            _restore(pc, s)
            planted.append((s, s, n - 1))
        run = ops.attn_decode_tma if kernel.startswith("tma") else ops.attn_decode_bf16
        got = run(
            q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV),
            slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV),
            kv_len=torch.tensor(lens, dtype=torch.int32, device=DEV), page=64, scale=scale,
            max_kv_len=512, window=W, n_splits=int(kernel[-1])).cpu()
        ops.check_kernel_errors()
    else:
        # (tokens already held, tokens of this step); planted rows by position
        plan = [(0, 260), (50, 200)]
        spots = {0: [63 + W, 210], 1: [63 + W, 249]}
        lens = [a + n for a, n in plan]
        pc = Paged(lens, nkv, D, dt, 62, fill=300.0)
        cu = [0, plan[0][1], plan[0][1] + plan[1][1]]
        q = _rand((cu[-1], nq, D), dt, 63)
        planted = []
        for s, (held, n) in enumerate(plan):
            _clear_axis(pc, s)
            for pos in spots[s]:
                _plant_window_edge(q, cu[s] + pos - held, pc, s, pos, W)
                planted.append((cu[s] + pos - held, s, pos))
            _restore(pc, s)
        common = dict(cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
                      slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV),
                      kv_len=torch.tensor(lens, dtype=torch.int32, device=DEV),
                      q_lens=tuple(n for _, n in plan), page=64, scale=scale, window=W)
        args = (q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV))
        if kernel == "mma":
            got = ops.attn_prefill_bf16(*args, **common).cpu()
        else:
            got = ops.attn_prefill_tc(*args, rows_per_block=int(kernel[3:]), **common).cpu()
            ops.check_kernel_errors()
    g = nq // nkv
    for row, s, pos in planted:
        for h in range(nq):
            inner = pc.v[s][pos - W + 1, h // g].double()
            outer = pc.v[s][pos - W, h // g].double()
            assert torch.allclose(got[row, h].double(), inner, atol=1e-2, rtol=1e-2), \
                (kernel, row, s, pos, h, "outer key seen" if torch.allclose(
                    got[row, h].double(), outer, atol=1e-2, rtol=1e-2) else "inner key missed")


@pytest.mark.parametrize("N", [200, 2560])
def test_add_rmsnorm_takes_partial_sums(N):
    """The residual add accepts the 32-bit partial sums of a split-K product."""
    dt = torch.bfloat16
    rows, S = 9, 5
    res = _rand((rows, N), torch.float32, 90)
    parts = _rand((S, rows, N), torch.float32, 91)
    w = (1 + 0.1 * _rand((N,), torch.float32, 92)).to(dt)
    want_res = res.double() + parts.double().sum(0)
    want_y = plain.rms_norm(want_res, w, 1e-5)
    r = res.clone().to(DEV)
    res_out, y = _ops().add_rmsnorm(r, parts.to(DEV), w.to(DEV), 1e-5, dtype=dt)
    assert torch.allclose(res_out.cpu().double(), want_res, atol=2e-6, rtol=1e-6)
    assert torch.allclose(y.cpu().double(), want_y, atol=4 * _eps(dt), rtol=2 * _eps(dt))
    idx = torch.tensor([8, 0, 3], dtype=torch.int32)
    res2, y2 = _ops().add_rmsnorm(res.to(DEV), parts.to(DEV), w.to(DEV), 1e-5, dtype=dt, rows=idx.to(DEV))
    assert torch.allclose(res2.cpu().double(), want_res[idx.long()], atol=2e-6, rtol=1e-6)
    assert torch.allclose(y2.cpu().double(), want_y[idx.long()], atol=4 * _eps(dt), rtol=2 * _eps(dt))


@pytest.mark.parametrize("nq,nkv,D", [(6, 2, 48), (8, 1, 128), (3, 3, 64)])
def test_qk_prepare_takes_partial_sums(nq, nkv, D):
    dt = torch.bfloat16
    pc = Paged([3, 70], nkv, D, dt, 93)
    places = [(0, 2), (1, 63), (1, 64)]
    T, S = len(places), 3
    width = (nq + 2 * nkv) * D
    parts = _rand((S, T, width), torch.float32, 94)
    whole = parts.double().sum(0)
    q_w = (1 + 0.1 * _rand((D,), torch.float32, 95)).to(dt)
    k_w = (1 + 0.1 * _rand((D,), torch.float32, 96)).to(dt)
    theta, eps = 50000.0, 1e-5
    inv = torch.from_numpy(plain.rope_inv_freq(D, theta))
    pos = [p for _, p in places]
    x = whole.view(T, nq + 2 * nkv, D)
    cos, sin = plain.rope_cos_sin(pos, D, theta)
    want_q = plain.apply_rope(plain.rms_norm(x[:, :nq], q_w, eps), cos, sin)
    want_k = plain.apply_rope(plain.rms_norm(x[:, nq:nq + nkv], k_w, eps), cos, sin)
    kp, vp = pc.k_pages.to(DEV), pc.v_pages.to(DEV)
    q, _ = _ops().qk_prepare(
        parts.to(DEV), nq, nkv, D, q_w=q_w.to(DEV), k_w=k_w.to(DEV), eps=eps, inv_freq=inv.to(DEV),
        rot_dim=D, token_seq=torch.tensor([s for s, _ in places], dtype=torch.int32, device=DEV),
        token_pos=torch.tensor(pos, dtype=torch.int32, device=DEV),
        slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV),
        block_table=pc.table.to(DEV), k_pages=kp, v_pages=vp, page=64)
    tol = dict(atol=6 * _eps(dt), rtol=4 * _eps(dt))
    assert q.dtype == dt and torch.allclose(q.cpu().double(), want_q, **tol)
    for r, (s, p) in enumerate(places):
        pg = int(pc.table[pc.slot_of[s], p // 64])
        assert torch.allclose(kp[pg, :, p % 64].cpu().double(), want_k[r], **tol)
        assert torch.allclose(vp[pg, :, p % 64].cpu().double(), x[r, nq + nkv:], **tol)


def test_pages_beyond_two_to_the_31_elements():
    """The same sequences in the first pages of a cache and in pages whose element
    offsets need more than 31 bits: every attention kernel and the q/k preparation
    must return and store the same bits."""
    ops = _ops()
    dt = torch.bfloat16
    nq, nkv, D, page = 16, 8, 128, 64
    free, total = torch.cuda.mem_get_info()
    far = (1 << 31) // (nkv * page * D) + 200           # first far page: offset > 2^31 elements
    plan = [(0, 130), (70, 100), (0, 1), (5, 63)]
    lens = [s + n for s, n in plan]
    pc = Paged(lens, nkv, D, dt, 90, fill=0.0)
    n_small = pc.k_pages.shape[0]
    need = 2 * (far + n_small) * nkv * page * D * 2
    if free < need + (2 << 30):
        pytest.skip("not enough free device memory for a cache of 2^31 elements")
    big_k = torch.empty((far + n_small, nkv, page, D), dtype=dt, device=DEV)
    big_v = torch.empty_like(big_k)
    big_k[far:] = pc.k_pages.to(DEV)
    big_v[far:] = pc.v_pages.to(DEV)
    big_k[:n_small].zero_()
    big_v[:n_small].zero_()
    near = (pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV))
    there = (big_k, big_v, (pc.table + far).to(DEV))
    q_lens = [n for _, n in plan]
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    q = _rand((T, nq, D), dt, 91).to(DEV)
    qd = _rand((len(lens), nq, D), dt, 92).to(DEV)
    scale = 1.0 / math.sqrt(D)
    slots = torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV)
    kvl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=DEV)
    tok_seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(q_lens)]).to(DEV)
    tok_pos = torch.cat([torch.arange(s, s + n, dtype=torch.int32) for s, n in plan]).to(DEV)

    def all_kernels(kp, vp, table):
        outs = [
            ops.attn_decode_bf16(qd, kp, vp, table, slots=slots, kv_len=kvl, page=page, scale=scale,
                                 max_kv_len=256, n_splits=3),
            ops.attn_prefill_tc(q, kp, vp, table, cu_q=cu_t, slots=slots, kv_len=kvl,
                                q_lens=tuple(q_lens), page=page, scale=scale),
            ops.attn_prefill_bf16(q, kp, vp, table, cu_q=cu_t, slots=slots, kv_len=kvl,
                                  q_lens=tuple(q_lens), page=page, scale=scale),
            ops.attn_generic(q, kp, vp, table, token_seq=tok_seq, token_pos=tok_pos, slots=slots,
                             page=page, scale=scale),
        ]
        torch.cuda.synchronize()
        ops.check_kernel_errors()
        return [o.clone() for o in outs]

    a, b = all_kernels(*near), all_kernels(*there)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    # the q/k preparation stores the step's keys and values where the table says
    qkv = _rand((T, (nq + 2 * nkv) * D), dt, 93).to(DEV)
    w = _rand((D,), dt, 94).abs().to(DEV)
    inv = (1.0 / (1e4 ** (torch.arange(0, D, 2).float() / D))).to(DEV)
    near_kv = (near[0].clone(), near[1].clone())
    for rows in (slice(cu[3], cu[4]), slice(0, T)):      # the few-token kernel, and a prompt's
        stored = []
        for (kp, vp, table), first in (((*near_kv, near[2]), 0), (there, far)):
            ops.qk_prepare(qkv[rows], nq, nkv, D, q_w=w, k_w=w, eps=1e-6, inv_freq=inv, rot_dim=D,
                           token_seq=tok_seq[rows], token_pos=tok_pos[rows], slots=slots,
                           block_table=table, k_pages=kp, v_pages=vp, page=page)
            torch.cuda.synchronize()
            stored.append((kp[first:].clone(), vp[first:].clone()))
        assert torch.equal(stored[0][0], stored[1][0]) and torch.equal(stored[0][1], stored[1][1])
        assert not torch.equal(stored[0][0], near[0])        # something was stored
    assert bool((big_k[:n_small] == 0).all()) and bool((big_v[:n_small] == 0).all())   # nothing strayed
