"""Each part alone: built from its spec, given random tensors, run on a small
step, and compared with the plain implementation's function for that part."""

import pytest
import torch

from plain import qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": dict(atol=2e-5, rtol=2e-4), "bfloat16": dict(atol=0.02, rtol=0.035)}


def _ctx(dtype):
    from grout_b200.parts import BuildContext
    return BuildContext(DT[dtype], DEV)


def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


def _params(part, seed, dtype):
    """Random tensors for a part: matrices N(0, 0.05), vectors 1 + N(0, 0.1), rounded to bf16
    so that both precisions and the oracle see the same values."""
    out = {}
    for i, (name, spec) in enumerate(sorted(part.param_specs().items())):
        t = _rand(spec.shape, seed + i, 0.1 if spec.kind == "vector" else 0.05)
        if spec.kind == "vector":
            t = 1.0 + t
        out[name] = t.to(torch.bfloat16)
    return out


def _load(part, params, dtype):
    part.load({k: v.to(DT[dtype]).to(DEV) for k, v in params.items()})


def _step(entries, want=None):
    from grout_b200.engine.batch import make_context
    return make_context(entries, want, DEV)


@pytest.mark.parametrize("dtype", list(DT))
def test_rmsnorm_part(dtype):
    from grout_b200.parts import PartSpec, build_part
    norm = build_part("norm", PartSpec("rmsnorm", dict(dim=200, eps=3e-6)), _ctx(dtype))
    p = _params(norm, 1, dtype)
    _load(norm, p, dtype)
    x = _rand((7, 200), 2).to(torch.bfloat16)
    res = _rand((7, 200), 3)
    y = norm.forward(x.to(DT[dtype]).to(DEV))
    assert torch.allclose(y.double().cpu(), plain.rms_norm(x, p["weight"], 3e-6), **TOL[dtype])
    r2, y2 = norm.add_norm(res.clone().to(DEV), x.to(DT[dtype]).to(DEV))
    assert torch.allclose(r2.double().cpu(), res.double() + x.double(), atol=1e-6, rtol=1e-6)
    assert torch.allclose(y2.double().cpu(), plain.rms_norm(res.double() + x.double(), p["weight"], 3e-6),
                          **TOL[dtype])


def test_rotary_part_table_is_the_plain_table():
    from grout_b200.parts import PartSpec, build_part
    for D, theta in ((16, 10000.0), (48, 5e5), (128, 1e6)):
        pe = build_part("position", PartSpec("rotary_half_split", dict(head_dim=D, theta=theta)),
                        _ctx("float32"))
        rot = pe.rotary()
        assert rot.rot_dim == D
        assert torch.equal(rot.inv_freq.cpu(), torch.from_numpy(plain.rope_inv_freq(D, theta)))


@pytest.mark.parametrize("dtype", list(DT))
def test_swiglu_part(dtype):
    from grout_b200.parts import PartSpec, build_part
    ff = build_part("feedforward", PartSpec("swiglu", dict(hidden=96, intermediate=200)), _ctx(dtype))
    p = _params(ff, 10, dtype)
    _load(ff, p, dtype)
    for rows in (3, 70):                  # the decode product and the library product
        x = _rand((rows, 96), 11 + rows).to(torch.bfloat16)
        got = ff.forward(x.to(DT[dtype]).to(DEV), None)
        want = plain.swiglu(x.double(), p["gate_proj.weight"], p["up_proj.weight"], p["down_proj.weight"])
        assert torch.allclose(got.double().cpu(), want, **TOL[dtype]), rows


@pytest.mark.parametrize("kernel", ["auto", "pair", "tc", "library"])
def test_swiglu_part_with_every_prompt_product(kernel):
    """The feed-forward of a prompt through each of the products a Linear can be told
    to use; "pair" fuses SiLU into the gate|up product on pairs of SMs."""
    from grout_b200.parts import BuildContext, PartSpec, ProductChoice, build_part
    ctx = BuildContext(torch.bfloat16, DEV, ProductChoice(prefill=kernel))
    ff = build_part("feedforward", PartSpec("swiglu", dict(hidden=96, intermediate=208)), ctx)
    p = _params(ff, 12, "bfloat16")
    _load(ff, p, "bfloat16")
    assert ff.gate_up.prefill_kernel == ff.down.prefill_kernel == kernel
    for rows in (65, 300):
        x = _rand((rows, 96), 13 + rows).to(torch.bfloat16)
        got = ff.forward(x.to(DEV), None)
        if got.dim() == 3:
            got = got.sum(0)
        want = plain.swiglu(x.double(), p["gate_proj.weight"], p["up_proj.weight"], p["down_proj.weight"])
        assert torch.allclose(got.double().cpu(), want, **TOL["bfloat16"]), rows
    from grout_b200.kernels import ops
    ops.check_kernel_errors()


@pytest.mark.parametrize("window", [None, 24])
@pytest.mark.parametrize("dtype", list(DT))
def test_attention_part_prefill_then_decode(dtype, window):
    """The mixer alone with a cache of its own: a prompt in one step, then three
    single tokens; every output row against the plain attention block."""
    from grout_b200.cache import CacheLayout, SequenceCache
    from grout_b200.parts import PartSpec, build_part
    H, nq, nkv, D, eps, theta = 80, 6, 3, 32, 1e-5, 5e4
    spec = PartSpec("gqa_attention", dict(
        hidden=H, n_heads=nq, n_kv_heads=nkv, head_dim=D, qk_norm_eps=eps, window=window,
        position=PartSpec("rotary_half_split", dict(head_dim=D, theta=theta))))
    attn = build_part("mixer", spec, _ctx(dtype))
    p = _params(attn, 20, dtype)
    _load(attn, p, dtype)
    cache = SequenceCache(CacheLayout.from_specs([attn.cache_spec()]), max_tokens=512, max_slots=4,
                          max_seq_len=256, dtype=DT[dtype], device=DEV)
    lens = [70, 9]
    T = [n + 3 for n in lens]
    xs = [_rand((t, H), 30 + i).to(torch.bfloat16) for i, t in enumerate(T)]
    cfg = dict(num_attention_heads=nq, num_key_value_heads=nkv, head_dim=D, rms_norm_eps=eps,
               rope_theta=theta)
    w = {"L.self_attn." + k: v for k, v in p.items()}
    want = [plain.attention_block(x.double(), w, "L.", cfg, list(range(x.shape[0])), window) for x in xs]
    slots = [cache.open() for _ in lens]
    got = [[] for _ in lens]

    def run(chunks):
        entries = []
        for s, (a, b) in zip(slots, chunks):
            cache.reserve(s, b - a)
            entries.append((s, cache.length[s], [0] * (b - a)))
        cache.flush()
        step = _step(entries)
        x = torch.cat([xs[i][a:b] for i, (a, b) in enumerate(chunks)]).to(DT[dtype]).to(DEV)
        y = attn.forward(x, step, cache.view(0)).double().cpu()
        o = 0
        for i, (a, b) in enumerate(chunks):
            got[i].append(y[o:o + b - a])
            o += b - a
            cache.advance(slots[i], b - a)

    run([(0, n) for n in lens])
    for k in range(3):
        run([(n + k, n + k + 1) for n in lens])
    for i in range(len(lens)):
        assert torch.allclose(torch.cat(got[i]), want[i], **TOL[dtype]), i
    for s in slots:
        cache.close(s)
    cache.check()


@pytest.mark.parametrize("dtype", list(DT))
def test_prenorm_block_and_io_parts(dtype):
    """Embedding, one block, final norm and head chained by hand, as the model does."""
    from grout_b200.cache import CacheLayout, SequenceCache
    from grout_b200.parts import PartSpec, build_part
    H, I, V, nq, nkv, D, eps, theta = 64, 96, 130, 4, 2, 16, 1e-6, 1e4
    ctx = _ctx(dtype)
    norm = PartSpec("rmsnorm", dict(dim=H, eps=eps))
    block = build_part("block", PartSpec("prenorm", dict(
        norm1=norm, norm2=norm,
        mixer=PartSpec("gqa_attention", dict(hidden=H, n_heads=nq, n_kv_heads=nkv, head_dim=D,
                                             qk_norm_eps=eps,
                                             position=PartSpec("rotary_half_split",
                                                               dict(head_dim=D, theta=theta)))),
        feedforward=PartSpec("swiglu", dict(hidden=H, intermediate=I)))), ctx)
    emb = build_part("embedding", PartSpec("token", dict(vocab=V, hidden=H)), ctx)
    fin = build_part("norm", norm, ctx)
    head = build_part("head", PartSpec("linear", dict(vocab=V, hidden=H, tied=True)), ctx)
    names = {"norm1": "input_layernorm.", "mixer": "self_attn.", "norm2": "post_attention_layernorm.",
             "feedforward": "mlp."}
    w = {}
    for role, part in block.named_parts().items():
        p = _params(part, 40 + len(w), dtype)
        _load(part, p, dtype)
        w.update({"model.layers.0." + names[role] + k: v for k, v in p.items()})
    for part, prefix, seed in ((emb, "model.embed_tokens.", 60), (fin, "model.norm.", 61)):
        p = _params(part, seed, dtype)
        _load(part, p, dtype)
        w.update({prefix + k: v for k, v in p.items()})
    head.tie(emb.weight)
    cfg = dict(num_hidden_layers=1, num_attention_heads=nq, num_key_value_heads=nkv, head_dim=D,
               rms_norm_eps=eps, rope_theta=theta, tie_word_embeddings=True)
    tokens = [5, 129, 0, 77, 31, 8, 8, 100, 64]
    cache = SequenceCache(CacheLayout.from_specs([block.cache_spec()]), max_tokens=128, max_slots=2,
                          max_seq_len=128, dtype=DT[dtype], device=DEV)
    s = cache.open()
    cache.reserve(s, len(tokens))
    cache.flush()
    step = _step([(s, 0, tokens)], [[0, len(tokens) - 1]])
    x = emb.forward(step.tokens, step)
    res, pending = block.forward(None, x, step, cache.view(0))
    _r, h = fin.add_norm(res, pending, rows=step.want_rows)
    logits = head.forward(h)
    assert logits.dtype == torch.float32
    want = plain.logits(w, cfg, tokens, rows=[0, len(tokens) - 1])
    assert torch.allclose(logits.double().cpu(), want, **TOL[dtype])
