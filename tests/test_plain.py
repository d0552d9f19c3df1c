"""The plain implementation checked against itself and against hand computation (no GPU)."""
import math

import numpy as np
import torch

from conftest import random_tokens
from plain import qwen3 as plain
from plain import sampling as plain_sampling


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    y = plain.rms_norm(x, w, 0.0)
    r = math.sqrt((9 + 16) / 2)
    assert torch.allclose(y, torch.tensor([[3 / r * 2, 4 / r * 0.5]], dtype=torch.float64))


def test_rope_is_a_rotation_of_half_split_pairs():
    D, theta = 8, 10000.0
    inv = plain.rope_inv_freq(D, theta)
    assert inv.dtype == np.float32 and np.allclose(inv, [1.0, 0.1, 0.01, 0.001], rtol=1e-6)
    x = torch.randn(3, 2, D, dtype=torch.float64)
    cos, sin = plain.rope_cos_sin([0, 1, 7], D, theta)
    y = plain.apply_rope(x, cos, sin)
    assert torch.allclose(y[0], x[0])                       # position 0 rotates by nothing
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))   # lengths are kept
    a = 7 * float(inv[1])
    j = 1
    want_lo = x[2, 0, j] * math.cos(a) - x[2, 0, j + D // 2] * math.sin(a)
    assert abs(float(y[2, 0, j]) - float(want_lo)) < 1e-6


def test_attention_is_causal_and_grouped():
    T, nq, nkv, D = 6, 4, 2, 8
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(T, n, D, generator=g, dtype=torch.float64) for n in (nq, nkv, nkv))
    o = plain.causal_attention(q, k, v)
    assert torch.allclose(o[0, 0], v[0, 0]) and torch.allclose(o[0, 3], v[0, 1])
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, 9.0                               # later keys cannot matter
    assert torch.allclose(plain.causal_attention(q, k2, v2)[:4], o[:4])
    ow = plain.causal_attention(q, k, v, window=1)          # a window of one sees itself only
    assert torch.allclose(ow[:, 0], v[:, 0])


def test_logits_of_a_prefix_do_not_depend_on_what_follows(plain_weights):
    for name in ("A", "C"):
        cfg, w = plain_weights[name]
        toks = random_tokens(50, cfg["vocab_size"], 9)
        full = plain.logits(w, cfg, toks)
        part = plain.logits(w, cfg, toks[:31])
        assert torch.allclose(full[:31], part, atol=1e-12)
        rows = plain.logits(w, cfg, toks, rows=[3, 49])
        assert torch.allclose(rows, full[[3, 49]], atol=1e-12)


def test_tied_and_untied_heads(plain_weights):
    cfg, w = plain_weights["A"]
    assert cfg["tie_word_embeddings"] and "lm_head.weight" not in w
    cfg_b, w_b = plain_weights["B"]
    assert "lm_head.weight" in w_b
    assert plain.logits(w_b, cfg_b, [1, 2, 3]).shape == (3, 384)


def test_greedy_stops_before_the_stop_token(plain_weights):
    cfg, w = plain_weights["A"]
    free = plain.greedy_generate(w, cfg, [5, 6, 7], 6)
    assert len(free) == 6
    stopped = plain.greedy_generate(w, cfg, [5, 6, 7], 6, stop_ids=(free[2],))
    first = free.index(free[2])
    assert stopped == free[:first]


def test_plain_sampling():
    logits = [0.0, 2.0, 1.0, 2.0, -1.0]
    assert plain_sampling.argmax_first(logits) == 1
    assert plain_sampling.sample_next(logits, 0.0, 0, 1.0, 0.7) == 1
    kept = plain_sampling.kept_set(logits, 1.0, 2, 1.0)
    assert [i for i, _ in kept] == [1, 3]
    kept = plain_sampling.kept_set(logits, 1.0, 0, 0.5)
    assert [i for i, _ in kept] == [1, 3]
    assert plain_sampling.sample_next(logits, 1.0, 2, 1.0, 0.25) == 1
    assert plain_sampling.sample_next(logits, 1.0, 2, 1.0, 0.75) == 3
    counts = [0] * 5
    import random
    rng = random.Random(0)
    for _ in range(4000):
        counts[plain_sampling.sample_next(logits, 0.8, 0, 1.0, rng.random())] += 1
    z = [math.exp(v / 0.8) for v in logits]
    for i in range(5):
        assert abs(counts[i] / 4000 - z[i] / sum(z)) < 0.03


def test_host_sampler_follows_the_plain_sampler():
    """The library's host-side sampler (numpy, vectorised) against the plain one, fed the
    same logits and draws: ties, top-k, top-p, both, and a temperature at its floor."""
    import random

    import numpy as np

    from grout_b200.sampling import SamplingParams
    from grout_b200.sampling.host import choose_one
    rng = random.Random(3)
    g = torch.Generator().manual_seed(4)
    for trial in range(300):
        v = rng.choice([5, 37, 300])
        logits = (torch.randn(v, generator=g) * rng.choice([0.5, 3.0])).float()
        if trial % 4 == 0:                       # equal scores: index order decides
            logits[rng.randrange(v)] = logits[rng.randrange(v)]
            logits = (logits * 4).round() / 4
        t = rng.choice([1e-5, 0.3, 0.8, 1.0, 2.5])
        k = rng.choice([0, 1, 2, 7, v, v + 3])
        p = rng.choice([1.0, 0.9, 0.5, 0.05, 0.0])
        u = rng.random()
        params = SamplingParams(True, t, k, p).normalised()
        got = choose_one(np.asarray(logits), params, u)
        want = plain_sampling.sample_next(logits.tolist(), params.temperature, params.top_k, params.top_p, u)
        assert got == want, (trial, v, t, k, p, u)
    assert choose_one(np.asarray([1.0, 3.0, 3.0], dtype=np.float32), SamplingParams().normalised(), 0.9) == 1
