"""Argmax and sampling kernels against the plain sampler, fed the same draws."""
import random

import pytest
import torch

from plain import sampling as plain_sampling

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from grout_b200.kernels import ops
    return ops


def test_argmax_first_maximum_wins():
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(6, 1003, generator=g)
    logits[1, 17] = logits[1, 900] = 9.0           # a tie: the lower index wins
    logits[2, 1002] = 11.0                         # the last element
    logits[3, 0] = 11.0
    logits[4, 5] = float("nan")                    # NaN never wins
    logits[5] = 0.25                               # all equal
    got = _ops().argmax(logits.to(DEV)).cpu().tolist()
    want = [plain_sampling.argmax_first([v if v == v else float("-inf") for v in row.tolist()])
            for row in logits]
    assert got == want and got[1] == 17 and got[5] == 0


CASES = [(1.0, 0, 1.0), (0.8, 0, 1.0), (0.8, 20, 1.0), (0.8, 0, 0.9), (0.7, 50, 0.95),
         (1.5, 1, 1.0), (1.0, 0, 0.0), (0.3, 5, 0.5), (2.0, 1002, 0.999), (1e-6, 10, 0.5)]


@pytest.mark.parametrize("quantised", [False, True])
def test_sample_matches_plain_sampler(quantised):
    """Rows with continuous logits, and rows rounded to a coarse grid so that the
    thresholds of top-k and top-p fall on ties."""
    rng = random.Random(1)
    g = torch.Generator().manual_seed(2)
    V = 1003
    rows, temps, ks, ps, us = [], [], [], [], []
    for t, k, p in CASES:
        for _ in range(6):
            row = torch.randn(V, generator=g) * 2.0
            if quantised:
                row = (row * 2).round() / 2
            rows.append(row)
            temps.append(t), ks.append(k), ps.append(p), us.append(rng.random())
    logits = torch.stack(rows)
    got = _ops().sample(logits.to(DEV), torch.tensor(temps, device=DEV),
                        torch.tensor(ks, dtype=torch.int32, device=DEV),
                        torch.tensor(ps, device=DEV), torch.tensor(us, device=DEV)).cpu().tolist()
    us32 = torch.tensor(us).tolist()               # the kernel sees float32 draws
    for i in range(len(rows)):
        want = plain_sampling.sample_next(rows[i].tolist(), temps[i], ks[i], ps[i], us32[i])
        assert got[i] == want, (i, temps[i], ks[i], ps[i], us32[i], got[i], want)


def test_sample_stays_inside_top_k_and_follows_the_distribution():
    V, n = 257, 4000
    g = torch.Generator().manual_seed(3)
    row = torch.randn(V, generator=g)
    logits = row.repeat(n, 1).to(DEV)
    u = torch.rand(n, generator=g).to(DEV)
    got = _ops().sample(logits, torch.full((n,), 0.9, device=DEV),
                        torch.full((n,), 8, dtype=torch.int32, device=DEV),
                        torch.ones(n, device=DEV), u).cpu()
    top = torch.topk(row, 8).indices
    assert set(got.tolist()) <= set(top.tolist())
    p = torch.softmax(row[top] / 0.9, 0)
    for j, idx in enumerate(top.tolist()):
        assert abs((got == idx).float().mean().item() - p[j].item()) < 0.03


def test_host_sampler_agrees_with_plain():
    from grout_b200.sampling import SamplingParams, choose_one
    rng = random.Random(4)
    g = torch.Generator().manual_seed(5)
    for t, k, p in CASES:
        row = ((torch.randn(300, generator=g) * 4).round() / 2)
        u = rng.random()
        want = plain_sampling.sample_next(row.tolist(), t, k, p, u)
        got = choose_one(row.numpy(), SamplingParams(True, t, k, p).normalised(), u)
        assert got == want, (t, k, p)
