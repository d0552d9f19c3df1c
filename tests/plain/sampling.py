"""Plain sampling, restating the reference's ``sample_next``
(src/model.rs:2212-2270), with the random draw given from outside."""
from __future__ import annotations

import math


def argmax_first(logits) -> int:
    """First maximum wins (src/model.rs:6075-6086)."""
    best, idx = -math.inf, 0
    for i, v in enumerate(logits):
        if v > best:
            best, idx = v, i
    return idx


def kept_set(logits, temperature: float, top_k: int, top_p: float):
    """Indices and unnormalised probabilities that survive top-k and top-p.

    Scale by 1/temperature, sort descending (stable, so equal scores keep index
    order), keep ``top_k`` if 0 < top_k < V (src/model.rs:2221-2230); p_i =
    exp(s_i - s_max) in float64 (2232-2239); with top_p < 1 keep the shortest
    prefix whose normalised mass reaches top_p (2241-2258)."""
    inv_t = 1.0 / float(temperature)
    scores = sorted(((i, float(v) * inv_t) for i, v in enumerate(logits)),
                    key=lambda t: -t[1])
    if 0 < top_k < len(scores):
        scores = scores[:top_k]
    s_max = scores[0][1]
    probs = [(i, math.exp(s - s_max)) for i, s in scores]
    if top_p < 1.0:
        total = sum(p for _, p in probs)
        kept, cum = [], 0.0
        for i, p in probs:
            cum += p / total
            kept.append((i, p))
            if cum >= top_p:
                break
        probs = kept
    return probs


def sample_next(logits, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """Greedy when temperature <= 1e-5 (src/model.rs:2216-2218); else the kept
    set is walked with threshold u * sum(p) (2260-2269).  The reference walks
    it in descending order of probability; this library walks it in index order,
    which draws from the same distribution and needs no sort of the vocabulary
    on the device."""
    if temperature <= 1.0e-5:
        return argmax_first(logits)
    probs = sorted(kept_set(logits, temperature, top_k, top_p))
    total = sum(p for _, p in probs)
    if not math.isfinite(total) or total <= 0.0:
        return argmax_first(logits)
    threshold = u * total
    cum = 0.0
    for i, p in probs:
        cum += p
        if cum >= threshold:
            return i
    return probs[-1][0]
