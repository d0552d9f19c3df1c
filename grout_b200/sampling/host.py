"""Choosing tokens on the host from logits copied back, the way the reference
does when the device argmax is off (src/model.rs:2120-2171, sample_next
2212-2270).  Kept for ``--device-argmax`` being absent and as a second opinion
on the device sampler; generation defaults to the device."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .params import SamplingParams


def choose_one(logits: np.ndarray, p: SamplingParams, u: float) -> int:
    if p.greedy:
        return int(np.argmax(logits))          # first maximum
    s = logits.astype(np.float32) * np.float32(1.0 / p.temperature)
    s = np.where(np.isnan(s), -np.inf, s)
    order = np.argsort(-s, kind="stable")      # descending, equal scores keep index order
    if 0 < p.top_k < s.shape[0]:
        order = order[:p.top_k]
    probs = np.exp((s[order] - s[order[0]]).astype(np.float64))
    if p.top_p < 1.0:
        total = probs.sum()
        if np.isfinite(total) and total > 0:
            cum = np.cumsum(probs / total)
            keep = int(np.searchsorted(cum, p.top_p, side="left")) + 1
            order, probs = order[:keep], probs[:keep]
    total = probs.sum()
    if not np.isfinite(total) or total <= 0:
        return int(np.argmax(logits))
    # the kept set is walked in index order, as the device kernel does
    by_index = np.argsort(order, kind="stable")
    order, probs = order[by_index], probs[by_index]
    cum = np.cumsum(probs)
    i = int(np.searchsorted(cum, u * total, side="left"))
    return int(order[min(i, order.shape[0] - 1)])


class HostSampler:
    def __init__(self, device=None):
        pass

    def kernel_modules(self):
        return ()

    def choose(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               draws: Sequence[float]) -> List[int]:
        rows = logits.detach().float().cpu().numpy()
        return [choose_one(rows[i], params[i], draws[i]) for i in range(rows.shape[0])]
