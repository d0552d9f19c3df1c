"""Choosing tokens on the GPU from the step's 32-bit logits."""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams


class DeviceSampler:
    """Rows of logits -> one token per row.  Greedy rows go through the argmax
    kernel; if any row samples, all rows go through the sampling kernel, which
    treats a temperature at the floor as greedy."""

    def __init__(self, device):
        self.device = torch.device(device)

    def kernel_modules(self):
        return ("sample",)

    def choose(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               draws: Sequence[float]) -> torch.Tensor:
        n = logits.shape[0]
        if len(params) != n or len(draws) != n:
            raise ValueError("one SamplingParams and one draw per row of logits are needed")
        if all(p.greedy for p in params):
            return ops.argmax(logits)
        host = np.zeros((4, n), dtype=np.float32)
        for i, p in enumerate(params):
            host[0, i] = 0.0 if p.greedy else p.temperature
            host[1, i] = np.int32(p.top_k).view(np.float32)
            host[2, i] = p.top_p
            host[3, i] = draws[i]
        dev = torch.from_numpy(host).to(self.device)
        return ops.sample(logits, dev[0], dev[1].view(torch.int32), dev[2], dev[3])
