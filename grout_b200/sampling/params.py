"""How the next token is chosen.

The reference reads these from generation_config.json only (do_sample,
temperature clamped to >= 1e-5, top_k, top_p clamped to [0, 1];
src/model.rs:1345-1353) and switches sampling on with ``--sample``; its random
source is unseeded (src/model.rs:2053).  Here they can also be given per
request, and the seed is explicit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class SamplingParams:
    do_sample: bool = False
    temperature: float = 1.0
    top_k: int = 0            # 0: no limit
    top_p: float = 1.0        # 1: no limit
    seed: Optional[int] = None

    def normalised(self) -> "SamplingParams":
        return SamplingParams(self.do_sample, max(float(self.temperature), 1.0e-5),
                              max(int(self.top_k), 0), min(max(float(self.top_p), 0.0), 1.0),
                              self.seed)

    @property
    def greedy(self) -> bool:
        """Greedy when sampling is off or the temperature is at its floor
        (src/model.rs:2216-2218)."""
        return (not self.do_sample) or self.temperature <= 1.0e-5

    @staticmethod
    def from_generation_config(gen, do_sample: Optional[bool] = None, seed=None) -> "SamplingParams":
        if gen is None:
            return SamplingParams(bool(do_sample), seed=seed).normalised()
        return SamplingParams(
            gen.do_sample if do_sample is None and gen.do_sample is not None else bool(do_sample),
            gen.temperature if gen.temperature is not None else 1.0,
            gen.top_k if gen.top_k is not None else 0,
            gen.top_p if gen.top_p is not None else 1.0, seed).normalised()
