"""Blocks: how a layer's norm, mixer and feed-forward are arranged.

Interface of the family: ``forward(res, pending, step, cache) -> (res, pending)``.
The hidden state travels between blocks as a pair: ``res``, the residual stream
in 32-bit ([T, hidden], None before the first block), and ``pending``, a
contribution in the compute dtype that has not been added yet.  Leaving the last
sum pending lets the next norm do it in the same kernel that normalises (the
reference defers the MLP's residual add into the next layer's norm in the same
way, src/model.rs:3151-3164).
"""
from __future__ import annotations

from typing import Dict

from .base import BuildContext, Part, PartSpec, build_part, register_part


class Block(Part):
    family = "block"

    def forward(self, res, pending, step, cache):
        raise NotImplementedError

    def cache_spec(self):
        return None


@register_part("block", "prenorm")
class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += feedforward(norm2(x)) (src/training.rs:303-349)."""

    roles = ("norm1", "mixer", "norm2", "feedforward")

    def __init__(self, ctx: BuildContext, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec,
                 feedforward: PartSpec):
        super().__init__(ctx)
        self.norm1 = build_part("norm", norm1, ctx)
        self.mixer = build_part("mixer", mixer, ctx)
        self.norm2 = build_part("norm", norm2, ctx)
        self.feedforward = build_part("feedforward", feedforward, ctx)

    def children(self):
        return (self.norm1, self.mixer, self.norm2, self.feedforward)

    def named_parts(self) -> Dict[str, Part]:
        return {r: getattr(self, r) for r in self.roles}

    def cache_spec(self):
        return self.mixer.cache_spec()

    def captures_prompts(self):
        return True

    def forward(self, res, pending, step, cache):
        res, n = self.norm1.add_norm(res, pending)
        a = self.mixer.forward(n, step, cache)
        res, m = self.norm2.add_norm(res, a)
        return res, self.feedforward.forward(m, step)
