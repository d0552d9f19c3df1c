"""Position encodings.  Interface of the family:

* ``rotary() -> RotaryTable | None``: an encoding that is a rotation of the
  first ``rot_dim`` elements of every query and key head by angle
  ``pos * inv_freq[j]`` returns its table, and attention folds it into the
  kernel that also normalises q and k and writes the cache.
* ``apply_qk(q, k, token_pos) -> (q, k)``: any other encoding of queries and
  keys ([T, heads, D]); attention calls it between its projection and the
  cache write when ``rotary()`` is None.

An encoding that is added to the embeddings is not of this family: it is an
``embedding`` part, whose ``forward(tokens, step)`` has every row's position in
``step.token_pos``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .base import BuildContext, Part, register_part


@dataclass
class RotaryTable:
    inv_freq: torch.Tensor   # float32 [rot_dim / 2] on the device
    rot_dim: int


class PositionEncoding(Part):
    family = "position"

    def rotary(self) -> Optional[RotaryTable]:
        return None

    def apply_qk(self, q, k, token_pos):
        return q, k


@register_part("position", "none")
class NoPosition(PositionEncoding):
    def __init__(self, ctx: BuildContext):
        super().__init__(ctx)

    def captures_prompts(self):
        return True


@register_part("position", "rotary_half_split")
class RotaryHalfSplit(PositionEncoding):
    """Half-split ("NeoX") rotation: element j pairs with j + rot_dim/2;
    inv_freq[j] = 1 / theta^(2j / rot_dim), computed in float32 on the host and
    uploaded (src/model.rs:5992-5997); the angle pos * inv_freq[j] and its sine
    and cosine are float32 in the kernel (src/kernels.rs:3640-3648)."""

    def __init__(self, ctx: BuildContext, head_dim: int, theta: float,
                 rot_dim: Optional[int] = None):
        super().__init__(ctx)
        self.head_dim = int(head_dim)
        self.rot_dim = int(rot_dim if rot_dim is not None else head_dim)
        if self.rot_dim % 2 or not 0 < self.rot_dim <= self.head_dim:
            raise ValueError(f"rot_dim={self.rot_dim} must be even and at most head_dim={head_dim}")
        self.theta = float(theta)
        i = np.arange(0, self.rot_dim, 2, dtype=np.float32)
        p = i / np.float32(self.rot_dim)
        inv = (np.float32(1.0) / np.power(np.float32(self.theta), p, dtype=np.float32))
        self._table = RotaryTable(torch.from_numpy(inv.astype(np.float32)).to(ctx.device),
                                  self.rot_dim)

    def rotary(self):
        return self._table

    def captures_prompts(self):
        return True
