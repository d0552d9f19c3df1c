"""Norms.  Interface of the family:

* ``forward(x) -> y``: normalises rows of ``x`` [T, N] (compute dtype).
* ``add_norm(res, delta, rows=None) -> (res, y)``: adds ``delta`` (compute
  dtype, may be None) into the 32-bit residual stream ``res`` (may be None on
  the first layer), optionally keeps only ``rows``, and returns the updated
  stream with its normalised rows.  ``delta`` may also arrive as a stack of
  32-bit partial sums [S, T, N] (a split-K projection leaves its reduction to
  the norm); they are added in order.  The default does the steps one after the
  other; RMSNorm does all of it in one kernel.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..kernels import ops
from .base import BuildContext, ParamSpec, Part, register_part


class Norm(Part):
    family = "norm"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_norm(self, res: Optional[torch.Tensor], delta: Optional[torch.Tensor],
                 rows: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        res = residual_add(res, delta, rows)
        return res, self.forward(ops.cast(res, self.ctx.dtype))


def residual_add(res, delta, rows=None) -> torch.Tensor:
    """32-bit residual sum for norms without a fused kernel (a library call on
    small tensors; parts of this package use the fused kernel instead)."""
    if delta is not None and delta.dim() == 3:      # partial sums of a split-K product
        delta = delta.sum(dim=0)
    if res is None:
        out = delta.float()
    elif delta is None:
        out = res
    else:
        out = res + delta.float()
    return out if rows is None else out.index_select(0, rows.long())


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * w; the weight multiplies as it is
    (src/kernels.rs:316-341, src/training.rs:233-238)."""

    def __init__(self, ctx: BuildContext, dim: int, eps: float):
        super().__init__(ctx)
        self.dim, self.eps = int(dim), float(eps)
        self.weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.dim,), "vector")}

    def load(self, params):
        self.weight = params["weight"].contiguous()

    def kernel_modules(self):
        return ("norm",)

    def captures_prompts(self):
        return True

    def forward(self, x):
        _res, y = ops.add_rmsnorm(None, x, self.weight, self.eps, dtype=self.ctx.dtype,
                                  write_res=False)
        return y

    def add_norm(self, res, delta, rows=None):
        return ops.add_rmsnorm(res, delta, self.weight, self.eps, dtype=self.ctx.dtype, rows=rows)
