"""Feed-forward parts.  Interface of the family: ``forward(x, step) -> y`` with
``x`` and ``y`` [T, hidden] in the compute dtype (``y`` may be a stack of 32-bit
partial sums [S, T, hidden], which the next norm adds: see ``Norm.add_norm``).  A feed-forward with experts
routes inside ``forward``; the rows' packing is the step's and does not change.
"""
from __future__ import annotations

import torch

from .base import BuildContext, ParamSpec, Part, register_part
from .linear import Linear


class FeedForward(Part):
    family = "feedforward"

    def forward(self, x, step):
        raise NotImplementedError


@register_part("feedforward", "swiglu")
class SwiGLU(FeedForward):
    """d = (silu(x Wg^T) * (x Wu^T)) Wd^T, no biases (src/training.rs:344-349).
    Gate and up are fused into one product at load (src/model.rs:1401)."""

    def __init__(self, ctx: BuildContext, hidden: int, intermediate: int):
        super().__init__(ctx)
        self.hidden, self.intermediate = int(hidden), int(intermediate)
        self.gate_up = self.down = None
        self.interleave = 0

    def param_specs(self):
        return {"gate_proj.weight": ParamSpec((self.intermediate, self.hidden)),
                "up_proj.weight": ParamSpec((self.intermediate, self.hidden)),
                "down_proj.weight": ParamSpec((self.hidden, self.intermediate))}

    def load(self, params):
        g, u = params["gate_proj.weight"], params["up_proj.weight"]
        if g.dtype != u.dtype:
            raise ValueError("gate and up projections must be stored in one dtype to be fused")
        # bf16: rows interleaved in groups of 8 (8 gates, their 8 ups, ...) so that
        # the decode product holds a gate and its up in one tile and can apply
        # silu(gate) * up before it stores
        self.interleave = 8 if (g.dtype == torch.bfloat16 and self.intermediate % 8 == 0
                                and self.hidden % 8 == 0) else 0
        if self.interleave:
            k = self.interleave
            fused = torch.stack([g.view(-1, k, self.hidden), u.view(-1, k, self.hidden)], dim=1)
            self.gate_up = Linear(fused.reshape(2 * self.intermediate, self.hidden), self.ctx.products)
        else:
            self.gate_up = Linear(torch.cat([g, u], dim=0), self.ctx.products)
        self.down = Linear(params["down_proj.weight"], self.ctx.products)

    def kernel_modules(self):
        return ("elementwise",) + self.gate_up.kernel_modules() + self.down.kernel_modules()

    def captures_prompts(self):
        return True

    def forward(self, x, step):
        return self.down(self.gate_up.silu_mul(x, self.interleave), partial_ok=True)
