"""The two ends of the model: token embedding and output head."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import BuildContext, ParamSpec, Part, register_part
from .linear import Linear


class Embedding(Part):
    family = "embedding"

    def forward(self, tokens, step):
        raise NotImplementedError


@register_part("embedding", "token")
class TokenEmbedding(Embedding):
    """x[t] = E[ids[t]], no scaling (src/training.rs:278-282)."""

    def __init__(self, ctx: BuildContext, vocab: int, hidden: int):
        super().__init__(ctx)
        self.vocab, self.hidden = int(vocab), int(hidden)
        self.weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab, self.hidden))}

    def load(self, params):
        self.weight = params["weight"].contiguous()

    def kernel_modules(self):
        return ("embed", "elementwise")

    def captures_prompts(self):
        return True

    def forward(self, tokens, step):
        x = ops.embed(self.weight, tokens)
        return ops.cast(x, self.ctx.dtype) if x.dtype != self.ctx.dtype else x


class Head(Part):
    family = "head"

    def forward(self, h):
        raise NotImplementedError


@register_part("head", "linear")
class LinearHead(Head):
    """logits = h W^T in 32-bit; W is the embedding table when ``tied``
    (src/training.rs:352-362)."""

    def __init__(self, ctx: BuildContext, vocab: int, hidden: int, tied: bool):
        super().__init__(ctx)
        self.vocab, self.hidden, self.tied = int(vocab), int(hidden), bool(tied)
        self.proj: Optional[Linear] = None

    def param_specs(self):
        return {} if self.tied else {"weight": ParamSpec((self.vocab, self.hidden))}

    def load(self, params):
        if not self.tied:
            self.proj = Linear(params["weight"], self.ctx.products)

    def tie(self, table: torch.Tensor) -> None:
        self.proj = Linear(table, self.ctx.products)   # shares the allocation (src/model.rs:1375-1377)

    def kernel_modules(self):
        return self.proj.kernel_modules() if self.proj else ()

    def captures_prompts(self):
        return True

    def forward(self, h):
        return self.proj(h, out_dtype=torch.float32)
