"""A model built from a ``ModelPlan``: parts, their tensors, and one forward
over the tokens of a step.  This file names no architecture; the reference's
counterpart is the hand-emitted op list of ``build_step_graph_rows``
(src/model.rs:3708-4031), which is Qwen3 by construction.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..cache import CacheLayout, SequenceCache
from ..parts.base import BuildContext, ParamSpec, Part, build_part
from ..parts.plan import ModelPlan
from .batch import StepContext


def _walk(part: Part):
    yield part
    for c in part.children():
        yield from _walk(c)


class Model:
    def __init__(self, plan: ModelPlan, ctx: BuildContext):
        plan.validate()
        self.plan, self.ctx = plan, ctx
        self.embedding = build_part("embedding", plan.embedding, ctx)
        self.blocks = [build_part("block", lp.block, ctx) for lp in plan.layers]
        self.final_norm = build_part("norm", plan.final_norm, ctx)
        self.head = build_part("head", plan.head, ctx)
        self._layout: Optional[CacheLayout] = None

    # -- tensors -----------------------------------------------------------
    def _named_parts(self) -> List[Tuple[str, Part]]:
        """(checkpoint prefix, part) of every part that reads tensors."""
        out = [(self.plan.embedding_prefix, self.embedding)]
        for lp, block in zip(self.plan.layers, self.blocks):
            named = block.named_parts() if hasattr(block, "named_parts") else {}
            for role, part in named.items():
                out.append((lp.prefix + lp.part_prefix.get(role, role + "."), part))
            out.append((lp.prefix, block))
        out.append((self.plan.final_norm_prefix, self.final_norm))
        out.append((self.plan.head_prefix, self.head))
        return out

    def expected(self) -> Dict[str, ParamSpec]:
        exp: Dict[str, ParamSpec] = {}
        for prefix, part in self._named_parts():
            for local, spec in part.param_specs().items():
                name = prefix + local
                if name in exp:
                    raise ValueError(f"two parts read tensor '{name}'")
                exp[name] = spec
        return exp

    def load(self, get: Callable[[str], torch.Tensor]) -> None:
        """``get(name)`` returns the placed tensor; each part takes its own."""
        for prefix, part in self._named_parts():
            specs = part.param_specs()
            if specs:
                part.load({local: get(prefix + local) for local in specs})
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding.weight)

    # -- cache -------------------------------------------------------------
    def cache_layout(self) -> CacheLayout:
        if self._layout is None:
            specs = []
            for e in self.plan.schedule:
                specs.append(None if e.cache_of is not None else self.blocks[e.layer].cache_spec())
            self._layout = CacheLayout.from_specs(specs)
        return self._layout

    def kernel_modules(self) -> Tuple[str, ...]:
        mods: List[str] = []
        for top in [self.embedding, *self.blocks, self.final_norm, self.head]:
            for p in _walk(top):
                mods.extend(p.kernel_modules())
        return tuple(dict.fromkeys(mods))

    def captures_prompts(self) -> bool:
        """Whether every part allows prompt steps to be captured (``Part.captures_prompts``)."""
        return all(p.captures_prompts()
                   for top in [self.embedding, *self.blocks, self.final_norm, self.head]
                   for p in _walk(top))

    # -- forward -----------------------------------------------------------
    def forward(self, step: StepContext, cache: SequenceCache) -> Optional[torch.Tensor]:
        """Runs the step's tokens through every scheduled layer; returns 32-bit
        logits [n_want, vocab] at ``step.want_rows`` (None when nothing is wanted)."""
        layout = self.cache_layout()
        pending = self.embedding.forward(step.tokens, step)
        res = None
        for i, e in enumerate(self.plan.schedule):
            owner = i if e.cache_of is None else e.cache_of
            view = cache.view(owner) if owner in layout.where else None
            res, pending = self.blocks[e.layer].forward(res, pending, step, view)
        if step.n_want == 0:
            return None
        _res, h = self.final_norm.add_norm(res, pending, rows=step.want_rows)
        return self.head.forward(h)


def expected_tensors(plan: ModelPlan) -> Dict[str, ParamSpec]:
    """Names, shapes and kinds of the tensors a plan reads (no device needed)."""
    return Model(plan, BuildContext(torch.bfloat16, torch.device("cpu"))).expected()
