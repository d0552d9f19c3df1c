"""The layout of a model as data: which parts, in which order, reading which
tensors.  An architecture's ``plan(config)`` returns a ``ModelPlan``; the engine
builds every model from one, so a new architecture is a new plan and, where it
needs them, new parts.

* ``layers`` — one ``LayerPlan`` per set of weights: the block's kind, the spec
  of each of its parts, and under which checkpoint prefix each part's tensors
  lie.  Layers are independent, so different layers may have different mixers
  or feed-forwards.
* ``schedule`` — the order in which layers run, as data: a list of
  ``ScheduleEntry(layer, cache_of)``.  A layer may be named twice (its weights
  run twice; each run that owns a cache has its own), and an entry may read
  another entry's cache instead of owning one (``cache_of`` = index into the
  schedule).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

from .base import PartSpec


@dataclass(frozen=True)
class LayerPlan:
    block: PartSpec                       # family "block"; its args name the parts' specs
    prefix: str                           # e.g. "model.layers.3."
    part_prefix: Dict[str, str]           # block role -> sub-prefix, e.g. {"mixer": "self_attn."}


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int
    cache_of: Optional[int] = None        # schedule index whose cache this entry uses


@dataclass(frozen=True)
class ModelPlan:
    embedding: PartSpec
    embedding_prefix: str                 # "model.embed_tokens."
    layers: Tuple[LayerPlan, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    final_norm_prefix: str                # "model.norm."
    head: PartSpec
    head_prefix: str                      # "lm_head."
    vocab_size: int
    max_position: int                     # longest sequence the architecture allows
    stop_tokens: Tuple[int, ...] = ()

    def validate(self) -> None:
        n = len(self.layers)
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < n:
                raise ValueError(f"schedule entry {i} names layer {e.layer} of {n}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < len(self.schedule) or e.cache_of == i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, "
                                     f"which owns none")
