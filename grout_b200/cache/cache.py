"""The cache of a model: one slot per live sequence, one store per group of
layers, each sequence with its own length.

``CacheLayout`` is derived from the model's layers: every layer that owns a
cache names what it needs (``KVSpec``, ``StateSpec`` or a spec of its own with a
``make_store`` method); layers with equal needs share a store, which the spec
makes (and, for keys and values, one block table).  A layer that
reads another layer's cache owns nothing and is given that layer's view.

``SequenceCache.open()`` hands out a slot, ``reserve`` grows it before a step,
``advance`` records the step's tokens, ``close`` gives everything back.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .slots import SlotList
from .spec import CacheFull, StoreSizes
from .stores import pages_for


@dataclass
class CacheLayout:
    """groups[g] = (spec, [owner layer indices]); where[layer] = (g, index in group)."""
    groups: List[Tuple[Any, List[int]]]
    where: Dict[int, Tuple[int, int]]

    @staticmethod
    def from_specs(specs: Sequence[Optional[Any]]) -> "CacheLayout":
        """``specs[i]`` is what layer i owns (None: nothing)."""
        groups: List[Tuple[Any, List[int]]] = []
        where: Dict[int, Tuple[int, int]] = {}
        for layer, spec in enumerate(specs):
            if spec is None:
                continue
            for g, (s, members) in enumerate(groups):
                if s == spec:
                    where[layer] = (g, len(members))
                    members.append(layer)
                    break
            else:
                where[layer] = (len(groups), 0)
                groups.append((spec, [layer]))
        return CacheLayout(groups, where)


class SequenceCache:
    def __init__(self, layout: CacheLayout, *, max_tokens: int, max_slots: int, max_seq_len: int,
                 dtype: torch.dtype, device, allocate: bool = True):
        if max_tokens <= 0 or max_slots <= 0 or max_seq_len <= 0:
            raise ValueError("max_tokens, max_slots and max_seq_len must be positive")
        self.layout = layout
        self.max_tokens = max_tokens
        self.max_seq_len = max_seq_len
        n_pages = pages_for(max_tokens)
        self.max_slots = min(max_slots, n_pages)
        self.slots = SlotList(self.max_slots)
        self.length: Dict[int, int] = {}
        self.stores: List[Any] = []
        self.sizes = StoreSizes(n_pages=n_pages, max_slots=self.max_slots,
                                max_pages_per_seq=min(pages_for(max_seq_len), n_pages),
                                max_seq_len=max_seq_len)
        for spec, members in layout.groups:
            if not callable(getattr(spec, "make_store", None)):
                raise TypeError(f"cache need {spec!r} has no make_store(n_layers, sizes, dtype, "
                                f"device, allocate)")
            self.stores.append(spec.make_store(len(members), self.sizes, dtype, device, allocate))

    # -- sequences ---------------------------------------------------------
    def open(self) -> int:
        slot = self.slots.acquire()
        for st in self.stores:
            st.open(slot)
        self.length[slot] = 0
        return slot

    def reserve(self, slot: int, new_tokens: int) -> None:
        """Room for ``new_tokens`` more tokens of the slot (call before the step)."""
        total = self._len(slot) + new_tokens
        if total > self.max_seq_len:
            raise CacheFull(f"sequence of {total} tokens exceeds max_seq_len={self.max_seq_len}")
        for st in self.stores:
            st.reserve(slot, total)

    def advance(self, slot: int, new_tokens: int) -> None:
        """Records that the step stored ``new_tokens`` tokens (call after the step)."""
        self.length[slot] = self._len(slot) + new_tokens
        for st in self.stores:
            st.trim(slot, self.length[slot])

    def close(self, slot: int) -> None:
        self._len(slot)
        for st in self.stores:
            st.close(slot)
        del self.length[slot]
        self.slots.release(slot)

    def _len(self, slot: int) -> int:
        if slot not in self.length:
            raise ValueError(f"slot {slot} is not open")
        return self.length[slot]

    def flush(self) -> None:
        for st in self.stores:
            st.flush()

    def view(self, layer: int):
        g, i = self.layout.where[layer]
        return self.stores[g].layer(i)

    def tokens_held(self) -> int:
        return max((st.tokens_held() for st in self.stores), default=0)

    def check(self) -> None:
        self.slots.check()
        if set(self.length) != set(self.slots.held()):
            raise AssertionError("open sequences and held slots differ")
        for st in self.stores:
            st.check()
