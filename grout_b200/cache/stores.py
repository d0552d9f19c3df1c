"""Device storage of the cache, one store per group of layers with the same needs.

``KVStore``: keys and values in pages of ``PAGE_TOKENS`` tokens,
``[layers, pages, kv heads, PAGE_TOKENS, head_dim]``, with one block table
``[slots, pages per sequence]`` shared by the group's layers.  Pointers never
change after construction, so a captured CUDA graph stays valid.  Pages are
zero-filled once and never cleared again: a sequence's length gates every read.  (The reference keeps one
``[kv heads, S, D]`` pair per layer for its single sequence,
src/model.rs:1450-1455.)  A store with a window gives pages back as soon as
every token in them has left the window of all later queries.

``StateStore``: ``[layers, slots + 1, *shape]`` of fixed-size state, zeroed when a
slot is opened; the last row belongs to no sequence and is where padding rows
(slot -1) may be pointed, so that a mixer needs no branch for them (the reference's packed backend keeps such state per layer,
src/quantized.rs:160-169, 376-410).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from .slots import PagePool
from .spec import CacheFull, KVSpec, PAGE_TOKENS, StateSpec


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


@dataclass
class KVLayerView:
    """What an attention layer sees of its store."""
    k_pages: torch.Tensor        # [pages, kv heads, PAGE_TOKENS, head_dim]
    v_pages: torch.Tensor
    block_table: torch.Tensor    # int32 [slots, pages per sequence]
    page: int
    spec: KVSpec


@dataclass
class StateLayerView:
    state: torch.Tensor          # [slots + 1, *shape]; the last row is for padding rows
    spec: StateSpec


class KVStore:
    def __init__(self, spec: KVSpec, n_layers: int, n_pages: int, max_slots: int,
                 max_pages_per_seq: int, dtype: torch.dtype, device, allocate: bool = True):
        self.spec, self.n_layers = spec, n_layers
        self.n_pages, self.max_slots, self.max_pages_per_seq = n_pages, max_slots, max_pages_per_seq
        self.pool = PagePool(n_pages)
        self.table_host = np.zeros((max_slots, max_pages_per_seq), dtype=np.int32)
        self.pages_of: Dict[int, List[Optional[int]]] = {}
        self._dirty: Dict[int, int] = {}    # slot -> first table entry not yet on the device
        self.device = torch.device(device)
        self.k = self.v = self.table_dev = None
        if allocate:
            shape = (n_layers, max(n_pages, 1), spec.n_kv_heads, PAGE_TOKENS, spec.head_dim)
            # zero-filled once: rows beyond a sequence's length are masked by every
            # kernel, but a tensor-core product of probability 0 with a NaN that
            # happened to be in fresh memory would still be NaN
            self.k = torch.zeros(shape, dtype=dtype, device=self.device)
            self.v = torch.zeros(shape, dtype=dtype, device=self.device)
            self.table_dev = torch.zeros((max_slots, max_pages_per_seq), dtype=torch.int32,
                                         device=self.device)

    # -- sequences ---------------------------------------------------------
    def open(self, slot: int) -> None:
        if slot in self.pages_of:
            raise ValueError(f"slot {slot} is already open in this store")
        self.pages_of[slot] = []

    def reserve(self, slot: int, n_tokens: int) -> None:
        """Makes sure pages exist for tokens 0..n_tokens-1 of the slot."""
        pages = self.pages_of[slot]
        need = pages_for(n_tokens)
        if need > self.max_pages_per_seq:
            raise CacheFull(f"{n_tokens} tokens exceed the longest sequence this cache was "
                            f"built for ({self.max_pages_per_seq * PAGE_TOKENS})")
        if need > len(pages):
            first = len(pages)
            new = self.pool.acquire_many(need - len(pages))
            pages.extend(new)
            self.table_host[slot, first:need] = new
            self._dirty[slot] = min(self._dirty.get(slot, first), first)

    def trim(self, slot: int, length: int) -> None:
        """With a window: frees pages whose tokens no query at position >= length
        can see any more (all their positions are <= length - window)."""
        w = self.spec.window
        if w is None:
            return
        pages = self.pages_of[slot]
        dead = max(0, length - w + 1) // PAGE_TOKENS   # pages [0, dead) are out of reach
        for i in range(min(dead, len(pages))):
            if pages[i] is not None:
                self.pool.release(pages[i])
                pages[i] = None

    def close(self, slot: int) -> None:
        for p in self.pages_of.pop(slot):
            if p is not None:
                self.pool.release(p)
        self._dirty.pop(slot, None)

    def tokens_held(self) -> int:
        return self.pool.n_held * PAGE_TOKENS

    # -- device ------------------------------------------------------------
    def flush(self) -> None:
        """Brings the device's block table up to date (before a step)."""
        if self.table_dev is None:
            self._dirty.clear()
            return
        for slot, first in self._dirty.items():
            n = len(self.pages_of.get(slot, ()))
            if n > first:
                self.table_dev[slot, first:n].copy_(torch.from_numpy(self.table_host[slot, first:n]))
        self._dirty.clear()

    def layer(self, index: int) -> KVLayerView:
        return KVLayerView(self.k[index], self.v[index], self.table_dev, PAGE_TOKENS, self.spec)

    def check(self) -> None:
        self.pool.check()
        listed = [p for pages in self.pages_of.values() for p in pages if p is not None]
        if len(listed) != len(set(listed)):
            raise AssertionError("a page belongs to two sequences")
        if set(listed) != set(self.pool.held()):
            raise AssertionError("held pages and the sequences' pages differ")


class StateStore:
    def __init__(self, spec: StateSpec, n_layers: int, max_slots: int, device, allocate: bool = True):
        self.spec, self.n_layers, self.max_slots = spec, n_layers, max_slots
        self.device = torch.device(device)
        self.state = None
        self.open_slots = set()
        if allocate:
            self.state = torch.zeros((n_layers, max_slots + 1) + tuple(spec.shape),
                                     dtype=spec.dtype, device=self.device)

    def open(self, slot: int) -> None:
        if slot in self.open_slots:
            raise ValueError(f"slot {slot} is already open in this store")
        self.open_slots.add(slot)
        if self.state is not None:
            self.state[:, slot].zero_()

    def reserve(self, slot: int, n_tokens: int) -> None:
        pass

    def trim(self, slot: int, length: int) -> None:
        pass

    def close(self, slot: int) -> None:
        self.open_slots.remove(slot)

    def flush(self) -> None:
        pass

    def tokens_held(self) -> int:
        return 0

    def layer(self, index: int) -> StateLayerView:
        return StateLayerView(self.state[index], self.spec)

    def check(self) -> None:
        pass
