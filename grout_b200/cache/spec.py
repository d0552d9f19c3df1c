"""What a layer asks of the cache.

A need is a frozen (hashable, comparable) object with one method,
``make_store(n_layers, sizes, dtype, device, allocate)``, which returns the
storage for a group of ``n_layers`` layers that all have this need.  Layers
whose needs compare equal share a store.  A store has the methods of
``stores.Store``: ``open``, ``reserve``, ``trim``, ``close``, ``flush``,
``tokens_held``, ``layer(index)`` (what the layer's part is handed as its
``cache`` argument) and ``check``.  The cache itself knows no kind of need: a
mixer that keeps something else (keys and values of different widths, a
compressed latent) brings its own spec and store.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

PAGE_TOKENS = 64   # tokens per page of a key/value store; requests hold whole pages


@dataclass(frozen=True)
class StoreSizes:
    """The limits a cache was built with, handed to every ``make_store``."""
    n_pages: int               # pages of PAGE_TOKENS tokens in a paged store
    max_slots: int             # sequences alive at once
    max_pages_per_seq: int     # pages of the longest sequence
    max_seq_len: int


@dataclass(frozen=True)
class KVSpec:
    """Keys and values of ``n_kv_heads`` heads of ``head_dim`` for every token
    (``window`` None) or for the last ``window`` tokens."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def make_store(self, n_layers: int, sizes: StoreSizes, dtype, device, allocate: bool = True):
        from .stores import KVStore
        return KVStore(self, n_layers, sizes.n_pages, sizes.max_slots, sizes.max_pages_per_seq,
                       dtype, device, allocate)


@dataclass(frozen=True)
class StateSpec:
    """Per-sequence state of fixed size: one tensor of ``shape`` per sequence and
    layer, zero when the sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32

    def make_store(self, n_layers: int, sizes: StoreSizes, dtype, device, allocate: bool = True):
        from .stores import StateStore
        return StateStore(self, n_layers, sizes.max_slots, device, allocate)


class CacheFull(RuntimeError):
    """No free slot or page is left."""
