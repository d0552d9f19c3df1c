"""What a layer asks of the cache."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

PAGE_TOKENS = 64   # tokens per page of a key/value store; requests hold whole pages


@dataclass(frozen=True)
class KVSpec:
    """Keys and values of ``n_kv_heads`` heads of ``head_dim`` for every token
    (``window`` None) or for the last ``window`` tokens."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """Per-sequence state of fixed size: one tensor of ``shape`` per sequence and
    layer, zero when the sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class CacheFull(RuntimeError):
    """No free slot or page is left."""
