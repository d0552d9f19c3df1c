"""The uniform numbers that sampling consumes: one stream per request, made on
the host from the request's seed, one number per generated token.  Keeping the
draws outside the kernel makes a sampled run repeatable from its seed alone and
lets a plain implementation be fed the very same numbers."""
from __future__ import annotations

import numpy as np


class DrawStream:
    def __init__(self, seed: int, index: int = 0):
        self._gen = np.random.Generator(np.random.Philox(key=[int(seed) & (2**64 - 1), int(index)]))

    def next(self) -> float:
        """A float32 in [0, 1)."""
        return float(np.float32(self._gen.random(dtype=np.float32)))
