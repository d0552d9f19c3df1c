"""The decode step as a CUDA graph, one per batch-size bucket.

A decode step is a few hundred short kernels; launched one by one the host
cannot keep up with the GPU.  The whole step (embedding to logits) is captured
once per bucket and replayed.  Everything that changes from step to step —
tokens, slots, positions, lengths — is read by the kernels from one device
buffer whose address is fixed and whose contents are refreshed by a single copy
before each replay; the cache's block tables and pages never move.  Rows beyond
the live sequences carry slot -1 and store nothing.  (The reference captures its
single-sequence decode step the same way, src/model.rs:3118-3647, and feeds it
a position by a 4-byte copy, 363-400.)
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch

from .batch import context_from, layout_sizes


def bucket_for(n: int, largest: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b if b <= largest else 0


class DecodeGraph:
    def __init__(self, model, cache, n_seqs: int, device):
        self.model, self.cache, self.n, self.device = model, cache, n_seqs, device
        off, total = layout_sizes(n_seqs, n_seqs, n_seqs)
        # pinned staging buffers in a ring: a buffer is rewritten only after the
        # copy that read it has finished, so steps may be queued without a sync
        self.staging = [torch.zeros(total, dtype=torch.int32).pin_memory() for _ in range(4)]
        self.copied = [None] * len(self.staging)
        self.turn = 0
        self.off = off
        self.views = []
        for st in self.staging:          # numpy views of every array of the layout
            flat = st.numpy()
            v = {name: flat[o:o + cnt] for name, (o, cnt) in off.items()}
            v["token_seq"][:] = np.arange(n_seqs, dtype=np.int32)
            v["cu_q"][:] = np.arange(n_seqs + 1, dtype=np.int32)
            v["want_rows"][:] = np.arange(n_seqs, dtype=np.int32)
            self.views.append(v)
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)
        self.graph = None
        self.logits = None
        self.kernels_per_replay = 0

    def _fill(self, entries) -> dict:
        """Writes the live sequences plus padding rows into a staging buffer and
        copies it to the device.  Every row's logits are computed: the head reads
        its weights once anyway.  Only what changes from step to step (tokens,
        slots, positions, lengths) is rewritten; the rest of the layout is constant
        for a bucket and was filled when the buffer was made."""
        n_real = len(entries)
        k = self.turn
        self.turn = (k + 1) % len(self.staging)
        if self.copied[k] is not None:
            self.copied[k].synchronize()
        out = self.views[k]
        n = self.n
        slots = [e[0] for e in entries]
        starts = [e[1] for e in entries]
        out["tokens"][:n_real] = [e[2][0] for e in entries]
        out["tokens"][n_real:] = 0
        out["token_pos"][:n_real] = starts
        out["token_pos"][n_real:] = 0
        out["slots"][:n_real] = slots
        out["slots"][n_real:] = -1
        out["kv_len"][:n_real] = starts
        out["kv_len"][:n_real] += 1
        out["kv_len"][n_real:] = 1
        self.dev.copy_(self.staging[k], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.copied[k] = ev
        return dict(n_tokens=n, n_seqs=n, n_want=n, off=self.off, q_lens=(1,) * n,
                    starts=tuple(starts) + (0,) * (n - n_real),
                    slot_list=tuple(slots) + (-1,) * (n - n_real), decode=True, max_q_len=1,
                    max_kv_len=max(starts, default=0) + 1)

    def _capture(self) -> None:
        """Warm-up with padding rows only (which store nothing), then capture."""
        meta = self._fill([])
        step = context_from(self.dev, meta)
        # bounds that kernels size their launches with must hold for every replay
        step.max_kv_len = self.cache.max_seq_len
        step.q_lens = step.starts = step.slot_list = ()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.model.forward(step, self.cache)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.current_stream().synchronize()
        from ..kernels import ops
        before = ops.launch_count()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.logits = self.model.forward(step, self.cache)
        self.kernels_per_replay = ops.launch_count() - before   # this library's kernels in the graph
        self.graph = g

    def run(self, entries, tokens_from=None) -> torch.Tensor:
        """entries: (slot, start, [token]) of the live sequences, at most n.
        Returns logits [n, vocab]; rows beyond the live sequences are padding.
        ``tokens_from`` = (int32 device tensor, rows): the token of entry k is
        ``tensor[rows[k]]``, copied on the device after the staging copy, so that
        the step can be queued before the host has seen the tokens."""
        if self.graph is None:
            self._capture()
        self._fill(entries)
        if tokens_from is not None:
            chosen, rows = tokens_from
            o, _cnt = self.off["tokens"]
            dst = self.dev[o:o + len(rows)]
            if list(rows) == list(range(len(rows))):
                dst.copy_(chosen[:len(rows)], non_blocking=True)
            else:
                idx = torch.tensor(list(rows), device=self.device)
                torch.index_select(chosen, 0, idx, out=dst)
        self.graph.replay()
        return self.logits


class DecodeGraphs:
    def __init__(self, model, cache, device, largest: int = 256):
        self.model, self.cache, self.device, self.largest = model, cache, device, largest
        self.graphs: Dict[int, DecodeGraph] = {}

    def get(self, n_live: int):
        b = bucket_for(n_live, self.largest)
        if not b:
            return None
        g = self.graphs.get(b)
        if g is None:
            g = self.graphs[b] = DecodeGraph(self.model, self.cache, b, self.device)
        return g
