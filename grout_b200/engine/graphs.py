"""Steps as CUDA graphs: decode steps always, prompt steps of up to a thousand
tokens when every part of the model allows it.

A step is a few hundred short kernels; launched one by one the host cannot keep
up with the GPU (a prompt of 18 tokens costs three decode steps that way).  A
whole step (embedding to logits) is captured once per bucket of sizes and
replayed.  Everything that changes from step to step — tokens, slots,
positions, lengths, how rows divide into sequences — is read by the kernels
from one device buffer whose address is fixed and whose contents are refreshed
by a single copy before each replay; the cache's block tables and pages never
move.  Rows beyond the live ones carry slot -1 and store nothing.  (The
reference captures its single-sequence decode step the same way,
src/model.rs:3118-3647, feeds it a position by a 4-byte copy, 363-400, and keeps
one graph per sequence length, 2310-2318.)

Buckets.  A decode step of B sequences runs in the graph of (2^k >= B, L), L
being the power of two, at least 512, that bounds the longest sequence after the
step: it is what ``step.max_kv_len`` says in the capture, so a mixer that sizes
its work by the longest sequence (the split of decode attention over the keys)
sizes it for the sequences that are there and not for the longest the cache
could hold.  A prompt step runs in the graph of (tokens, sequences, wanted
rows), each rounded up to a power of two; rows left over form one padding
sequence, sequences left over have no rows.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import numpy as np
import torch

from .batch import context_from, layout_sizes, pack_step_padded

PROMPT_TOKENS_MOST = 1024       # longer prompt steps are bound by the device, not by launches
PROMPT_SEQS_MOST = 64
PROMPT_TOKENS_LEAST = 16
PROMPT_GRAPHS_MOST = 48         # captured prompt shapes kept; further shapes run launch by launch
PROMPT_LOGITS_MOST = 2 << 30    # bytes of logits the captured prompt shapes may hold between them
LENGTH_LEAST = 512


def bucket_for(n: int, largest: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b if b <= largest else 0


def length_bucket(n: int, most: int, least: int = LENGTH_LEAST) -> int:
    """The bound on the longest sequence that a decode graph is captured for: the
    power of two >= n, at least ``least``, at most ``most`` (the cache's limit)."""
    b = least
    while b < n:
        b *= 2
    return min(b, most)


def prompt_bucket(n_tokens: int, n_seqs: int, n_want: int) -> Optional[Tuple[int, int, int]]:
    """(tokens, sequences, wanted rows) of the graph a prompt step runs in, or None
    when it is too large for one.  A step whose rows do not fill the bucket needs
    one sequence more, for the padding rows."""
    tb = bucket_for(n_tokens, PROMPT_TOKENS_MOST)
    if not tb:
        return None
    tb = max(tb, PROMPT_TOKENS_LEAST)
    sb = bucket_for(n_seqs + (1 if n_tokens < tb else 0), PROMPT_SEQS_MOST)
    wb = bucket_for(n_want, tb) if n_want else 0
    if not sb or (n_want and not wb):
        return None
    return tb, sb, wb


class StepGraph:
    """One captured step of fixed sizes.  Subclasses fill the staging buffer."""

    def __init__(self, model, cache, device, pool, *, n_tokens: int, n_seqs: int, n_want: int,
                 decode: bool, max_kv_len: int):
        self.model, self.cache, self.device, self.pool = model, cache, device, pool
        self.n_tokens, self.n_seqs, self.n_want = n_tokens, n_seqs, n_want
        self.decode, self.max_kv_len = decode, max_kv_len
        self.off, total = layout_sizes(n_tokens, n_seqs, n_want)
        # pinned staging buffers in a ring: a buffer is rewritten only after the
        # copy that read it has finished, so steps may be queued without a sync
        self.staging = [torch.zeros(total, dtype=torch.int32).pin_memory() for _ in range(4)]
        self.copied = [None] * len(self.staging)
        self.turn = 0
        self.views = []
        for st in self.staging:          # numpy views of every array of the layout
            flat = st.numpy()
            self.views.append({name: flat[o:o + cnt] for name, (o, cnt) in self.off.items()})
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)
        self.graph = None
        self.logits = None
        self.kernels_per_replay = 0

    def _next_staging(self) -> int:
        k = self.turn
        self.turn = (k + 1) % len(self.staging)
        if self.copied[k] is not None:
            self.copied[k].synchronize()
        return k

    def _send(self, k: int) -> None:
        self.dev.copy_(self.staging[k], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.copied[k] = ev

    def _fill_padding(self) -> None:
        raise NotImplementedError

    def _capture(self) -> None:
        """Warm-up with padding rows only (which store nothing), then capture."""
        self._fill_padding()
        meta = dict(n_tokens=self.n_tokens, n_seqs=self.n_seqs, n_want=self.n_want, off=self.off,
                    q_lens=(), starts=(), slot_list=(), decode=self.decode,
                    max_q_len=1 if self.decode else self.n_tokens,
                    # bounds that kernels size their launches with must hold for every replay
                    max_kv_len=self.max_kv_len)
        step = context_from(self.dev, meta)
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.model.forward(step, self.cache)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.current_stream().synchronize()
        from ..kernels import ops
        before = ops.launch_count()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, pool=self.pool):
            self.logits = self.model.forward(step, self.cache)
        self.kernels_per_replay = ops.launch_count() - before   # this library's kernels in the graph
        self.graph = g


class DecodeGraph(StepGraph):
    def __init__(self, model, cache, n_seqs: int, device, pool=None, max_kv_len: Optional[int] = None):
        super().__init__(model, cache, device, pool, n_tokens=n_seqs, n_seqs=n_seqs, n_want=n_seqs,
                         decode=True, max_kv_len=max_kv_len or cache.max_seq_len)
        self.n = n_seqs
        for v in self.views:             # what is constant for a bucket is filled once
            v["token_seq"][:] = np.arange(n_seqs, dtype=np.int32)
            v["cu_q"][:] = np.arange(n_seqs + 1, dtype=np.int32)
            v["want_rows"][:] = np.arange(n_seqs, dtype=np.int32)

    def _fill(self, entries) -> None:
        """Writes the live sequences plus padding rows into a staging buffer and
        copies it to the device.  Every row's logits are computed: the head reads
        its weights once anyway.  Only what changes from step to step (tokens,
        slots, positions, lengths) is rewritten."""
        n_real = len(entries)
        k = self._next_staging()
        out = self.views[k]
        starts = [e[1] for e in entries]
        out["tokens"][:n_real] = [e[2][0] for e in entries]
        out["tokens"][n_real:] = 0
        out["token_pos"][:n_real] = starts
        out["token_pos"][n_real:] = 0
        out["slots"][:n_real] = [e[0] for e in entries]
        out["slots"][n_real:] = -1
        out["kv_len"][:n_real] = starts
        out["kv_len"][:n_real] += 1
        out["kv_len"][n_real:] = 1
        self._send(k)

    def _fill_padding(self) -> None:
        self._fill([])

    def run(self, entries, tokens_from=None) -> torch.Tensor:
        """entries: (slot, start, [token]) of the live sequences, at most n.
        Returns logits [n, vocab]; rows beyond the live sequences are padding.
        The tensor is the graph's own and the next replay rewrites it.
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


class PromptGraph(StepGraph):
    def __init__(self, model, cache, device, pool, n_tokens: int, n_seqs: int, n_want: int):
        super().__init__(model, cache, device, pool, n_tokens=n_tokens, n_seqs=n_seqs,
                         n_want=n_want, decode=False, max_kv_len=cache.max_seq_len)

    def _fill(self, entries, want) -> int:
        buf, meta = pack_step_padded(entries, want, self.n_tokens, self.n_seqs, self.n_want)
        k = self._next_staging()
        self.staging[k].numpy()[:] = buf
        self._send(k)
        return meta["n_real_want"]

    def _fill_padding(self) -> None:
        self._fill([], None)

    def run(self, entries, want) -> Optional[torch.Tensor]:
        """entries: (slot, start, tokens); want: wanted places per entry.  Returns
        the wanted rows' logits (a view of the graph's own buffer, which the next
        replay rewrites) or None when nothing was wanted."""
        if self.graph is None:
            self._capture()
        n_real_want = self._fill(entries, want)
        self.graph.replay()
        return self.logits[:n_real_want] if n_real_want else None


class StepGraphs:
    """The captured steps of one engine.  All graphs draw their buffers from one
    memory pool: they run one after the other on one stream and keep nothing
    between replays but their logits, which stay allocated."""

    def __init__(self, model, cache, device, largest: int = 256):
        self.model, self.cache, self.device, self.largest = model, cache, device, largest
        self.decode_graphs: Dict[Tuple[int, int], DecodeGraph] = {}
        self.prompt_graphs: Dict[Tuple[int, int, int], PromptGraph] = {}
        self._prompt_logits_bytes = 0
        self._pool = None
        self._prompts_ok: Optional[bool] = None

    def pool(self):
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        return self._pool

    def decode(self, n_live: int, longest: int) -> Optional[DecodeGraph]:
        """The graph for ``n_live`` sequences of which the longest holds ``longest``
        tokens after the step; None beyond the largest bucket."""
        b = bucket_for(n_live, self.largest)
        if not b:
            return None
        key = (b, length_bucket(longest, self.cache.max_seq_len))
        g = self.decode_graphs.get(key)
        if g is None:
            g = self.decode_graphs[key] = DecodeGraph(self.model, self.cache, b, self.device,
                                                      self.pool(), key[1])
        return g

    def prompt(self, n_tokens: int, n_seqs: int, n_want: int) -> Optional[PromptGraph]:
        """The graph for a prompt step of these sizes, or None: the model has a
        part that does not allow it, the step is too large, or too many shapes
        have been captured already."""
        if self._prompts_ok is None:
            self._prompts_ok = bool(self.model.captures_prompts())
        key = prompt_bucket(n_tokens, n_seqs, n_want) if self._prompts_ok else None
        if key is None:
            return None
        g = self.prompt_graphs.get(key)
        if g is None:
            # every captured shape keeps its logits [wanted rows, vocabulary] allocated
            held = 4 * key[2] * self.model.plan.vocab_size
            if len(self.prompt_graphs) >= PROMPT_GRAPHS_MOST or \
                    self._prompt_logits_bytes + held > PROMPT_LOGITS_MOST:
                return None
            self._prompt_logits_bytes += held
            g = self.prompt_graphs[key] = PromptGraph(self.model, self.cache, self.device,
                                                      self.pool(), *key)
        return g
