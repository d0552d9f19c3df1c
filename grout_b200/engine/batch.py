"""The description of one step that every part receives.

A step runs the tokens it is given and nothing else: for each sequence of the
batch its next ``q_len`` tokens, which continue the ``start`` tokens that the
cache already holds for its slot.  Sequences are packed one after the other
("varlen"): row t of every activation belongs to sequence ``token_seq[t]`` and
has absolute position ``token_pos[t]``.

All arrays live in one int32 device buffer that is filled by a single
host-to-device copy.  In a captured decode graph the buffer's address is fixed
and only its contents change, so parts must read sizes that vary from step to
step (positions, lengths, slots) from the device arrays, never from the host
fields, which describe the step the graph was captured with.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class StepContext:
    n_tokens: int                 # rows of every activation in this step
    n_seqs: int                   # sequences, padding rows included
    tokens: torch.Tensor          # int32 [n_tokens]
    token_seq: torch.Tensor       # int32 [n_tokens]   index into slots
    token_pos: torch.Tensor       # int32 [n_tokens]   absolute position
    cu_q: torch.Tensor            # int32 [n_seqs + 1] first row of each sequence
    slots: torch.Tensor           # int32 [n_seqs]     cache slot, -1 for padding
    kv_len: torch.Tensor          # int32 [n_seqs]     tokens held after this step
    want_rows: Optional[torch.Tensor]   # int32 [n_want] rows whose logits are asked for
    n_want: int
    decode: bool                  # every sequence brings exactly one token
    max_q_len: int
    max_kv_len: int               # upper bound of kv_len (host knowledge)
    # host copies, valid for eager steps only (empty in a captured step)
    q_lens: Tuple[int, ...] = ()
    starts: Tuple[int, ...] = ()
    slot_list: Tuple[int, ...] = ()

    def q_blocks(self, rows: int) -> int:
        """How many blocks of ``rows`` query rows the step's sequences make, each
        sequence starting a block of its own: the exact count when the host knows
        the lengths, else (a captured step, whose lengths change from replay to
        replay) the most that ``n_tokens`` rows in ``n_seqs`` sequences can make.
        A kernel sizes its grid with it and finds each block's sequence from
        ``cu_q`` on the device; blocks beyond the real count find none."""
        if self.q_lens:
            return sum((n + rows - 1) // rows for n in self.q_lens)
        return self.n_tokens // rows + self.n_seqs


def layout_sizes(n_tokens: int, n_seqs: int, n_want: int):
    """Offsets of the arrays inside the step's int32 buffer."""
    off, o = {}, 0
    for name, n in (("tokens", n_tokens), ("token_seq", n_tokens), ("token_pos", n_tokens),
                    ("cu_q", n_seqs + 1), ("slots", n_seqs), ("kv_len", n_seqs),
                    ("want_rows", n_want)):
        off[name] = (o, n)
        o += n
    return off, o


def pack_step(entries: Sequence[Tuple[int, int, Sequence[int]]],
              want: Optional[Sequence[Sequence[int]]], pad_seqs: int = 0):
    """entries: (slot, start, tokens) per sequence; want: per sequence the places
    among its tokens whose logits are asked for.  ``pad_seqs`` appends sequences
    of one token with slot -1, which compute nothing that is kept.
    Returns (flat int32 array, meta dict)."""
    n_real = len(entries)
    q_lens = [len(e[2]) for e in entries] + [1] * pad_seqs
    n_seqs = n_real + pad_seqs
    n_tokens = sum(q_lens)
    want = [list(w) for w in want] if want is not None else [[] for _ in entries]
    if len(want) != n_real:
        raise ValueError("one list of wanted places per entry is needed")
    n_want = sum(len(w) for w in want)
    off, total = layout_sizes(n_tokens, n_seqs, n_want)
    buf = np.zeros(total, dtype=np.int32)
    cu = np.zeros(n_seqs + 1, dtype=np.int64)
    cu[1:] = np.cumsum(q_lens)
    slots = [e[0] for e in entries] + [-1] * pad_seqs
    starts = [e[1] for e in entries] + [0] * pad_seqs
    o = off["tokens"][0]
    for i, (_slot, _start, toks) in enumerate(entries):
        buf[o + cu[i]: o + cu[i + 1]] = np.asarray(toks, dtype=np.int64)
    seq = np.repeat(np.arange(n_seqs, dtype=np.int32), q_lens)
    buf[off["token_seq"][0]: off["token_seq"][0] + n_tokens] = seq
    pos = np.arange(n_tokens, dtype=np.int64) - cu[:-1][seq] + np.asarray(starts, dtype=np.int64)[seq]
    buf[off["token_pos"][0]: off["token_pos"][0] + n_tokens] = pos
    buf[off["cu_q"][0]: off["cu_q"][0] + n_seqs + 1] = cu
    buf[off["slots"][0]: off["slots"][0] + n_seqs] = slots
    buf[off["kv_len"][0]: off["kv_len"][0] + n_seqs] = np.asarray(starts) + np.asarray(q_lens)
    rows = []
    for i, w in enumerate(want):
        for p in w:
            if not 0 <= p < q_lens[i]:
                raise ValueError(f"wanted place {p} is outside the {q_lens[i]} tokens of entry {i}")
            rows.append(int(cu[i]) + p)
    buf[off["want_rows"][0]: off["want_rows"][0] + n_want] = rows
    meta = dict(n_tokens=n_tokens, n_seqs=n_seqs, n_want=n_want, off=off, q_lens=tuple(q_lens),
                starts=tuple(starts), slot_list=tuple(slots),
                decode=all(q == 1 for q in q_lens),
                max_q_len=max(q_lens) if q_lens else 0,
                max_kv_len=max((s + q for s, q in zip(starts, q_lens)), default=0))
    return buf, meta


def pack_step_padded(entries: Sequence[Tuple[int, int, Sequence[int]]],
                     want: Optional[Sequence[Sequence[int]]], n_tokens: int, n_seqs: int,
                     n_want: int):
    """The same layout filled up to fixed sizes, for a step that replays a captured
    graph: after the real sequences comes, if rows are left, one padding sequence
    (slot -1, positions from 0) that takes all of them, then sequences without
    rows; the list of wanted rows is filled up with row 0.  Raises ValueError when
    the entries do not fit."""
    real_tokens = sum(len(e[2]) for e in entries)
    filler = n_tokens - real_tokens
    want = [list(w) for w in want] if want is not None else [[] for _ in entries]
    real_want = sum(len(w) for w in want)
    if filler < 0 or len(entries) + (1 if filler else 0) > n_seqs or real_want > n_want:
        raise ValueError(f"{len(entries)} sequences with {real_tokens} tokens and {real_want} "
                         f"wanted rows do not fit a step of {n_seqs} / {n_tokens} / {n_want}")
    padded = list(entries) + ([(-1, 0, [0] * filler)] if filler else [])
    empty = n_seqs - len(padded)
    buf, meta = pack_step(padded, want + [[] for _ in range(len(padded) - len(entries))])
    off, total = layout_sizes(n_tokens, n_seqs, n_want)
    out = np.zeros(total, dtype=np.int32)
    for name, (o, cnt) in meta["off"].items():
        out[off[name][0]: off[name][0] + cnt] = buf[o:o + cnt]
    n_in = len(padded)
    o = off["cu_q"][0]
    out[o + n_in + 1: o + n_seqs + 1] = n_tokens           # sequences without rows
    o = off["slots"][0]
    out[o + n_in: o + n_seqs] = -1
    meta = dict(meta, off=off, n_seqs=n_seqs, n_want=n_want, n_real_want=real_want,
                q_lens=meta["q_lens"] + (0,) * empty, starts=meta["starts"] + (0,) * empty,
                slot_list=meta["slot_list"] + (-1,) * empty)
    return out, meta


def context_from(dev_buf: torch.Tensor, meta: dict) -> StepContext:
    """Views of the device buffer as a StepContext."""
    off = meta["off"]

    def view(name):
        o, n = off[name]
        return dev_buf[o:o + n]

    return StepContext(
        n_tokens=meta["n_tokens"], n_seqs=meta["n_seqs"], tokens=view("tokens"),
        token_seq=view("token_seq"), token_pos=view("token_pos"), cu_q=view("cu_q"),
        slots=view("slots"), kv_len=view("kv_len"),
        want_rows=view("want_rows") if meta["n_want"] else None, n_want=meta["n_want"],
        decode=meta["decode"], max_q_len=meta["max_q_len"], max_kv_len=meta["max_kv_len"],
        q_lens=meta["q_lens"], starts=meta["starts"], slot_list=meta["slot_list"])


def make_context(entries, want, device, pad_seqs: int = 0) -> StepContext:
    buf, meta = pack_step(entries, want, pad_seqs)
    dev = torch.from_numpy(buf).to(device)
    return context_from(dev, meta)
