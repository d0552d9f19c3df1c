"""Counts and times of the steps of a run, the ``--profile`` report.

The reference's RunProfile (src/model.rs:1121-1209) keeps the number of prompt
and decode steps and their wall-clock totals; here the times are device times
between CUDA events around each step, read only when the report is made.
"""
from __future__ import annotations

from typing import List, Tuple

import torch


class StepProfile:
    def __init__(self):
        self.records: List[Tuple[str, int, int, torch.cuda.Event, torch.cuda.Event]] = []

    def begin(self):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    def end(self, kind: str, n_seqs: int, n_tokens: int, start) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.records.append((kind, n_seqs, n_tokens, start, ev))

    def report(self) -> str:
        torch.cuda.synchronize()
        rows = {}
        for kind, n_seqs, n_tokens, a, b in self.records:
            r = rows.setdefault(kind, [0, 0, 0.0])
            r[0] += 1
            r[1] += n_tokens
            r[2] += a.elapsed_time(b)
        lines = ["profile: kind     steps    tokens      ms   ms/step    tok/s"]
        for kind in sorted(rows):
            n, toks, ms = rows[kind]
            lines.append(f"         {kind:<8}{n:>6}{toks:>10}{ms:>8.2f}{ms / max(n, 1):>10.3f}"
                         f"{(toks / ms * 1e3 if ms > 0 else 0):>9.0f}")
        return "\n".join(lines)
