"""The generation loop above the step function.

Requests are served batch after batch.  The requests of a batch start together:
their prompts, of unequal lengths, go through one step; then every live request
brings one token per step.  A request ends when it draws a stop token (which is
neither returned nor fed back, as in the reference, src/model.rs:2063,
2086-2089) or reaches its budget; it then leaves the batch, its slot and pages
are given back at once, and the others go on.  When a batch is done the next
one starts, reusing what was given back.

The loop talks to the model only through ``open_sequence`` / ``step`` /
``close_sequence`` and a chooser, so its decisions can be tested with a scripted
stand-in and no GPU.  (The reference's loop is ``Qwen3Engine::generate``,
src/model.rs:1979-2196, for one request.)

Looking ahead.  Reading a step's tokens on the host and only then queueing the
next step leaves the GPU idle for the host's share of a step.  A stepper that
offers ``can_step_ahead(n)`` and ``step_ahead(entries, chosen)`` lets the loop
queue the next step first, its input tokens taken on the device from the chosen
tokens of this one, and read the tokens while it runs.  Who goes on is then
decided before the tokens are known: a request that has budget left takes part
in the next step, and if its token turns out to be a stop token that step was
run for nothing for its row (its slot is given back as usual, and nothing of the
row is returned).  In the 32-bit path the tokens that come back are the same
either way: no kernel's order of sums depends on how many rows a step has.  In
bfloat16 the row that ran for nothing can put that step into the next bucket of
rows (17 rows instead of 16), whose products cut their sums differently; the
other rows' logits then differ by rounding, and a near-tie between two tokens
may fall the other way.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

from ..cache.spec import PAGE_TOKENS
from ..sampling.draws import DrawStream
from ..sampling.params import SamplingParams


@dataclass
class Request:
    prompt: Sequence[int]
    max_new_tokens: int = 128                     # the reference's default, src/main.rs:26
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: Tuple[int, ...] = ()
    include_stop: bool = False                    # return the stop token too


@dataclass
class GenerationOutput:
    """Per request, the fields of the reference's GenerationOutput
    (src/model.rs:1251-1289) that do not need a tokenizer."""
    token_ids: List[int]
    prompt_tokens: int
    generated_tokens: int
    finish_reason: str                            # "stop" | "length"
    prompt_elapsed: float = 0.0                   # seconds, of the request's batch
    decode_elapsed: float = 0.0
    total_elapsed: float = 0.0
    text: Optional[str] = None

    def prompt_tps(self) -> float:
        return self.prompt_tokens / self.prompt_elapsed if self.prompt_elapsed > 0 else 0.0

    def decode_phase_tps(self) -> float:
        n = max(self.generated_tokens - 1, 0)
        return n / self.decode_elapsed if self.decode_elapsed > 0 else 0.0

    def total_tps(self) -> float:
        return self.generated_tokens / self.total_elapsed if self.total_elapsed > 0 else 0.0


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def validate(requests: Sequence[Request], max_seq_len: int, vocab: int) -> None:
    for i, r in enumerate(requests):
        if len(r.prompt) == 0:
            raise ValueError(f"request {i}: the prompt has no tokens")           # src/model.rs:1992
        if r.max_new_tokens < 0:
            raise ValueError(f"request {i}: max_new_tokens is negative")
        if len(r.prompt) + r.max_new_tokens > max_seq_len:
            raise ValueError(f"request {i}: {len(r.prompt)} prompt + {r.max_new_tokens} new tokens "
                             f"exceed max_seq_len={max_seq_len}")                # src/model.rs:1995
        bad = [t for t in r.prompt if not 0 <= int(t) < vocab]
        if bad:
            raise ValueError(f"request {i}: token {bad[0]} is outside the vocabulary of {vocab}")


def plan_batches(requests: Sequence[Request], max_batch: int, max_tokens: int) -> List[List[int]]:
    """Requests in their order, cut into batches that fit: at most ``max_batch``
    sequences, and the tokens they may come to hold (prompt + budget, each
    rounded up to whole pages) within ``max_tokens``."""
    batches: List[List[int]] = []
    cur: List[int] = []
    held = 0
    for i, r in enumerate(requests):
        if r.max_new_tokens == 0:
            continue
        need = _round_up(len(r.prompt) + r.max_new_tokens, PAGE_TOKENS)
        if need > max_tokens:
            raise ValueError(f"request {i} needs room for {need} tokens; the cache holds {max_tokens}")
        if cur and (len(cur) >= max_batch or held + need > max_tokens):
            batches.append(cur)
            cur, held = [], 0
        cur.append(i)
        held += need
    if cur:
        batches.append(cur)
    return batches


class GenerationLoop:
    """stepper: has open_sequence(), close_sequence(slot), step(entries, want);
    choose(logits, params, draws) -> one token per row (anything indexable by row
    whose items convert with int())."""

    def __init__(self, stepper, choose: Callable, *, max_batch: int, max_tokens: int,
                 max_seq_len: int, vocab_size: int, clock: Callable[[], float] = time.perf_counter,
                 sync: Callable[[], None] = lambda: None, choose_ahead: Optional[Callable] = None):
        """``choose_ahead(logits, params, draws)``: like ``choose`` but returns at
        once with a handle ``h`` for which ``stepper.step_ahead(entries, h)`` can take
        its tokens and ``h.tolist()`` gives them to the host.  With it, and a stepper
        that can step ahead, the loop looks ahead (see the module's text)."""
        self.stepper, self.choose = stepper, choose
        self.choose_ahead = choose_ahead
        self.max_batch, self.max_tokens = max_batch, max_tokens
        self.max_seq_len, self.vocab_size = max_seq_len, vocab_size
        self.clock, self.sync = clock, sync
        self.steps_run = 0            # model steps, for tests and profiles

    def run(self, requests: Sequence[Request]) -> List[GenerationOutput]:
        validate(requests, self.max_seq_len, self.vocab_size)
        outputs: List[Optional[GenerationOutput]] = [None] * len(requests)
        for i, r in enumerate(requests):
            if r.max_new_tokens == 0:     # nothing to do: no step is run for it
                outputs[i] = GenerationOutput([], len(r.prompt), 0, "length")
        for batch in plan_batches(requests, self.max_batch, self.max_tokens):
            self._run_batch(requests, batch, outputs)
        return outputs  # type: ignore[return-value]

    def _run_batch(self, requests, batch: List[int], outputs) -> None:
        ahead = getattr(self.stepper, "can_step_ahead", None)
        if self.choose_ahead is not None and ahead is not None and ahead(len(batch)):
            self._run_batch_ahead(requests, batch, outputs)
        else:
            self._run_batch_in_turn(requests, batch, outputs)

    def _run_batch_ahead(self, requests, batch: List[int], outputs) -> None:
        t0 = self.clock()
        slots = {i: self.stepper.open_sequence() for i in batch}
        generated = {i: [] for i in batch}
        reason = {}
        draws = {i: DrawStream(requests[i].sampling.seed if requests[i].sampling.seed is not None
                               else 0, i) for i in batch}
        live = list(batch)          # row r of ``logits`` belongs to live[r]
        try:
            logits = self.stepper.step([(slots[i], list(requests[i].prompt)) for i in live],
                                       [[len(requests[i].prompt) - 1] for i in live])
            self.steps_run += 1
            t_prompt = None
            while True:
                params = [requests[i].sampling for i in live]
                us = [0.0 if p.greedy else draws[i].next() for i, p in zip(live, params)]
                chosen = self.choose_ahead(logits, params, us)
                # whoever has budget left after this token takes part in the next step
                going = [(r, i) for r, i in enumerate(live)
                         if len(generated[i]) + 1 < requests[i].max_new_tokens]
                nxt = None
                if going:
                    nxt = self.stepper.step_ahead([(slots[i], r) for r, i in going], chosen)
                    self.steps_run += 1
                tokens = [int(t) for t in chosen.tolist()]     # waits for this step only
                if t_prompt is None:
                    t_prompt = self.clock()
                for i, tok in zip(live, tokens):
                    r = requests[i]
                    if tok in r.stop_ids:
                        if r.include_stop:
                            generated[i].append(tok)
                        reason[i] = "stop"
                    else:
                        generated[i].append(tok)
                        if len(generated[i]) >= r.max_new_tokens:
                            reason[i] = "length"
                    if i in reason:
                        self.stepper.close_sequence(slots.pop(i))
                keep = [k for k, (_r, i) in enumerate(going) if i not in reason]
                if not keep:
                    break
                live = [going[k][1] for k in keep]
                logits = nxt if len(keep) == len(going) else self.stepper.rows(nxt, keep)
            self.sync()
            t_end = self.clock()
        finally:
            for s in slots.values():
                self.stepper.close_sequence(s)
        for i in batch:
            outputs[i] = GenerationOutput(generated[i], len(requests[i].prompt), len(generated[i]),
                                          reason[i], t_prompt - t0, t_end - t_prompt, t_end - t0)

    def _run_batch_in_turn(self, requests, batch: List[int], outputs) -> None:
        t0 = self.clock()
        slots = {i: self.stepper.open_sequence() for i in batch}
        generated = {i: [] for i in batch}
        reason = {}
        draws = {i: DrawStream(requests[i].sampling.seed if requests[i].sampling.seed is not None
                               else 0, i) for i in batch}
        live = list(batch)
        try:
            logits = self.stepper.step([(slots[i], list(requests[i].prompt)) for i in live],
                                       [[len(requests[i].prompt) - 1] for i in live])
            self.steps_run += 1
            first = True
            t_prompt = None
            while True:
                params = [requests[i].sampling for i in live]
                us = [0.0 if p.greedy else draws[i].next() for i, p in zip(live, params)]
                chosen = self.choose(logits, params, us)
                tokens = [int(chosen[r]) for r in range(len(live))]
                if first:
                    self.sync()
                    t_prompt = self.clock()
                    first = False
                still = []
                for i, tok in zip(live, tokens):
                    r = requests[i]
                    if tok in r.stop_ids:
                        if r.include_stop:
                            generated[i].append(tok)
                        reason[i] = "stop"
                    else:
                        generated[i].append(tok)
                        if len(generated[i]) >= r.max_new_tokens:
                            reason[i] = "length"     # no step is run after the last token
                    if i in reason:
                        self.stepper.close_sequence(slots.pop(i))
                    else:
                        still.append(i)
                live = still
                if not live:
                    break
                logits = self.stepper.step([(slots[i], [generated[i][-1]]) for i in live],
                                           [[0] for _ in live])
                self.steps_run += 1
            self.sync()
            t_end = self.clock()
        finally:
            for s in slots.values():
                self.stepper.close_sequence(s)
        for i in batch:
            outputs[i] = GenerationOutput(generated[i], len(requests[i].prompt), len(generated[i]),
                                          reason[i], t_prompt - t0, t_end - t_prompt, t_end - t0)
