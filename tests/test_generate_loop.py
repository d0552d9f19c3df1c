"""The generation loop's decisions with a scripted stand-in for the model (no GPU)."""
import pytest

from grout_b200.cache import PAGE_TOKENS
from grout_b200.engine.generate import GenerationLoop, Request, plan_batches
from grout_b200.sampling import SamplingParams


class Script:
    """Stands in for the engine: request r's n-th generated token is script[r][n];
    a step returns, per row, which request it belongs to and how long it is now."""

    def __init__(self, prompts, script, max_slots=4):
        self.prompts, self.script = prompts, script
        self.by_prompt = {tuple(p): i for i, p in enumerate(prompts)}
        self.free = list(range(max_slots))
        self.open, self.request_of, self.steps, self.max_live = {}, {}, [], 0
        self.history = []

    def open_sequence(self):
        s = self.free.pop()
        self.open[s] = []
        self.request_of[s] = None
        self.history.append(("open", s))
        return s

    def close_sequence(self, s):
        assert s in self.open, "closed twice"
        del self.open[s]
        self.free.append(s)
        self.history.append(("close", s))

    def step(self, entries, want):
        self.max_live = max(self.max_live, len(self.open))
        rows = []
        for (slot, toks), w in zip(entries, want):
            assert slot in self.open
            self.open[slot].extend(toks)
            if self.request_of[slot] is None:
                assert tuple(self.open[slot]) in self.by_prompt, "first step must bring the prompt"
                self.request_of[slot] = self.by_prompt[tuple(self.open[slot])]
                assert w == [len(toks) - 1]
            else:
                assert len(toks) == 1 and w == [0]
            rows.append((self.request_of[slot], len(self.open[slot])))
        self.steps.append([r for r, _ in rows])
        return rows

    def choose(self, rows, params, draws):
        return [self.script[r][length - len(self.prompts[r])] for r, length in rows]


def _loop(prompts, script, **kw):
    st = Script(prompts, script, kw.pop("max_slots", 4))
    loop = GenerationLoop(st, st.choose, max_batch=kw.pop("max_batch", 4),
                          max_tokens=kw.pop("max_tokens", 4096), max_seq_len=kw.pop("max_seq_len", 512),
                          vocab_size=1000)
    return st, loop


def test_stop_token_ends_a_request_and_is_not_returned():
    prompts = [[1, 2, 3], [4, 5]]
    script = [[10, 11, 99, 12], [20, 21, 22, 23, 24]]
    st, loop = _loop(prompts, script)
    outs = loop.run([Request(prompts[0], 8, stop_ids=(99,)), Request(prompts[1], 4, stop_ids=(99,))])
    assert outs[0].token_ids == [10, 11] and outs[0].finish_reason == "stop"
    assert outs[1].token_ids == [20, 21, 22, 23] and outs[1].finish_reason == "length"
    # the shorter request left the batch: later steps carry request 1 alone
    assert st.steps == [[0, 1], [0, 1], [0, 1], [1]]
    assert not st.open and sorted(st.free) == [0, 1, 2, 3]
    # no step after the last token: 1 prompt step + 3 decode steps for 4 tokens
    assert loop.steps_run == 4


def test_stop_token_can_be_returned_on_request():
    st, loop = _loop([[1]], [[5, 99]])
    out = loop.run([Request([1], 8, stop_ids=(99,), include_stop=True)])[0]
    assert out.token_ids == [5, 99] and out.finish_reason == "stop"


def test_first_token_may_already_stop():
    st, loop = _loop([[1, 2]], [[99]])
    out = loop.run([Request([1, 2], 8, stop_ids=(99,))])[0]
    assert out.token_ids == [] and out.generated_tokens == 0 and loop.steps_run == 1


def test_zero_budget_runs_nothing():
    st, loop = _loop([[1, 2]], [[5]])
    out = loop.run([Request([1, 2], 0)])[0]
    assert out.token_ids == [] and loop.steps_run == 0 and st.history == []


def test_batches_follow_one_another_and_reuse_slots():
    prompts = [[i + 1] * (i + 1) for i in range(5)]
    script = [[100 + i] * 3 for i in range(5)]
    st, loop = _loop(prompts, script, max_batch=2, max_slots=2)
    outs = loop.run([Request(p, 3) for p in prompts])
    assert [o.token_ids for o in outs] == script
    assert st.max_live <= 2
    opened = [s for what, s in st.history if what == "open"]
    assert len(opened) == 5 and set(opened) == {0, 1}
    assert [sorted(s) for s in st.steps if len(s) == 2][0] == [0, 1]


def test_token_budget_cuts_batches():
    reqs = [Request([1] * 10, 50), Request([1] * 70, 60), Request([1] * 5, 5), Request([1], 0)]
    # rounded to pages: 64, 192, 64
    assert plan_batches(reqs, 8, 4096) == [[0, 1, 2]]
    assert plan_batches(reqs, 8, 256) == [[0, 1], [2]]
    assert plan_batches(reqs, 1, 4096) == [[0], [1], [2]]
    with pytest.raises(ValueError):
        plan_batches(reqs, 8, 128)
    assert PAGE_TOKENS == 64


def test_limits_are_checked_before_anything_runs():
    st, loop = _loop([[1]], [[5]], max_seq_len=16)
    with pytest.raises(ValueError, match="no tokens"):
        loop.run([Request([], 4)])
    with pytest.raises(ValueError, match="max_seq_len"):
        loop.run([Request([1] * 10, 7)])
    with pytest.raises(ValueError, match="vocabulary"):
        loop.run([Request([1000], 2)])
    assert st.history == []


def test_slots_are_given_back_when_a_step_fails():
    st, loop = _loop([[1, 2]], [[5, 6, 7]])
    calls = {"n": 0}
    real = st.step

    def failing(entries, want):
        calls["n"] += 1
        if calls["n"] == 2:
            raise RuntimeError("boom")
        return real(entries, want)
    st.step = failing
    with pytest.raises(RuntimeError):
        loop.run([Request([1, 2], 3)])
    assert not st.open


def test_draws_are_per_request_and_repeatable():
    from grout_b200.sampling import DrawStream
    a = [DrawStream(7, 0).next() for _ in range(1)] + [DrawStream(7, 0).next()]
    assert a[0] == a[1] and 0.0 <= a[0] < 1.0
    s1, s2 = DrawStream(7, 0), DrawStream(7, 1)
    assert [s1.next() for _ in range(3)] != [s2.next() for _ in range(3)]
    assert SamplingParams(True, 0.0).normalised().temperature == 1e-5
    assert SamplingParams(False, 0.8).greedy and not SamplingParams(True, 0.8).greedy


class AheadScript(Script):
    """The scripted model with the two extra calls of a stepper that can run a
    step before the host has read the tokens of the one before."""

    class Chosen:
        def __init__(self, tokens):
            self.tokens = tokens
            self.read = False

        def tolist(self):
            self.read = True
            return list(self.tokens)

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.ahead_steps = []

    def can_step_ahead(self, n):
        return True

    def choose_ahead(self, rows, params, draws):
        return AheadScript.Chosen(self.choose(rows, params, draws))

    def step_ahead(self, entries, chosen):
        assert not chosen.read, "the step must be queued before the tokens are read"
        self.ahead_steps.append([r for _s, r in entries])
        return self.step([(slot, [chosen.tokens[r]]) for slot, r in entries], [[0] for _ in entries])

    def rows(self, logits, keep):
        return [logits[k] for k in keep]


def _ahead_loop(prompts, script, **kw):
    st = AheadScript(prompts, script, kw.pop("max_slots", 4))
    loop = GenerationLoop(st, st.choose, max_batch=kw.pop("max_batch", 4),
                          max_tokens=kw.pop("max_tokens", 4096), max_seq_len=kw.pop("max_seq_len", 512),
                          vocab_size=1000, choose_ahead=st.choose_ahead)
    return st, loop


def test_looking_ahead_returns_the_same_tokens():
    prompts = [[1, 2, 3], [4, 5], [6]]
    script = [[10, 11, 99, 12, 13], [20, 21, 22, 23, 24], [30, 99, 31, 32, 33]]
    reqs = [Request(prompts[0], 8, stop_ids=(99,)), Request(prompts[1], 4, stop_ids=(99,)),
            Request(prompts[2], 5, stop_ids=(99,), include_stop=True)]
    st0, loop0 = _loop(prompts, script)
    want = loop0.run(reqs)
    st, loop = _ahead_loop(prompts, script)
    outs = loop.run(reqs)
    assert [o.token_ids for o in outs] == [o.token_ids for o in want]
    assert [o.finish_reason for o in outs] == [o.finish_reason for o in want]
    assert outs[0].token_ids == [10, 11] and outs[2].token_ids == [30, 99]
    # every decode step was queued before its tokens were read; a request that drew a
    # stop token had already been sent into one more step, which changes nothing returned
    assert st.steps == [[0, 1, 2], [0, 1, 2], [0, 1, 2], [0, 1]]
    assert st.ahead_steps == [[0, 1, 2], [0, 1, 2], [0, 1]]
    assert want and st0.steps == [[0, 1, 2], [0, 1, 2], [0, 1], [1]]   # in turn: no row runs for nothing
    assert not st.open and sorted(st.free) == [0, 1, 2, 3]


def test_looking_ahead_runs_no_step_beyond_a_budget():
    prompts = [[1, 2], [3]]
    script = [[10, 11, 12, 13], [20, 21, 22, 23]]
    st, loop = _ahead_loop(prompts, script)
    outs = loop.run([Request(prompts[0], 1), Request(prompts[1], 3)])
    assert outs[0].token_ids == [10] and outs[1].token_ids == [20, 21, 22]
    assert all(o.finish_reason == "length" for o in outs)
    assert st.steps == [[0, 1], [1], [1]]          # as without looking ahead
    assert loop.steps_run == 3 and not st.open


def test_looking_ahead_serves_batch_after_batch():
    prompts = [[i + 1] for i in range(5)]
    script = [[100 + i, 99] for i in range(5)]
    st, loop = _ahead_loop(prompts, script, max_batch=2, max_slots=2)
    outs = loop.run([Request(p, 4, stop_ids=(99,)) for p in prompts])
    assert [o.token_ids for o in outs] == [[100 + i] for i in range(5)]
    assert st.max_live <= 2 and not st.open and sorted(st.free) == [0, 1]


def test_random_requests_in_turn_and_looking_ahead():
    """Random prompts, budgets, stop tokens and batch limits: both ways of running a batch
    return what the script and the rules say (a stop token ends the request and is returned
    only on request; a budget ends it with "length"), no request runs a step beyond its
    last token when stepping in turn, and every slot comes back."""
    import random
    rng = random.Random(11)
    for trial in range(60):
        n = rng.randint(1, 9)
        prompts, script, reqs, want = [], [], [], []
        for r in range(n):
            prompt = [r + 1] * (r + 1) + [rng.randint(1, 50) for _ in range(rng.randint(0, 4))]
            budget = rng.randint(0, 7)
            stream = [rng.choice([99, 98] + list(range(100, 120))) for _ in range(8)]
            stops = rng.choice([(), (99,), (99, 98)])
            include = rng.random() < 0.3
            prompts.append(prompt), script.append(stream)
            reqs.append(Request(prompt, budget, stop_ids=stops, include_stop=include))
            out, reason = [], "length"
            for tok in stream[:budget]:
                if tok in stops:
                    if include:
                        out.append(tok)
                    reason = "stop"
                    break
                out.append(tok)
            want.append((out, reason if budget else "length"))
        max_batch = rng.randint(1, 4)
        for make in (_loop, _ahead_loop):
            st, loop = make(prompts, script, max_batch=max_batch, max_slots=max_batch)
            outs = loop.run(reqs)
            for o, (toks, reason), rq in zip(outs, want, reqs):
                assert o.token_ids == toks, (trial, make.__name__)
                if rq.max_new_tokens:
                    assert o.finish_reason == reason
                assert o.prompt_tokens == len(rq.prompt) and o.generated_tokens == len(toks)
            assert not st.open and sorted(st.free) == list(range(max_batch))
            assert st.max_live <= max_batch
            if make is _loop:
                # in turn: request r took part in one prompt step and one step per token it
                # fed back, i.e. per generated token but the last one
                for r, (rq, (toks, reason)) in enumerate(zip(reqs, want)):
                    if rq.max_new_tokens == 0:
                        assert sum(s.count(r) for s in st.steps) == 0
                        continue
                    fed = len(toks) - (1 if (reason == "stop" and rq.include_stop) else 0)
                    done_by_budget = reason == "length"
                    expect = 1 + (fed - 1 if done_by_budget else fed)
                    assert sum(s.count(r) for s in st.steps) == max(expect, 1), (trial, r)
