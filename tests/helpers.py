"""Ways of cutting the same requests into steps, shared by the GPU tests."""
import torch


# The reference's own bars: fp32 against an independent fp32 model atol 2e-5,
# rtol 2e-4 (tests/reference_training.py:25); bf16 atol 0.012, rtol 0.035
# (tests/reference_quantized.py:94-95).
TOL = {"float32": dict(atol=2e-5, rtol=2e-4), "bfloat16": dict(atol=0.012, rtol=0.035)}


def assert_close(got, want, dtype, what=""):
    got = got.detach().double().cpu()
    want = want.detach().double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    tol = TOL[dtype]
    err = (got - want).abs()
    bound = tol["atol"] + tol["rtol"] * want.abs()
    if not bool((err <= bound).all()):
        bad = (err > bound).nonzero()
        first = tuple(int(v) for v in bad[0])
        raise AssertionError(
            f"{what}: {bad.shape[0]} of {err.numel()} values differ, first at {first}: "
            f"got {got[first].item():.6g}, want {want[first].item():.6g}; max err {err.max().item():.3g}")


def run_whole(engine, tokens):
    """One request alone, all its tokens in one step, logits everywhere."""
    s = engine.open_sequence()
    try:
        return engine.step([(s, tokens)], [list(range(len(tokens)))]).float().cpu()
    finally:
        engine.close_sequence(s)


def run_tail_decoded(engine, tokens, tail=32):
    """All but the last ``tail`` tokens in one step, then one token per step."""
    tail = min(tail, len(tokens) - 1)
    head = len(tokens) - tail
    s = engine.open_sequence()
    try:
        rows = [engine.step([(s, tokens[:head])], [list(range(head))]).float().cpu()]
        for t in tokens[head:]:
            rows.append(engine.step([(s, [t])], [[0]]).float().cpu())
        return torch.cat(rows, 0)
    finally:
        engine.close_sequence(s)


def run_batch(engine, requests, prompt_lens):
    """Requests that start together: prompts (of unequal lengths) in one step,
    then one token each per step; a request whose tokens are used up ends and its
    slot is given back while the others go on.  Returns logits of every position
    of every request."""
    slots = [engine.open_sequence() for _ in requests]
    out = [[] for _ in requests]
    live = list(range(len(requests)))
    try:
        logits = engine.step([(slots[i], requests[i][:prompt_lens[i]]) for i in live],
                             [list(range(prompt_lens[i])) for i in live]).float().cpu()
        o = 0
        for i in live:
            out[i].append(logits[o:o + prompt_lens[i]])
            o += prompt_lens[i]
        cursor = list(prompt_lens)
        while True:
            for i in list(live):
                if cursor[i] >= len(requests[i]):
                    engine.close_sequence(slots[i])
                    slots[i] = None
                    live.remove(i)
            if not live:
                break
            logits = engine.step([(slots[i], [requests[i][cursor[i]]]) for i in live],
                                 [[0] for _ in live]).float().cpu()
            for r, i in enumerate(live):
                out[i].append(logits[r:r + 1])
                cursor[i] += 1
        return [torch.cat(o, 0) for o in out]
    finally:
        for s in slots:
            if s is not None:
                engine.close_sequence(s)


def run_chunks(engine, tokens, chunks):
    """One request alone, its tokens fed in steps of the given sizes (which must
    add up to its length), logits everywhere."""
    assert sum(chunks) == len(tokens)
    s = engine.open_sequence()
    try:
        rows, o = [], 0
        for n in chunks:
            rows.append(engine.step([(s, tokens[o:o + n])], [list(range(n))]).float().cpu())
            o += n
        return torch.cat(rows, 0)
    finally:
        engine.close_sequence(s)


def run_schedule(engine, requests, schedule):
    """``schedule``: a list of steps, each a dict request index -> number of tokens
    that request brings in that step (a request may be absent from a step, start in
    a later one, bring one token while another brings many).  Every request's
    tokens must be used up by the end.  Returns logits of every position of every
    request; a request's slot is given back after its last token."""
    slots, cursor = {}, [0] * len(requests)
    out = [[] for _ in requests]
    try:
        for stepno, bring in enumerate(schedule):
            entries, want, order = [], [], []
            for i, n in bring.items():
                if i not in slots:
                    assert cursor[i] == 0
                    slots[i] = engine.open_sequence()
                entries.append((slots[i], requests[i][cursor[i]:cursor[i] + n]))
                want.append(list(range(n)))
                order.append((i, n))
            logits = engine.step(entries, want).float().cpu()
            o = 0
            for i, n in order:
                out[i].append(logits[o:o + n])
                o += n
                cursor[i] += n
                if cursor[i] == len(requests[i]):
                    engine.close_sequence(slots.pop(i))
        assert cursor == [len(r) for r in requests], "the schedule does not use every token"
        return [torch.cat(o, 0) for o in out]
    finally:
        for s in slots.values():
            engine.close_sequence(s)
