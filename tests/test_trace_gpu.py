"""bin/trace_run driven as a user would: the same requests whole, with the last
32 tokens one by one, in batches of unequal lengths, in chunks, and in steps that
mix one and several tokens, in both precisions."""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from conftest import ROOT, TINY, random_tokens
from helpers import assert_close
from plain import qwen3 as plain

pytestmark = pytest.mark.gpu


def _trace():
    """Steps (as JSON lines) and, per step, which (request, positions) its output rows are."""
    V = TINY["B"]["vocab_size"]
    reqs = {f"r{i}": random_tokens(n, V, 800 + i) for i, n in enumerate([1, 7, 30, 64, 90, 130])}
    steps, rows = [], []

    def add(entries, end=()):
        steps.append({"step": len(steps), "entries": [
            {"id": rid, "tokens": reqs[rid][a:b], "want": list(range(b - a)) if want else []}
            for rid, a, b, want in entries], "end": list(end)})
        rows.append([(rid, a, b) for rid, a, b, want in entries if want])

    # whole, alone
    add([("r4", 0, 90, True)], end=["r4"])
    # the same request again: all but the last 32 tokens, then one by one
    reqs["r4b"] = reqs["r4"]
    add([("r4b", 0, 58, True)])
    for t in range(58, 90):
        add([("r4b", t, t + 1, True)], end=["r4b"] if t == 89 else [])
    # a batch of unequal lengths; shorter requests end earlier; a step that wants nothing
    starts = {"r0": 1, "r1": 4, "r2": 30, "r3": 60, "r5": 101}
    add([(rid, 0, n, rid != "r2") for rid, n in starts.items()])
    cur = dict(starts)
    while cur:
        live = [rid for rid in cur if cur[rid] < len(reqs[rid])]
        ended = [rid for rid in cur if cur[rid] >= len(reqs[rid])]
        if not live:
            steps[-1]["end"] += ended
            break
        ending = [rid for rid in live if cur[rid] + 1 >= len(reqs[rid])]
        add([(rid, cur[rid], cur[rid] + 1, True) for rid in live], end=ending + ended)
        for rid in ended + ending:
            cur.pop(rid, None)
        for rid in live:
            if rid in cur:
                cur[rid] += 1
    # a second batch that reuses what the first gave back
    reqs["s0"], reqs["s1"] = random_tokens(65, V, 820), random_tokens(3, V, 821)
    add([("s0", 0, 64, True), ("s1", 0, 2, True)])
    add([("s0", 64, 65, True), ("s1", 2, 3, True)], end=["s0", "s1"])
    # a prompt fed in pieces that end one short of a page, on it and beyond it
    reqs["c0"] = random_tokens(140, V, 830)
    o = 0
    for n in (63, 1, 64, 12):
        add([("c0", o, o + n, True)], end=["c0"] if o + n == 140 else [])
        o += n
    # steps that mix one and several tokens, and a request that starts while others go on
    reqs["m0"], reqs["m1"], reqs["m2"] = (random_tokens(n, V, 840 + n) for n in (26, 11, 71))
    add([("m0", 0, 20, True), ("m1", 0, 9, False)])
    add([("m0", 20, 25, True), ("m1", 9, 10, True), ("m2", 0, 70, True)])
    add([("m0", 25, 26, True), ("m1", 10, 11, True), ("m2", 70, 71, True)], end=["m0", "m1", "m2"])
    return reqs, steps, rows


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay(model_dirs, plain_weights, tmp_path, dtype):
    cfg, w = plain_weights["B"]
    reqs, steps, rows = _trace()
    out = tmp_path / f"out_{dtype}"
    # the most tokens live at once: the first batch (1, 4, 30, 60 and 101 tokens, growing to 1, 7, 30, 64 and 130: 384 in whole pages)
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs["B"],
                           "--dtype", dtype, "--out", str(out), "--max-tokens", "384"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == \
        [f"done {i}" for i in range(len(steps))]
    oracle = {rid: plain.logits(w, cfg, toks) for rid, toks in reqs.items()}
    V = cfg["vocab_size"]
    for i, wanted in enumerate(rows):
        path = out / f"{i}.f32"
        if not wanted:
            assert not path.exists()
            continue
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(-1, V).copy())
        want = torch.cat([oracle[rid][a:b] for rid, a, b in wanted], 0)
        assert_close(got, want, dtype, f"step {i}")
