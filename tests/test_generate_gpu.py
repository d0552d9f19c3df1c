"""Generation through the Python entry point and the command line."""
import json
import os
import subprocess
import sys

import pytest
import torch

from conftest import ROOT, TINY, random_tokens
from plain import qwen3 as plain
from plain import sampling as plain_sampling

pytestmark = pytest.mark.gpu


def _engine(model_dirs, name, dtype, **kw):
    from grout_b200.engine import Engine
    return Engine.load(model_dirs[name], dtype=dtype, max_tokens=2048, max_batch=4, **kw)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain_in_32_bit(model_dirs, plain_weights, name):
    cfg, w = plain_weights[name]
    eng = _engine(model_dirs, name, "float32")
    lens = [5, 11, 17] if name == "A" else [1, 7, 30, 64]
    n_new = 8 if name == "A" else 16
    prompts = [random_tokens(n, cfg["vocab_size"], 700 + i) for i, n in enumerate(lens)]
    free = [plain.greedy_generate(w, cfg, p, n_new) for p in prompts]
    outs = eng.generate(prompts, n_new, ignore_eos=True)
    assert [o.token_ids for o in outs] == free
    assert all(o.finish_reason == "length" and o.generated_tokens == n_new for o in outs)
    # a stop token: the third token of the first request ends it, the others go on
    stop = free[0][2]
    want = [plain.greedy_generate(w, cfg, p, n_new, stop_ids=(stop,)) for p in prompts]
    outs = eng.generate(prompts, n_new, stop_ids=[stop])
    assert [o.token_ids for o in outs] == want
    assert outs[0].finish_reason == "stop" and len(outs[0].token_ids) <= 2
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and eng.cache.tokens_held() == 0


def test_more_requests_than_slots_are_served_batch_after_batch(model_dirs, plain_weights):
    cfg, w = plain_weights["A"]
    eng = _engine(model_dirs, "A", "float32")
    prompts = [random_tokens(3 + 2 * i, 256, 720 + i) for i in range(9)]    # 9 requests, 4 slots
    outs = eng.generate(prompts, 5, ignore_eos=True)
    assert [o.token_ids for o in outs] == [plain.greedy_generate(w, cfg, p, 5) for p in prompts]
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_looking_ahead_changes_no_token(model_dirs, dtype):
    """Queueing a step before the host has read the tokens of the one before
    (their input taken on the device) returns what stepping in turn returns:
    unequal budgets, stop tokens at different places, sampled and greedy rows,
    more requests than slots."""
    from grout_b200.engine.generate import Request
    from grout_b200.sampling import SamplingParams
    eng = _engine(model_dirs, "B", dtype)
    prompts = [random_tokens(n, 384, 760 + n) for n in (2, 9, 33, 64, 5, 17)]
    free = eng.generate(prompts, 14, ignore_eos=True, look_ahead=False)
    stops = (free[0].token_ids[3], free[2].token_ids[1], free[4].token_ids[13])
    reqs = [Request(p, budget, SamplingParams(True, t, k, 0.9, seed=11 + i).normalised()
                    if t else SamplingParams().normalised(), stops)
            for i, (p, budget, t, k) in enumerate(zip(prompts, (14, 1, 9, 14, 14, 2),
                                                      (0, 0, 0, 0.8, 0, 0.7), (0, 0, 0, 20, 0, 0)))]
    in_turn = eng.generate(reqs, look_ahead=False)
    ahead = eng.generate(reqs, look_ahead=True)
    assert [o.token_ids for o in ahead] == [o.token_ids for o in in_turn]
    assert [o.finish_reason for o in ahead] == [o.finish_reason for o in in_turn]
    for i, budget in ((0, 14), (1, 1), (2, 9), (4, 14)):      # the greedy requests
        want = []
        for tok in free[i].token_ids[:budget]:
            if tok in stops:
                break
            want.append(tok)
        assert in_turn[i].token_ids == want
    assert in_turn[0].finish_reason == "stop" and in_turn[1].finish_reason == "length"
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and eng.cache.tokens_held() == 0


@pytest.mark.parametrize("device_argmax", [True, False])
def test_bf16_greedy_choices_are_the_plain_best_within_rounding(model_dirs, plain_weights,
                                                                device_argmax):
    cfg, w = plain_weights["B"]
    eng = _engine(model_dirs, "B", "bfloat16")
    prompts = [random_tokens(n, 384, 740 + n) for n in (3, 40, 70)]
    outs = eng.generate(prompts, 12, ignore_eos=True, device_argmax=device_argmax)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o.token_ids:
            row = plain.logits(w, cfg, seq, rows=[len(seq) - 1])[0]
            assert float(row[tok]) >= float(row.max()) - 0.03
            seq.append(tok)


def test_sampled_generation_is_repeatable_and_follows_the_plain_sampler(model_dirs, plain_weights):
    from grout_b200.sampling import DrawStream, SamplingParams
    cfg, w = plain_weights["B"]
    eng = _engine(model_dirs, "B", "float32")
    prompts = [random_tokens(n, 384, 760 + n) for n in (1, 7, 30, 64)]
    sp = SamplingParams(True, 0.8, 0, 1.0, seed=11)
    a = eng.generate(prompts, 16, sampling=sp, ignore_eos=True)
    b = eng.generate(prompts, 16, sampling=sp, ignore_eos=True)
    assert [o.token_ids for o in a] == [o.token_ids for o in b]
    c = eng.generate(prompts, 16, sampling=SamplingParams(True, 0.8, 0, 1.0, seed=12), ignore_eos=True)
    assert [o.token_ids for o in a] != [o.token_ids for o in c]
    for i, (p, o) in enumerate(zip(prompts, a)):
        draws, seq = DrawStream(11, i), list(p)
        for tok in o.token_ids:
            row = plain.logits(w, cfg, seq, rows=[len(seq) - 1])[0]
            assert plain_sampling.sample_next(row.tolist(), 0.8, 0, 1.0, draws.next()) == tok
            seq.append(tok)
    # top-k and top-p through the same entry point
    sp2 = SamplingParams(True, 0.9, 5, 0.8, seed=3)
    for o, p in zip(eng.generate(prompts[:2], 6, sampling=sp2, ignore_eos=True), prompts):
        draws, seq = DrawStream(3, prompts.index(p)), list(p)
        for tok in o.token_ids:
            row = plain.logits(w, cfg, seq, rows=[len(seq) - 1])[0]
            assert plain_sampling.sample_next(row.tolist(), 0.9, 5, 0.8, draws.next()) == tok
            seq.append(tok)


def test_limits(model_dirs):
    eng = _engine(model_dirs, "A", "float32")
    with pytest.raises(ValueError, match="max_seq_len"):
        eng.generate([[1] * 100], 100)
    with pytest.raises(ValueError, match="no tokens"):
        eng.generate([[]], 4)
    assert eng.generate([[1, 2]], 0)[0].token_ids == []
    with pytest.raises(ValueError, match="vocabulary"):
        eng.step([(eng.open_sequence(), [256])])
    # a wanted place beyond the entry's tokens is refused on every path: prompt and decode
    # steps, captured (bfloat16) or launched one by one (32-bit)
    for dtype in ("float32", "bfloat16"):
        e = _engine(model_dirs, "A", dtype)
        s = e.open_sequence()
        with pytest.raises(ValueError, match="outside the 3 tokens"):
            e.step([(s, [1, 2, 3])], [[3]])
        assert e.length(s) == 0                      # a refused step stores nothing
        e.step([(s, [1, 2, 3])], [[2]])
        with pytest.raises(ValueError, match="outside the 1 tokens"):
            e.step([(s, [4])], [[1]])
        assert e.step([(s, [4])], [[0]]).shape == (1, 256) and e.length(s) == 4
        e.close_sequence(s)


def test_looking_ahead_across_a_bucket_of_rows(model_dirs):
    """17 requests of which one draws a stop token early: stepping in turn, the step
    after it has 16 rows; looking ahead, the request still holds a row there and the
    step has 17, which is the next bucket of the captured steps.  The 32-bit path gives
    the same tokens either way; the bfloat16 path, where the wider bucket's products
    round differently, is held to the same finish reasons."""
    from grout_b200.engine import Engine
    from grout_b200.engine.generate import Request
    from grout_b200.sampling import SamplingParams
    prompts = [random_tokens(3 + i, 384, 1760 + i) for i in range(17)]
    for dtype in ("float32", "bfloat16"):
        eng = Engine.load(model_dirs["B"], dtype=dtype, max_tokens=32 * 64, max_batch=32,
                          max_seq_len=64, use_graphs=True)
        free = eng.generate(prompts, 8, ignore_eos=True, look_ahead=False)
        stop = free[5].token_ids[2]
        reqs = [Request(p, 8, SamplingParams().normalised(), (stop,)) for p in prompts]
        in_turn = eng.generate(reqs, look_ahead=False)
        ahead = eng.generate(reqs, look_ahead=True)
        assert in_turn[5].finish_reason == "stop" and len(in_turn[5].token_ids) <= 2
        assert {16, 32} <= {b for b, _l in eng.graphs.decode_graphs}
        if dtype == "float32":
            assert [o.token_ids for o in ahead] == [o.token_ids for o in in_turn]
        assert [o.finish_reason for o in ahead] == [o.finish_reason for o in in_turn]
        eng.cache.check()


def test_a_kernel_that_gave_up_on_a_wait_is_reported(model_dirs):
    """The tensor-memory kernels bound their waits; when one runs out the role records
    a code in a device flag, raises its block's abort flag (which ends the waits of the
    block's other roles) and the block leaves.  A kernel made for this test walks that
    path by itself: one block, a barrier at which nobody arrives, a limit of one
    millisecond, nothing in flight.  ``Engine.check`` and generation then raise, the
    batch's slots come back all the same, and the next call is clean again."""
    import time
    from grout_b200.engine import Engine
    from grout_b200.kernels import ops
    eng = Engine.load(model_dirs["A"], dtype="bfloat16", max_tokens=1024, max_batch=4, max_seq_len=128)
    prompts = [random_tokens(9, TINY["A"]["vocab_size"], 77)]
    good = eng.generate(prompts, max_new_tokens=4, ignore_eos=True)
    t0 = time.time()
    assert ops.tc_wait_selftest(eng.device, limit_us=1000) == 2      # both roles left
    assert time.time() - t0 < 1.0                # the second role did not sit out its own 2 s
    with pytest.raises(ops.KernelError, match="stage that never arrived"):
        eng.check()
    eng.check()                                  # the flag was cleared by the report
    ops.tc_wait_selftest(eng.device, limit_us=1000)
    with pytest.raises(ops.KernelError, match="stage that never arrived"):
        eng.generate(prompts, max_new_tokens=4, ignore_eos=True)
    eng.cache.check()
    assert eng.cache.slots.n_held == 0                     # the batch's slots came back all the same
    again = eng.generate(prompts, max_new_tokens=4, ignore_eos=True)
    assert again[0].token_ids == good[0].token_ids


def test_command_line(model_dirs, plain_weights, tmp_path):
    cfg, w = plain_weights["A"]
    prompt = random_tokens(9, 256, 780)
    out = str(tmp_path / "out.json")
    env = dict(os.environ, PYTHONPATH=ROOT)
    for extra in (["--fp32"], ["--fp32", "--device-argmax", "--profile"],
                  ["--fp32", "--profile", "--profile-ops"]):
        r = subprocess.run([sys.executable, "-m", "grout_b200", "--model", model_dirs["A"],
                            "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "6",
                            "--ignore-eos", "--output-json", out] + extra,
                           capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert "t/s:" in r.stdout and "Generating 6 tokens" in r.stdout
        rec = json.load(open(out))
        assert rec["token_ids"] == plain.greedy_generate(w, cfg, prompt, 6)
        assert rec["generated_tokens"] == 6 and rec["prompt_tokens"] == 9
    assert "profile:" in r.stdout
    # the last run timed every operation: a row per kernel with its calls and rates
    assert "op profile" in r.stdout
    ops_rows = {l.split()[0]: l.split() for l in r.stdout.splitlines() if l.startswith("  ")}
    for name in ("embed", "add_rmsnorm", "qk_prepare", "attn_generic", "gemm_f32"):
        assert name in ops_rows and int(ops_rows[name][1]) > 0, (name, r.stdout[-2000:])
    # the bench binary's options: several measured generations, one JSON line each
    lines = str(tmp_path / "runs.jsonl")
    r = subprocess.run([sys.executable, "-m", "grout_b200", "--model", model_dirs["A"],
                        "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "5",
                        "--ignore-eos", "--reps", "3", "--json", lines, "--variant", "t", "--quiet"],
                       capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    recs = [json.loads(l) for l in open(lines)]
    assert [x["rep"] for x in recs] == [0, 1, 2]
    assert all(x["gen_tokens"] == 5 and x["prompt_tokens"] == 9 and x["variant"] == "t" and
               x["e2e_ms"] >= x["decode_ms"] > 0 for x in recs)
    assert "run 3/3" in r.stdout and "profile:" not in r.stdout
    # random weights from a configuration file and a seed: the same seed, the same tokens
    # (configuration B: its output head is not tied to the embedding, so that the greedy
    # continuation is not just the last token again, whatever the weights)
    seen = []
    for seed in ("4", "4", "5"):
        r = subprocess.run([sys.executable, "-m", "grout_b200", "--model",
                            "random:" + os.path.join(model_dirs["B"], "config.json"), "--seed", seed,
                            "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "6",
                            "--ignore-eos", "--output-json", out],
                           capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        seen.append(json.load(open(out))["token_ids"])
    assert seen[0] == seen[1] and seen[0] != seen[2] and len(seen[0]) == 6
