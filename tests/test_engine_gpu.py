"""The engine against the plain implementation, in every way of cutting the work."""
import pytest
import torch

from conftest import TINY, random_tokens
from helpers import (assert_close, run_batch, run_chunks, run_schedule, run_tail_decoded,
                     run_whole)
from plain import qwen3 as plain

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": [5, 70, 128], "B": [1, 7, 64, 150], "C": [33, 130, 300], "D": [3, 129, 400],
           "E": [2, 100, 200]}


@pytest.fixture(scope="module")
def engines(model_dirs):
    from grout_b200.engine import Engine
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = Engine.load(model_dirs[name], dtype=dtype, max_tokens=4096,
                                              max_batch=8, max_seq_len=512)
        return made[(name, dtype)]
    return get


@pytest.fixture(scope="module")
def oracle(plain_weights):
    memo = {}

    def get(name, tokens):
        key = (name, tuple(tokens))
        if key not in memo:
            cfg, w = plain_weights[name]
            memo[key] = plain.logits(w, cfg, list(tokens))
        return memo[key]
    return get


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(TINY))
def test_each_request_alone_and_whole(engines, oracle, name, dtype):
    eng = engines(name, dtype)
    for i, n in enumerate(LENGTHS[name]):
        toks = random_tokens(n, TINY[name]["vocab_size"], 100 + i)
        assert_close(run_whole(eng, toks), oracle(name, toks), dtype, f"{name} whole, {n} tokens")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and eng.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(TINY))
def test_last_32_tokens_one_by_one(engines, oracle, name, dtype):
    eng = engines(name, dtype)
    for i, n in enumerate(LENGTHS[name][1:]):
        toks = random_tokens(n, TINY[name]["vocab_size"], 200 + i)
        assert_close(run_tail_decoded(eng, toks), oracle(name, toks), dtype,
                     f"{name} tail decoded, {n} tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(TINY))
def test_unequal_batches_one_after_another(engines, oracle, name, dtype):
    """Three batches in a row on the same engine, so that slots and pages of an
    earlier batch are used again by a later one; within a batch the shorter
    requests end earlier."""
    eng = engines(name, dtype)
    V, top = TINY[name]["vocab_size"], TINY[name]["max_position_embeddings"]
    plans = [[(5, 3), (11, 9), (17, 1)],
             [(1, 20), (7, 2), (30, 11), (64, 5), (min(top - 40, 130), 33)],
             [(65, 4), (2, 4)]]
    used = []
    for b, plan in enumerate(plans):
        reqs = [random_tokens(p + d, V, 300 + 10 * b + i) for i, (p, d) in enumerate(plan)]
        got = run_batch(eng, reqs, [p for p, _ in plan])
        for i, r in enumerate(reqs):
            assert_close(got[i], oracle(name, r), dtype, f"{name} batch {b} request {i}")
        eng.cache.check()
        assert eng.cache.slots.n_held == 0
        used.append(True)
    assert len(used) == 3


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_long_decoding(engines, oracle, dtype):
    """A prompt of one token followed by 140 decoded tokens: the first positions
    of a sequence and a long run of single steps across two page boundaries."""
    eng = engines("B", dtype)
    toks = random_tokens(141, TINY["B"]["vocab_size"], 400)
    assert_close(run_tail_decoded(eng, toks, tail=140), oracle("B", toks), dtype, "long decoding")


def _chunkings(name):
    """Ways of cutting a prompt: tiny pieces; pieces that end one short of a page,
    on it and beyond it; pieces that cross the 64-token page twice."""
    if TINY[name]["max_position_embeddings"] < 140:
        return [[2, 1, 4], [63, 1, 62, 2], [60, 10, 58]]
    return [[2, 1, 4], [63, 1, 64, 2], [60, 10, 70]]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(TINY))
def test_a_prompt_fed_in_chunks(engines, oracle, name, dtype):
    """A sequence continued with more than one token: the step packs rows whose
    positions start beyond zero, attention reads keys of earlier steps and of this
    one, and a slot may grow by several pages in one step.  (The reference holds its
    engine to chunked == whole: src/bin/grout_quant_probe.rs:7-60.)"""
    eng = engines(name, dtype)
    for i, chunks in enumerate(_chunkings(name)):
        toks = random_tokens(sum(chunks), TINY[name]["vocab_size"], 700 + i)
        got = run_chunks(eng, toks, chunks)
        assert_close(got, oracle(name, toks), dtype, f"{name} chunks {chunks}")
        if dtype == "float32":
            assert (got - run_whole(eng, toks)).abs().max().item() < 2e-6, chunks
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


def _mixed_schedule():
    """Request 0 starts with 20 tokens and goes on with 5 at once; request 1 starts
    with 9 and brings one token at a time; request 2 joins in the third step with 70
    tokens while the others continue; later steps mix one and several tokens, and the
    requests end at different steps."""
    lengths = [20 + 5 + 1 + 3 + 1, 9 + 1 + 1 + 1 + 1 + 1, 70 + 1 + 2]
    schedule = [{0: 20, 1: 9}, {0: 5, 1: 1}, {0: 1, 1: 1, 2: 70}, {0: 3, 1: 1, 2: 1},
                {0: 1, 1: 1, 2: 2}, {1: 1}]
    return lengths, schedule


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(TINY))
def test_steps_that_mix_one_and_many_tokens(engines, oracle, name, dtype):
    eng = engines(name, dtype)
    lengths, schedule = _mixed_schedule()
    reqs = [random_tokens(n, TINY[name]["vocab_size"], 720 + i) for i, n in enumerate(lengths)]
    got = run_schedule(eng, reqs, schedule)
    for i, r in enumerate(reqs):
        assert_close(got[i], oracle(name, r), dtype, f"{name} mixed steps, request {i}")
        if dtype == "float32":
            assert (got[i] - run_whole(eng, r)).abs().max().item() < 2e-6, i
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.fixture(scope="module")
def wide_engines(model_dirs):
    """Engines with room for 64 sequences at once (graph buckets 32 and 64)."""
    from grout_b200.engine import Engine
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = Engine.load(model_dirs[name], dtype=dtype, max_tokens=64 * 128,
                                              max_batch=64, max_seq_len=128)
        return made[(name, dtype)]
    return get


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])     # D: heads of 64, the TMA decode attention at 64 live
@pytest.mark.parametrize("n_live", [20, 64])
def test_many_live_sequences(wide_engines, oracle, name, dtype, n_live):
    """20 and 64 sequences of unequal lengths alive at once (the captured steps of 32
    and 64 rows, the wider tiles of the decode product, decode attention over many
    sequences), the shorter ones ending earlier, two batches in a row so that every
    slot and page is used again."""
    import random
    eng = wide_engines(name, dtype)
    V = TINY[name]["vocab_size"]
    rng = random.Random(n_live)
    for b in range(2):
        plan = [(rng.choice([1, 2, 7, 30, 63, 64, 65]), rng.randint(1, 9)) for _ in range(n_live)]
        plan[rng.randrange(n_live)] = (40, 14)               # one that outlives the others
        reqs = [random_tokens(p + d, V, 5000 + 100 * b + i) for i, (p, d) in enumerate(plan)]
        got = run_batch(eng, reqs, [p for p, _ in plan])
        for i, r in enumerate(reqs):
            assert_close(got[i], oracle(name, r), dtype, f"{name} {n_live} live, batch {b}, request {i}")
        eng.cache.check()
        assert eng.cache.slots.n_held == 0 and eng.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_captured_steps_against_steps_launched_one_by_one(model_dirs, oracle, dtype):
    """Prompt steps and decode steps through captured graphs (padded to their buckets
    of tokens, sequences and wanted rows) against the same steps launched kernel by
    kernel: bit-equal in 32-bit, where no kernel's order of sums depends on the number
    of rows, and both within the bar of the plain implementation in bfloat16.  And the
    logits a step returns are the caller's: a later step does not change them."""
    from grout_b200.engine import Engine
    lengths, schedule = _mixed_schedule()
    reqs = [random_tokens(n, TINY["D"]["vocab_size"], 740 + i) for i, n in enumerate(lengths)]
    outs = {}
    for use in (True, False):
        eng = Engine.load(model_dirs["D"], dtype=dtype, max_tokens=2048, max_batch=8,
                          max_seq_len=512, use_graphs=use)
        outs[use] = run_schedule(eng, reqs, schedule)
        if use:
            assert eng.graphs.prompt_graphs and eng.graphs.decode_graphs
            s = eng.open_sequence()
            first = eng.step([(s, reqs[0][:7])], [[6]])
            kept = first.clone()
            second = eng.step([(s, reqs[0][7:8])], [[0]])
            third = eng.step([(s, reqs[0][8:9])], [[0]])
            kept2 = second.clone()
            eng.step([(s, reqs[0][9:16])], [[6]])
            assert torch.equal(first, kept) and torch.equal(second, kept2)
            assert first.data_ptr() != second.data_ptr() != third.data_ptr()
            eng.close_sequence(s)
        else:
            assert not eng.graphs.prompt_graphs and not eng.graphs.decode_graphs
        eng.check()
    for i, r in enumerate(reqs):
        assert_close(outs[True][i], oracle("D", r), dtype, f"captured, request {i}")
        assert_close(outs[False][i], oracle("D", r), dtype, f"launched one by one, request {i}")
        if dtype == "float32":
            assert torch.equal(outs[True][i], outs[False][i]), i


def test_tma_decode_attention_inside_the_engine(model_dirs, oracle, monkeypatch):
    """The decode attention whose tiles come by TMA is chosen from 128 (sequence, kv head)
    pairs up; forced here for every decode step, so that single sequences, small batches,
    sequences that end early and reused slots go through it inside the engine."""
    from grout_b200.engine import Engine
    from grout_b200.kernels import ops
    monkeypatch.setattr(ops, "DECODE_ATTENTION", "tma")
    eng = Engine.load(model_dirs["D"], dtype="bfloat16", max_tokens=4096, max_batch=8, max_seq_len=512)
    V = TINY["D"]["vocab_size"]
    toks = random_tokens(200, V, 1600)
    assert_close(run_tail_decoded(eng, toks, tail=80), oracle("D", toks), "bfloat16", "tma decode, one sequence")
    for b in range(2):
        plan = [(1, 20), (7, 2), (64, 5), (130, 33), (63, 3)]
        reqs = [random_tokens(p + d, V, 1610 + 10 * b + i) for i, (p, d) in enumerate(plan)]
        got = run_batch(eng, reqs, [p for p, _ in plan])
        for i, r in enumerate(reqs):
            assert_close(got[i], oracle("D", r), "bfloat16", f"tma decode, batch {b} request {i}")
    ops.check_kernel_errors()
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


def test_fp32_cuts_agree_tightly(engines):
    """Whole, tail-decoded and batched runs of the 32-bit path differ by rounding
    only; a looser agreement would point at the cache or the batch."""
    eng = engines("B", "float32")
    toks = random_tokens(100, TINY["B"]["vocab_size"], 500)
    other = random_tokens(37, TINY["B"]["vocab_size"], 501)
    whole = run_whole(eng, toks)
    tail = run_tail_decoded(eng, toks)
    batch = run_batch(eng, [other, toks], [5, 60])[1]
    assert (whole - tail).abs().max().item() < 2e-6
    assert (whole - batch).abs().max().item() < 2e-6


def test_padding_changes_nothing(engines):
    """A decode step through the captured graph (padded to a bucket) gives what
    the same step gives without a graph."""
    from grout_b200.engine import Engine
    eng = engines("A", "bfloat16")
    toks = [random_tokens(20 + i, 256, 600 + i) for i in range(3)]
    outs = []
    for use in (True, False):
        eng.use_graphs = use
        slots = [eng.open_sequence() for _ in toks]
        eng.step([(s, t[:-1]) for s, t in zip(slots, toks)])
        outs.append(eng.step([(s, [t[-1]]) for s, t in zip(slots, toks)],
                             [[0]] * 3).float().cpu())
        for s in slots:
            eng.close_sequence(s)
    eng.use_graphs = True
    assert torch.equal(outs[0], outs[1])


def test_prompt_products_on_pairs_of_sms_inside_the_engine(model_dirs, oracle):
    """With every prompt product on the 2-SM tcgen05 kernel (which the default only
    takes at sizes a tiny model never reaches): whole prompts, the tail decoded, and a
    batch, against the plain implementation."""
    from grout_b200.engine import Engine
    from grout_b200.kernels import ops
    from grout_b200.parts import ProductChoice
    eng = Engine.load(model_dirs["D"], dtype="bfloat16", max_tokens=4096, max_batch=8, max_seq_len=512,
                      products=ProductChoice(prefill="pair"))
    assert eng.model.blocks[0].mixer.qkv.prefill_kernel == "pair"
    reqs = [random_tokens(n, TINY["D"]["vocab_size"], 880 + n) for n in (400, 129, 70)]
    for r in reqs[:2]:
        assert_close(run_whole(eng, r), oracle("D", r), "bfloat16", "pair products, whole")
    assert_close(run_tail_decoded(eng, reqs[1], tail=20), oracle("D", reqs[1]), "bfloat16",
                 "pair products, tail decoded")
    got = run_batch(eng, reqs, [300, 100, 66])
    for g, r in zip(got, reqs):
        assert_close(g, oracle("D", r), "bfloat16", "pair products, batch")
    ops.check_kernel_errors()
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_across_a_bucket_of_lengths(tmp_path_factory, dtype):
    """Captured decode steps are kept per bound on the longest sequence (512, 1,024, ...).
    Two sequences decode from 505 and 40 tokens past 512: the steps before and after the
    boundary replay different graphs (with different splits of the attention over the
    keys), and every position must still equal the plain implementation."""
    import json
    import os
    from safetensors import safe_open
    from grout_b200.engine import Engine
    from grout_b200.weights import write_random_model
    cfg = dict(TINY["D"], max_position_embeddings=1100)
    d = write_random_model(cfg, 13, str(tmp_path_factory.mktemp("long")))
    with safe_open(os.path.join(d, "model.safetensors"), "pt") as f:
        w = {k: f.get_tensor(k) for k in f.keys()}
    raw = json.load(open(os.path.join(d, "config.json")))
    eng = Engine.load(d, dtype=dtype, max_tokens=2048, max_batch=4, max_seq_len=1100, use_graphs=True)
    reqs = [random_tokens(505 + 20, cfg["vocab_size"], 1500), random_tokens(40 + 20, cfg["vocab_size"], 1501)]
    got = run_batch(eng, reqs, [505, 40])
    for g, r in zip(got, reqs):
        assert_close(g, plain.logits(w, raw, r), dtype, "across the 512 boundary")
    assert {512, 1024} <= {length for _b, length in eng.graphs.decode_graphs}
    eng.check()
    eng.cache.check()
