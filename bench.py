#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-4B layer sizes with
random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W]

A "step" is one decode step of the whole batch (default 8 sequences that each
hold a 2,048-token prompt, context 4096).  ``value`` is decoded tokens per
second timed on the device with CUDA events over exactly K steps; ``regions``
cuts the same K steps into five consecutive regions (an event between them) and
gives the median and the quartiles of their times per step, in the manner of
the reference's repetitions (benchmarks/src/bin/grout_bench.rs:218-252);
``e2e`` is the same through ``Engine.generate`` with host token lists in and
out.  The line also carries the 2,048-token prefill, the decode step's HBM
roofline and decode at batch 1 and 64.  Every decode step reads the 8 GB of
weights, far more than the 126 MB L2, so nothing is flushed between timed steps.

    python bench.py --size 8b|32b      the same run at the other sizes of the workload list
    python bench.py --ops [--size S] [--batch B]
                                       a table of every kernel of one prompt step and of
                                       decode steps (launched one by one, an event pair
                                       around each): calls, time, GB/s, TFLOP/s, fractions
    python bench.py --requests S       the reference's request grid
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_4B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936,
                hidden_size=2560, intermediate_size=9728, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=1000000.0,
                rms_norm_eps=1e-6, max_position_embeddings=40960, tie_word_embeddings=True,
                use_sliding_window=False, eos_token_id=151645)
# The other two model sizes of the workload list, for --requests (layer sizes only; the
# default run and its contract stay with the 4B sizes).
SIZES = {
    "4b": QWEN3_4B,
    "8b": dict(QWEN3_4B, hidden_size=4096, intermediate_size=12288, tie_word_embeddings=False),
    "32b": dict(QWEN3_4B, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64,
                num_attention_heads=64, tie_word_embeddings=False),
}
# What the reference publishes for Qwen3-32B on a B200 (fp16, batch 1, its own engine):
# request_gen_tps = generated tokens / seconds of the whole request, and one prefill time
# (benchmarks/RESULTS.md:29-31, 45-47, 53-55).  (prompt tokens, generated tokens) -> figure.
PUBLISHED_32B = {(18, 36): 79.6, (18, 128): 79.9, (18, 512): 80.1, (128, 36): 79.0, (512, 36): 75.3,
                 (2048, 36): 61.4, (8192, 36): 37.2}
PUBLISHED_32B_PREFILL_MS = {8192: 513.78}
CONTEXT = 4096
PROMPT = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
SETTLE_S = 0.5      # idle between a batch's prompts and its decode steps (see decode_run)
REGIONS = 5


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as fh:
                p = json.load(fh)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6
                          for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": int(statistics.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons}


def weight_bytes(cfg, layers):
    H, D = cfg["hidden_size"], cfg["head_dim"]
    nq, nkv, I, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"], cfg["vocab_size"]
    per_layer = (nq + 2 * nkv) * D * H + nq * D * H + 3 * H * I + 2 * H + 2 * D
    return 2 * (layers * per_layer + V * H + H)          # bf16; the head reads the table once


def kv_bytes_per_token(cfg, layers):
    return layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, layers, T):
    H, D = cfg["hidden_size"], cfg["head_dim"]
    nq, nkv, I, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"], cfg["vocab_size"]
    linear = 2 * T * ((nq + 2 * nkv) * D * H + nq * D * H + 3 * H * I)
    attn = 2 * 2 * nq * D * T * (T + 1) // 2
    return layers * (linear + attn) + 2 * V * H


def run_requests(size: str, reps: int) -> int:
    """The reference's own request grid (one sequence: prompt of P tokens, T tokens generated,
    EOS ignored) through ``Engine.generate`` with random weights of the named size and random
    token ids: generated tokens per second of the whole request, host tokens in and out; the
    median of ``reps`` requests after two that are discarded, half a second apart."""
    import torch
    from grout_b200.engine import Engine
    cfg = SIZES[size]
    eng = Engine.random(cfg, 0, dtype="bfloat16", max_tokens=8192 + 576, max_batch=1,
                        max_seq_len=8192 + 512 + 64)
    g = torch.Generator().manual_seed(1)

    def prompt(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()

    cells = []
    for pp, tg in sorted(PUBLISHED_32B):
        runs = []
        for i in range(reps + 2):
            time.sleep(0.5)
            o = eng.generate([prompt(pp)], tg, ignore_eos=True)[0]
            if i >= 2:
                runs.append((o.generated_tokens / o.total_elapsed, o.prompt_elapsed * 1e3,
                             o.decode_phase_tps()))
        cell = {"prompt": pp, "generate": tg,
                "request_gen_tps": round(statistics.median(r[0] for r in runs), 1),
                "prefill_ms": round(statistics.median(r[1] for r in runs), 2),
                "decode_phase_tps": round(statistics.median(r[2] for r in runs), 1)}
        if size == "32b":
            cell["published_request_gen_tps"] = PUBLISHED_32B[(pp, tg)]
            if pp in PUBLISHED_32B_PREFILL_MS:
                cell["published_prefill_ms"] = PUBLISHED_32B_PREFILL_MS[pp]
        cells.append(cell)
    eng.check()
    print(json.dumps({"metric": f"request_gen_tps, one sequence, Qwen3-{size.upper()} layer sizes",
                      "unit": "tok/s", "dtype": "bf16", "data": "synthetic", "reps": reps,
                      "layers": cfg["num_hidden_layers"], "cells": cells}))
    return 0


def quartiles(xs):
    xs = sorted(xs)
    q = statistics.quantiles(xs, n=4, method="inclusive") if len(xs) > 1 else [xs[0]] * 3
    return q[0], q[1], q[2]


def run_ops(size: str, batch: int, layers: int, pk) -> int:
    """One prompt step of 2,048 tokens launched kernel by kernel with an event pair
    around each (the table of ``ops.OpProfile``: every kernel alone on the device),
    and the decode step of ``batch`` sequences as it runs inside its captured graph
    (``decode_timeline``)."""
    import torch
    from grout_b200.engine import Engine
    from grout_b200.kernels import ops
    cfg = dict(SIZES[size], num_hidden_layers=layers)
    eng = Engine.random(cfg, 0, dtype="bfloat16", max_tokens=batch * (PROMPT + 128),
                        max_batch=batch, max_seq_len=CONTEXT)
    eng.use_graphs = False
    g = torch.Generator().manual_seed(1)
    V = cfg["vocab_size"]

    def prompt():
        return torch.randint(0, V, (PROMPT,), generator=g).tolist()

    slots = [eng.open_sequence() for _ in range(batch)]
    eng.step([(slots[0], prompt())], [[PROMPT - 1]])                  # warm-up of every prompt kernel
    eng.close_sequence(slots[0])
    slots[0] = eng.open_sequence()
    prof = ops.OpProfile(pk["hbm_gbs"], pk["bf16_tflops"])
    ops.set_profile(prof)
    eng.step([(slots[0], prompt())], [[PROMPT - 1]])
    ops.set_profile(None)
    print(f"== prompt step, {PROMPT} tokens, Qwen3-{size.upper()} layer sizes, {layers} layers "
          f"(peaks: {pk['source']}, {pk['hbm_gbs']:.0f} GB/s, {pk['bf16_tflops']:.0f} TFLOP/s burst)")
    print(prof.report())
    for i in range(1, batch, 8):
        eng.step([(s, prompt()) for s in slots[i:i + 8]])
    eng.check()
    print(decode_timeline(eng, slots, V, g, pk))
    return 0


def decode_timeline(eng, slots, V, g, pk, steps: int = 3) -> str:
    """The kernels of a captured decode step as they ran inside it, from the activity
    records of the CUDA profiling interface (torch.profiler): per kernel its calls a
    step, its mean duration, and its mean *exposed* time, which is how much later it
    ended than everything before it (kernels overlap at their edges: a kernel is
    resident, fetching what no earlier kernel writes, while its predecessor drains).
    The exposed times add up to the step.  Times taken under the profiler's tracing:
    a breakdown, not a benchmark figure."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from grout_b200.kernels import ops
    batch = len(slots)
    eng.use_graphs = True
    tok = torch.randint(0, V, (batch,), generator=g).tolist()

    def step():
        eng.step([(s, [t]) for s, t in zip(slots, tok)], [[0]] * batch)

    # the capture of the step's graph (a warm-up pass and the captured pass) says, launch by
    # launch, which product each kernel of the step is; kernel names alone do not
    eng.graphs.decode_graphs.clear()
    ops.LAUNCH_LOG = []
    step()
    graph = eng.graphs.decode(batch, max(eng.cache.length[s] for s in slots))
    labels = ops.LAUNCH_LOG[-graph.kernels_per_replay:]         # the captured pass
    ops.LAUNCH_LOG = None
    for _ in range(5):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            step()
        torch.cuda.synchronize()
    ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
                 and "memcpy" not in e.name.lower() and "memset" not in e.name.lower()),
                key=lambda e: e.time_range.start)
    starts = [i for i, e in enumerate(ev) if "embed_kernel" in e.name]
    rows, total = {}, 0.0
    for a, b in zip(starts, starts[1:] + [len(ev)]):
        frontier = ev[a].time_range.start
        named = len(labels) == b - a
        for k, e in enumerate(ev[a:b]):
            end = e.time_range.end
            name = labels[k] if named else e.name.split("(")[0].replace("void ", "")
            r = rows.setdefault(name, [0, 0.0, 0.0])
            r[0] += 1
            r[1] += end - e.time_range.start
            r[2] += max(0.0, end - frontier)
            frontier = max(frontier, end)
        total += frontier - ev[a].time_range.start
    n = len(starts)
    if n and len(labels) != len(ev) // n:
        print(f"bench.py: {len(labels)} launches were logged for a step of {len(ev) // n} kernels; "
              f"rows are named by kernel", file=sys.stderr)
    kv = sum(eng.cache.length[s] for s in slots)
    cfg = eng.config

    def must_read(name):
        """Bytes a call of this kernel has to read: a product its weights, the decode
        attention the keys and values of the live sequences (one layer's)."""
        part = name.split()
        if part[0] == "gemm_tc_bf16" and len(part) > 1 and "x" in part[1]:
            rows_w, cols_w = part[1].split("x")
            return 2.0 * int(rows_w) * int(cols_w)
        if part[0].startswith("attn_decode") and "second" not in name:
            return 2.0 * kv * 2 * cfg.num_key_value_heads * cfg.head_dim
        return None

    lines = [f"== decode step, batch {batch}, {kv // batch} keys a sequence, as it ran inside the captured "
             f"graph ({n} steps traced): {total / n:.1f} us a step; GB/s = what the kernel has to read / "
             f"its exposed time, of the {pk['source']} {pk['hbm_gbs']:.0f} GB/s",
             f"  {'kernel':<36}{'calls/step':>11}{'mean_us':>9}{'exposed_us':>11}{'per step':>10}{'share':>7}"
             f"{'GB/s':>8}{'of hbm':>8}"]
    for name, (calls, dur, exposed) in sorted(rows.items(), key=lambda kv: -kv[1][2]):
        line = (f"  {name[:35]:<36}{calls / n:>11.1f}{dur / calls:>9.2f}{exposed / calls:>11.2f}"
                f"{exposed / n:>10.1f}{exposed / total:>7.1%}")
        nbytes = must_read(name)
        if nbytes and exposed > 0:
            gbs = nbytes / (exposed / calls * 1e-6) / 1e9
            line += f"{gbs:>8.0f}{gbs / pk['hbm_gbs']:>8.2f}"
        lines.append(line)
    return "\n".join(lines)


def main() -> int:
    global PROMPT, CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--size", default="4b", choices=sorted(SIZES),
                    help="layer sizes of the run (default: the 4B sizes the contract names)")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT,
                    help="tokens every sequence holds before decoding, and of the timed prompt step "
                         "(default: the 2,048 the contract names; other lengths for the profiles)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--phases", default="prefill,decode,points,e2e",
                    help="which measurements to run (a profiler wants one at a time)")
    ap.add_argument("--requests", default=None, choices=sorted(SIZES),
                    help="instead of the default run: the reference's request grid at this model size")
    ap.add_argument("--reps", type=int, default=5, help="measured requests per cell of --requests")
    ap.add_argument("--ops", action="store_true",
                    help="instead of the default run: the per-kernel table of a prompt step and of "
                         "decode steps at --size and --batch")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "NikVisel/grout is a Rust crate (Cargo.toml, no Python packaging); pip "
                          "cannot install it offline and no Rust toolchain or crates are present"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.requests:
        return run_requests(args.requests, max(1, args.reps))
    if args.prompt_len != PROMPT:
        if not 1 <= args.prompt_len <= 36864:
            print("bench.py: --prompt-len must be 1..36864", file=sys.stderr)
            return 2
        PROMPT = args.prompt_len
        CONTEXT = max(CONTEXT, (PROMPT + 2048 + 63) // 64 * 64)
    full_layers = SIZES[args.size]["num_hidden_layers"]
    layers = args.layers or full_layers
    pk = peaks()
    if args.ops:
        return run_ops(args.size, args.batch, layers, pk)
    W = max(args.warmup, 3)
    K = args.steps
    most = CONTEXT - PROMPT - W - 4      # the sequences hold 2,048 prompt tokens in a context of 4,096
    if K < 1 or K > most:
        print(f"bench.py: --steps must be 1..{most} with --warmup {W} (prompt {PROMPT}, context "
              f"{CONTEXT}); got {K}", file=sys.stderr)
        return 2
    phases = set(args.phases.split(","))
    if args.no_points:
        phases.discard("points")

    import torch
    from grout_b200.engine import Engine
    from grout_b200.kernels import ops

    cfg = dict(SIZES[args.size], num_hidden_layers=layers)
    torch.manual_seed(0)
    room = PROMPT + max(W + K, 129) + 64
    point_batches = [1, 64] if "points" in phases else []
    # (a cache for 64 sequences of a long prompt does not fit beside the weights: such a
    # run keeps the batch-1 point only)
    if 64 * room * kv_bytes_per_token(cfg, layers) > 100e9:
        point_batches = [b for b in point_batches if b * room * kv_bytes_per_token(cfg, layers) <= 100e9]
    biggest = max([args.batch] + point_batches)
    eng = Engine.random(cfg, 0, dtype="bfloat16", max_tokens=biggest * ((room + 63) // 64 * 64),
                        max_batch=biggest, max_seq_len=CONTEXT)
    g = torch.Generator().manual_seed(1)
    V = cfg["vocab_size"]

    def prompt():
        return torch.randint(0, V, (PROMPT,), generator=g).tolist()

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---- prefill of 2,048 tokens ---------------------------------------------------
    p = prompt()
    times = []
    for i in range(9 if "prefill" in phases else 0):      # three to warm up, the median of six
        s = eng.open_sequence()
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        eng.step([(s, p)], [[PROMPT - 1]])
        b.record()
        torch.cuda.synchronize()
        eng.close_sequence(s)
        if i >= 3:
            times.append(a.elapsed_time(b))
    prefill = None
    if times:
        pre_ms = statistics.median(times)
        rate = prefill_flops(cfg, layers, PROMPT) / (pre_ms * 1e-3) / 1e12
        # the step's flops / time / the peak of its dtype: against the burst peak (a product
        # timed alone) and against the sustained one (nine prompt steps back to back run at
        # the clocks of the power cap, as that peak was taken)
        prefill = {"value": round(PROMPT / pre_ms * 1e3, 1), "tokens": PROMPT, "ms": round(pre_ms, 3),
                   "frac": round(rate / pk["bf16_tflops"], 4),
                   "frac_sustained": round(rate / pk["bf16_tflops_sustained"], 4),
                   "tflops": round(rate, 1), "of": pk["source"]}

    # ---- decode --------------------------------------------------------------------
    def decode_run(batch, steps, warm, sample_clocks=False):
        slots = [eng.open_sequence() for _ in range(batch)]
        group = max(1, min(8, 16384 // PROMPT))            # prompts go in, 16,384 tokens at a time
        for i in range(0, batch, group):
            eng.step([(s, prompt()) for s in slots[i:i + group]])
        # the decode step as generation runs it: tokens chosen on the device (greedy)
        # feed the next step, which is queued without waiting for the host
        first = torch.randint(0, V, (batch,), generator=g).tolist()
        logits = eng.step([(s, [first[j]]) for j, s in enumerate(slots)], [[0]] * batch)
        # The prompts leave the GPU at the reduced clocks of its power cap, and it raises
        # them again over some thirty decode steps; the decode step is measured at the
        # clocks it settles at, so the GPU idles for half a second first.  (``e2e`` below
        # has no such pause: it is the request as a user runs it.)
        torch.cuda.synchronize()
        time.sleep(SETTLE_S)
        greedy = [eng.default_sampling()] * batch
        entries = [(s, j) for j, s in enumerate(slots)]
        for i in range(warm):
            logits = eng.step_ahead(entries, eng.choose_ahead(logits, greedy, [0.0] * batch))
        torch.cuda.synchronize()
        clocks = ClockSampler() if sample_clocks else None
        if clocks:
            clocks.start()
        before = ops.launch_count()
        cuts = sorted({round(steps * r / REGIONS) for r in range(1, REGIONS)} - {0, steps})
        marks = [ev()]
        marks[0].record()
        for i in range(steps):
            logits = eng.step_ahead(entries, eng.choose_ahead(logits, greedy, [0.0] * batch))
            if i + 1 in cuts:
                marks.append(ev())
                marks[-1].record()
        marks.append(ev())
        marks[-1].record()
        torch.cuda.synchronize()
        ms = marks[0].elapsed_time(marks[-1])
        bounds = [0] + cuts + [steps]
        per_step = [a.elapsed_time(b) / (hi - lo)
                    for a, b, lo, hi in zip(marks, marks[1:], bounds, bounds[1:])]
        launches = ops.launch_count() - before
        graph = eng.graphs.decode(batch, PROMPT + warm + steps + 1)
        if graph is not None and graph.graph is not None:
            launches += steps * graph.kernels_per_replay
        ctx_mid = PROMPT + warm + steps / 2.0
        for s in slots:
            eng.close_sequence(s)
        return ms, launches, ctx_mid, (clocks.stop() if clocks else None), per_step

    def step_bytes(batch, ctx):
        return weight_bytes(cfg, layers) + batch * ctx * kv_bytes_per_token(cfg, layers)

    ms, launches, ctx_mid, clocks, per_step = decode_run(args.batch, K, W, sample_clocks=True)
    value = args.batch * K / ms * 1e3
    achieved = step_bytes(args.batch, ctx_mid) / (ms / K * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]}
    q1, med, q3 = quartiles(per_step)
    regions = {"n": len(per_step), "ms_per_step_median": round(med, 4),
               "ms_per_step_q1": round(q1, 4), "ms_per_step_q3": round(q3, 4),
               "value_at_median": round(args.batch / med * 1e3, 1)}

    points = {}
    if point_batches:
        for bsz in point_batches:
            m, _l, c, _, _p = decode_run(bsz, 32, 4)
            points[f"decode_b{bsz}"] = round(bsz * 32 / m * 1e3, 1)
            points[f"decode_b{bsz}_hbm_frac"] = round(
                step_bytes(bsz, c) / (m / 32 * 1e-3) / 1e9 / pk["hbm_gbs"], 4)

    # ---- end to end through the Python entry point -----------------------------------
    e2e = None
    if "e2e" in phases:
        # at least 128 decode steps: the first thirty after the prompts run at the clocks the
        # power cap left behind, and a request of a few tokens would measure little else
        n_new = max(K, 128) + 1
        prompts = [prompt() for _ in range(args.batch)]
        eng.generate(prompts, 4, ignore_eos=True)              # warm-up
        outs = eng.generate(prompts, n_new, ignore_eos=True)
        e2e_tps = sum(o.generated_tokens - 1 for o in outs) / outs[0].decode_elapsed
        graph = eng.graphs.decode(args.batch, PROMPT + n_new)
        h2d = int(graph.dev.numel() * 4) if graph is not None else 0
        e2e = {"value": round(e2e_tps, 1), "unit": "tok/s", "steps": n_new - 1, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": 4 * args.batch}

    eng.check()      # a kernel that gave up on a bounded wait would have voided the numbers
    name = f"Qwen3-{args.size.upper()}"
    print(json.dumps({
        "metric": f"decode tok/s ({name} shape, batch {args.batch}, 2,048-token prompts)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": f"{name} layer sizes, random weights", "layers": layers,
                   "layers_of_config": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                   "vocab": V, "global_batch": args.batch, "seq_len": CONTEXT,
                   "prompt_len": PROMPT, "tied_head": bool(cfg["tie_word_embeddings"]),
                   "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 ({weight_bytes(cfg, layers) / 1e9:.0f} GB of weights "
                         f"per step), no flush",
                   "settle_s": SETTLE_S, "peaks": pk["source"]},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "prefill": prefill,
        "roofline": roofline, "regions": regions, "points": points}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
