"""Command line in the manner of the reference's ``grout`` binary
(src/main.rs:13-65 for the options, 96-153 for what is printed) with the
timing options of its bench binary (benchmarks/src/bin/grout_bench.rs:49-94).

    python -m grout_b200 --model DIR --prompt "Hello" --max-new-tokens 64
    python -m grout_b200 --model DIR --prompt-ids 1,2,3 --sample --temperature 0.8 --seed 1
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

IM_START, IM_END = "<|im_start|>", "<|im_end|>"


def apply_chat_template(prompt: str) -> str:
    """The reference's literal ChatML wrapper with an empty thinking block
    (src/model.rs:2198-2210); a prompt that already holds the start marker is
    left alone."""
    if IM_START in prompt:
        return prompt
    return (f"{IM_START}user\n{prompt}{IM_END}\n{IM_START}assistant\n"
            f"<think>\n\n</think>\n\n")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="grout_b200", description="Qwen3 dense text generation on one B200")
    ap.add_argument("--model", required=True,
                    help="model folder (config.json, safetensors), or random:CONFIG.json for "
                         "random weights made on the device from --seed (with --prompt-ids)")
    g = ap.add_mutually_exclusive_group(required=True)
    g.add_argument("--prompt", help="text; needs tokenizer.json in the model folder")
    g.add_argument("--prompt-ids", help="comma-separated token ids, bypassing the tokenizer")
    ap.add_argument("--max-new-tokens", type=int, default=128)
    ap.add_argument("--max-seq-len", type=int, default=None,
                    help="context limit; default min(4096, max_position_embeddings)")
    ap.add_argument("--sample", action="store_true", help="sample instead of greedy decoding")
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--raw-prompt", action="store_true", help="skip the chat template")
    ap.add_argument("--device-argmax", action="store_true",
                    help="choose tokens on the GPU (otherwise logits are copied back and the "
                         "host chooses)")
    ap.add_argument("--profile", action="store_true", help="print step counts and device times")
    ap.add_argument("--profile-ops", action="store_true",
                    help="with --profile: time every operation too (calls, time, GB/s, TFLOP/s per "
                         "kernel).  Steps are then launched kernel by kernel instead of replayed from "
                         "graphs, so the step times of this run are not the engine's.  The environment "
                         "variable GROUT_PROFILE_OPS=1 does the same (src/model.rs:1139)")
    ap.add_argument("--peaks", default=None, metavar="FILE",
                    help="JSON with hbm_gbs and bf16_tflops: the op profile then gives each kernel's "
                         "fraction of them")
    ap.add_argument("--warmup-reps", type=int, default=1,
                    help="discarded generations before the measured one")
    ap.add_argument("--ignore-eos", action="store_true", help="generate the whole budget")
    ap.add_argument("--reps", type=int, default=1,
                    help="measured generations; each prints its times (grout_bench.rs:49-50)")
    ap.add_argument("--json", default=None, metavar="FILE",
                    help="append one JSON object per measured generation to FILE (JSON lines, "
                         "the keys of grout_bench.rs:60-66)")
    ap.add_argument("--variant", default="default", help="label of the `variant` field of --json")
    ap.add_argument("--quiet", action="store_true",
                    help="do not print the generated text or the profile, only the times")
    ap.add_argument("--fp32", action="store_true", help="run the true 32-bit path")
    ap.add_argument("--output-json", default=None, help="write token ids, counts and seconds here")
    ap.add_argument("--device", default="cuda:0")
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    from .engine import Engine
    from .engine.profile import StepProfile
    from .sampling import SamplingParams

    tokenizer = None
    random_config = args.model[len("random:"):] if args.model.startswith("random:") else None
    if random_config is not None and args.prompt is not None:
        print("error: random weights have no tokenizer; use --prompt-ids", file=sys.stderr)
        return 2
    if args.prompt is not None:
        path = os.path.join(args.model, "tokenizer.json")
        if not os.path.exists(path):
            print(f"error: --prompt needs {path}; use --prompt-ids instead", file=sys.stderr)
            return 2
        from tokenizers import Tokenizer
        tokenizer = Tokenizer.from_file(path)
        text = args.prompt
        vocab = tokenizer.get_vocab(True)
        if not args.raw_prompt and IM_START in vocab and IM_END in vocab:   # src/model.rs:1336-1338
            text = apply_chat_template(text)
        prompt_ids = tokenizer.encode(text, add_special_tokens=True).ids
    else:
        try:
            prompt_ids = [int(t) for t in args.prompt_ids.replace(" ", "").split(",") if t != ""]
        except ValueError:
            print("error: --prompt-ids takes comma-separated integers", file=sys.stderr)
            return 2

    dtype = "float32" if args.fp32 else "bfloat16"
    if random_config is not None:
        with open(random_config, encoding="utf-8") as fh:
            engine = Engine.random(json.load(fh), args.seed, dtype=dtype, device=args.device,
                                   max_seq_len=args.max_seq_len, max_batch=1)
    else:
        engine = Engine.load(args.model, dtype=dtype, device=args.device,
                             max_seq_len=args.max_seq_len, max_batch=1)
    base = engine.default_sampling(args.sample, args.seed)
    sampling = SamplingParams(args.sample,
                              args.temperature if args.temperature is not None else base.temperature,
                              args.top_k if args.top_k is not None else base.top_k,
                              args.top_p if args.top_p is not None else base.top_p,
                              args.seed).normalised()
    print(f"Loaded model from {args.model}")
    print(f"Prompt: {args.prompt if args.prompt is not None else prompt_ids}")
    print(f"Generating {args.max_new_tokens} tokens...")

    def run(n):
        return engine.generate([prompt_ids], n, sampling=sampling, ignore_eos=args.ignore_eos,
                               device_argmax=args.device_argmax)[0]

    for _ in range(args.warmup_reps):          # src/main.rs:101-110
        run(min(args.max_new_tokens, 8))
    op_profile = None
    if args.profile:
        engine.profile = StepProfile()
        if args.profile_ops or os.environ.get("GROUT_PROFILE_OPS") == "1":
            from .kernels import ops
            peaks = {}
            if args.peaks:
                with open(args.peaks, encoding="utf-8") as fh:
                    peaks = json.load(fh)
            op_profile = ops.OpProfile(peaks.get("hbm_gbs"), peaks.get("bf16_tflops"))
            engine.use_graphs = False
            ops.set_profile(op_profile)
    reps = max(1, args.reps)
    for i in range(reps):                      # benchmarks/src/bin/grout_bench.rs:96-110, 150-190
        out = run(args.max_new_tokens)
        if reps > 1 or args.json:
            print(f"  run {i + 1}/{reps}: prompt_tokens={out.prompt_tokens}, "
                  f"gen_tokens={out.generated_tokens}, prefill_ms={out.prompt_elapsed * 1e3:.2f}, "
                  f"decode_ms={out.decode_elapsed * 1e3:.2f}, e2e_ms={out.total_elapsed * 1e3:.2f}, "
                  f"decode_phase_tps={out.decode_phase_tps():.1f}, e2e_tps={out.total_tps():.1f}")
        if args.json:
            with open(args.json, "a", encoding="utf-8") as fh:
                fh.write(json.dumps({"engine": "grout_b200", "variant": args.variant,
                                     "pp": out.prompt_tokens, "tg": args.max_new_tokens, "rep": i,
                                     "prompt_tokens": out.prompt_tokens,
                                     "gen_tokens": out.generated_tokens,
                                     "prefill_ms": out.prompt_elapsed * 1e3,
                                     "decode_ms": out.decode_elapsed * 1e3,
                                     "e2e_ms": out.total_elapsed * 1e3}) + "\n")
    text = tokenizer.decode(out.token_ids, skip_special_tokens=False) if tokenizer else None
    if not args.quiet:
        print()
        print(text if text is not None else " ".join(str(t) for t in out.token_ids))
    print(f"t/s: {out.prompt_tps():.2f} prompt, {out.decode_phase_tps():.2f} decode phase, "
          f"{out.total_tps():.2f} end-to-end (prompt_tokens={out.prompt_tokens}, "
          f"generated_tokens={out.generated_tokens}, prompt_s={out.prompt_elapsed:.3f}, "
          f"decode_s={out.decode_elapsed:.3f}, total_s={out.total_elapsed:.3f})")
    if args.profile and not args.quiet:
        print()
        print(engine.profile.report())
        if op_profile is not None:
            print(op_profile.report())
    if args.output_json:
        with open(args.output_json, "w", encoding="utf-8") as fh:
            json.dump({"text": text, "token_ids": out.token_ids, "prompt_tokens": out.prompt_tokens,
                       "generated_tokens": out.generated_tokens, "finish_reason": out.finish_reason,
                       "total_seconds": out.total_elapsed}, fh, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
