"""Command line: generate from token ids, or write a model folder with random weights.

    python -m llmengine --model DIR --prompt-ids 1,2,3 --max-new 16
    python -m llmengine --model DIR --prompt-len 128 --requests 8 --max-new 32 --budget 256 --dtype bf16
    python -m llmengine --random-weights OUT_DIR --config config.json --seed 0 --dtype bf16

Option names follow the reference's own scripts where it has them: --dtype, --requests, --max-new
and --budget are those of benchmarks/bench_throughput.py (:93-115), and the environment variables
LLMENGINE_MODEL and LLMENGINE_DTYPE those of its server (python/llmengine/server.py:78-79). The
reference has no command that generates from the command line; --prompt-ids, --prompt-len,
--temperature, --seed, --max-concurrent, --block-size, --num-blocks and --random-weights are
added here. There is no tokenizer: prompts are token ids. Results are printed as JSON lines, one
per request, then one line with prefill and decode tokens a second measured as the reference's
bench_e2e.py does (generate(prompt, 0) as prefill time, the rest as decode time).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="python -m llmengine", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default=os.environ.get("LLMENGINE_MODEL"), help="folder with config.json and *.safetensors")
    ap.add_argument("--dtype", default=os.environ.get("LLMENGINE_DTYPE", "fp32"), choices=["fp32", "bf16"])
    ap.add_argument("--prompt-ids", help="comma-separated token ids of one prompt")
    ap.add_argument("--prompt-len", type=int, help="use random prompts of this many token ids instead")
    ap.add_argument("--requests", type=int, default=1, help="number of random prompts (with --prompt-len)")
    ap.add_argument("--max-new", "--max-new-tokens", dest="max_new", type=int, default=16, help="tokens to generate per request")
    ap.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    ap.add_argument("--seed", "--sample-seed", dest="seed", type=int, default=0, help="seed of sampling and of random prompts / weights")
    ap.add_argument("--budget", "--max-prefill-tokens-per-step", dest="budget", type=int, default=256, help="prefill tokens per scheduler step")
    ap.add_argument("--max-concurrent", type=int, default=64)
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--num-blocks", type=int, default=None, help="pages in the pool (default: sized from free memory)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--random-weights", metavar="OUT_DIR", help="write a model folder with random weights and exit")
    ap.add_argument("--config", help="config.json for --random-weights")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import torch

    import llmengine

    if args.random_weights:
        if not args.config:
            print("--random-weights needs --config", file=sys.stderr)
            return 2
        with open(args.config) as f:
            cfg = json.load(f)
        dt = torch.bfloat16 if args.dtype == "bf16" else torch.float32
        llmengine.write_random_model(args.random_weights, cfg, seed=args.seed, dtype=dt)
        print(json.dumps({"wrote": args.random_weights, "dtype": args.dtype, "seed": args.seed}))
        return 0
    if not args.model:
        print("--model (or LLMENGINE_MODEL) is required", file=sys.stderr)
        return 2
    eng = llmengine.Engine(args.model, args.dtype, device=args.device, block_size=args.block_size,
                           num_blocks=args.num_blocks, max_concurrent=args.max_concurrent)
    vocab = eng.cfg.vocab_size
    if args.prompt_ids:
        prompts = [[int(t) for t in args.prompt_ids.split(",") if t.strip()]]
    elif args.prompt_len:
        g = torch.Generator().manual_seed(args.seed)
        prompts = torch.randint(0, vocab, (args.requests, args.prompt_len), generator=g).tolist()
    else:
        print("give --prompt-ids or --prompt-len", file=sys.stderr)
        return 2
    try:
        if len(prompts) == 1:
            eng.generate(prompts[0], 0)  # warm-up: weights, kernels
            t0 = time.perf_counter()
            eng.generate(prompts[0], 0)
            prefill_s = time.perf_counter() - t0
            t0 = time.perf_counter()
            toks, reason = eng.generate(prompts[0], args.max_new, temperature=args.temperature, seed=args.seed)
            total_s = time.perf_counter() - t0
            print(json.dumps({"seq_id": 0, "prompt_len": len(prompts[0]), "token_ids": toks, "finish_reason": reason}))
            n_new = len(toks) - len(prompts[0])
            print(json.dumps({"prefill_tok_s": round(len(prompts[0]) / prefill_s, 1),
                              "decode_tok_s": round(n_new / max(total_s - prefill_s, 1e-9), 1) if n_new else None}))
        else:
            sch = llmengine.ContinuousBatchScheduler(eng, None, max_concurrent=args.max_concurrent,
                                                     max_prefill_tokens_per_step=args.budget)
            for i, p in enumerate(prompts):
                sch.enqueue(p, args.max_new, temperature=args.temperature, seed=args.seed + i)
            t0 = time.perf_counter()
            sch.run_until_idle()
            wall = time.perf_counter() - t0
            gen = 0
            for r in sch.results:
                gen += len(r.token_ids) - r.prompt_len
                print(json.dumps({"seq_id": r.seq_id, "prompt_len": r.prompt_len, "token_ids": list(r.token_ids),
                                  "finish_reason": r.finish_reason}))
            print(json.dumps({"requests": len(prompts), "generated": gen, "seconds": round(wall, 4),
                              "aggregate_tok_s": round(gen / wall, 1), "steps": sch.steps}))
    except (ValueError, RuntimeError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0
