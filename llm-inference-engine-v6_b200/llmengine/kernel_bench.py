"""Single-kernel runs for timing and profiling.

    python -m llmengine.kernel_bench gemm --m 8 --n 16384 --k 2048 [--reps 20]
    python -m llmengine.kernel_bench attention --batch 8 --context 2048 --new 1
    python -m llmengine.kernel_bench attention --batch 1 --context 0 --new 2048

Each run launches ONE kind of kernel a few times on inputs that are larger than the L2 cache
(several copies of the operands are used in turn) and prints the mean device time per launch with
the bytes and flops it implies. The sizes default to the Llama 3.2 1B geometry. Meant to be run
alone or under a profiler with a small --reps.
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch


def _time(fn, reps: int) -> float:
    for _ in range(3):
        fn(0)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(reps):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e-3 / reps


def run_gemm(args) -> dict:
    from .engine.context import Workspace
    from .ops import get_ops
    ops = get_ops()
    dev = torch.device("cuda:0")
    M, N, K = args.m, args.n, args.k
    copies = max(2, int(300e6 // (N * K * 2)) + 1)  # weights rotate through > 2x the L2 size
    ws = [(torch.randn(N, K, device=dev) * 0.02).bfloat16() for _ in range(copies)]
    a = torch.randn(M, K, device=dev).bfloat16()
    space = Workspace(dev)
    sec = _time(lambda i: ops.gemm_partials(a, ws[i % copies], space, "bench"), args.reps)
    parts = ops.gemm_partials(a, ws[0], space, "bench")
    assert ops.tensor_core_error() == 0
    flops, nbytes = 2.0 * M * N * K, N * K * 2 + M * K * 2 + parts.numel() * 4
    return {"kernel": "gemm_tc", "M": M, "N": N, "K": K, "k_splits": parts.shape[0], "us": round(sec * 1e6, 2),
            "tflops": round(flops / sec / 1e12, 1), "gbs": round(nbytes / sec / 1e9, 1)}


class _Batch:
    pass


def run_attention(args) -> dict:
    from .engine.context import Workspace
    from .ops import get_ops
    ops = get_ops()
    dev = torch.device("cuda:0")
    nq, nkv, hd, page = args.heads, args.kv_heads, args.head_dim, args.page
    B, ctx, new = args.batch, args.context, args.new
    total = ctx + new
    blocks = (total + page - 1) // page
    layers = max(2, int(300e6 // max(B * total * nkv * hd * 4, 1)) + 1)  # caches of several "layers" in turn
    n_pages = B * blocks
    caches = [(torch.randn(n_pages + 1, nkv, page, hd, device=dev).bfloat16(), torch.randn(n_pages + 1, nkv, page, hd, device=dev).bfloat16())
              for _ in range(layers)]
    table = torch.randperm(n_pages, device=dev).to(torch.int32).view(B, blocks).contiguous()
    b = _Batch()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    b.seq_start, b.seq_ntok = i32([ctx] * B), i32([new] * B)
    b.seq_qoff = i32([i * new for i in range(B + 1)])
    b.positions = i32([ctx + j for _ in range(B) for j in range(new)])
    b.token_seq = i32([i for i in range(B) for _ in range(new)])
    b.n_tokens, b.n_seqs, b.max_new_tokens, b.max_seq_len = B * new, B, new, total
    b.ws = Workspace(dev)
    q = torch.randn(B * new, nq * hd, device=dev).bfloat16()
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(hd)
    sec = _time(lambda i: ops.paged_attention(q, caches[i % layers][0], caches[i % layers][1], b, table, out, nq, nkv, hd, scale), args.reps)
    keys = sum(ctx + j + 1 for j in range(new)) * B  # (query, key) pairs per head
    flops = 4.0 * keys * nq * hd
    nbytes = 2.0 * B * total * nkv * hd * 2
    return {"kernel": "paged_attention", "batch": B, "context": ctx, "new_tokens": new, "heads": nq, "kv_heads": nkv,
            "head_dim": hd, "us": round(sec * 1e6, 2), "tflops": round(flops / sec / 1e12, 2), "kv_gbs": round(nbytes / sec / 1e9, 1)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m llmengine.kernel_bench", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8); g.add_argument("--n", type=int, default=16384); g.add_argument("--k", type=int, default=2048)
    g.add_argument("--reps", type=int, default=20)
    a = sub.add_parser("attention")
    a.add_argument("--batch", type=int, default=8); a.add_argument("--context", type=int, default=2048); a.add_argument("--new", type=int, default=1)
    a.add_argument("--heads", type=int, default=32); a.add_argument("--kv-heads", type=int, default=8); a.add_argument("--head-dim", type=int, default=64)
    a.add_argument("--page", type=int, default=16); a.add_argument("--reps", type=int, default=20)
    args = ap.parse_args(argv)
    print(json.dumps(run_gemm(args) if args.what == "gemm" else run_attention(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
