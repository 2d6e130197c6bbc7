"""Single-kernel runs for timing and profiling.

    python -m llmengine.kernel_bench gemm --m 8 --n 16384 --k 2048 [--reps 20]
    python -m llmengine.kernel_bench gemm_few --m 8 --n 2048 --k 8192 --mode residual
    python -m llmengine.kernel_bench attention --batch 8 --context 2048 --new 1
    python -m llmengine.kernel_bench attention --batch 1 --context 0 --new 2048
    python -m llmengine.kernel_bench norm --rows 8 --dim 2048 --parts 16
    python -m llmengine.kernel_bench step --batch 8 --context 2048          (timeline of one decode step)
    python -m llmengine.kernel_bench step --batch 1 --context 2048 --prefill (timeline of one prompt step)

Each of these launches ONE kind of kernel a few times on inputs that are larger than the L2 cache
(several copies of the operands are used in turn) and prints the mean device time per launch with
the bytes and flops it implies. The sizes default to the Llama 3.2 1B geometry. Meant to be run
alone or under a profiler with a small --reps.

`step` runs the whole engine on a model folder with random weights (Llama 3.2 1B sizes unless
flags say otherwise), records the device timestamps of every kernel of one scheduler step with
torch.profiler and prints, for each kind of kernel, its launches, its mean duration and its
"critical" time: how much later it ends than everything launched before it, which is its share of
the step once the overlap through programmatic dependent launch is taken out.
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch


def _time(fn, reps: int) -> float:
    """Mean device time of fn(i), i < reps, launched back to back from one CUDA graph so that the
    host's launch cost (tens of microseconds from Python) is not what is measured."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(3):
            fn(0)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(reps):
                fn(i)
        graph.replay()
        stream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        graph.replay()
        b.record(stream)
        stream.synchronize()
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
    out_kind = getattr(args, "out", "partials")
    ops.use_cta_pairs({"auto": "auto", "on": True, "off": False}[getattr(args, "pairs", "off")])
    if out_kind == "swiglu":  # w as gate|up blocks of 128 rows; the output is silu(gate) * up, bfloat16 [M, N / 2]
        act = torch.empty(M, N // 2, device=dev, dtype=torch.bfloat16)
        sec = _time(lambda i: ops.gemm_swiglu(a, ws[i % copies], act, space), args.reps)
        splits, out_bytes = 1, act.numel() * 2
    elif out_kind == "bf16":
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        sec = _time(lambda i: ops.gemm(a, ws[i % copies], out, space), args.reps)
        splits, out_bytes = 1, out.numel() * 2
    else:  # float32 partial sums [splits, M, N], as the products before a norm are asked for
        sec = _time(lambda i: ops.gemm_partials(a, ws[i % copies], space, "bench"), args.reps)
        parts = ops.gemm_partials(a, ws[0], space, "bench")
        splits, out_bytes = parts.shape[0], parts.numel() * 4
    assert ops.tensor_core_error() == 0
    flops, nbytes = 2.0 * M * N * K, N * K * 2 + M * K * 2 + out_bytes
    form = ops.gemm_form(M, N, K, out_kind == "swiglu") if M > ops.SWAP_MAX_TOKENS else "swapped, weights on the accumulator lanes"
    return {"kernel": "gemm_tc", "form": form, "out": out_kind, "M": M, "N": N, "K": K, "k_splits": splits, "us": round(sec * 1e6, 2),
            "tflops": round(flops / sec / 1e12, 1), "gbs": round(nbytes / sec / 1e9, 1)}


def run_gemm_few(args) -> dict:
    """The product of a step with few tokens (K pieces added inside a cluster), in one of its forms:
    plain, residual (added into the stream, with the rows' sums of squares) or swiglu; activations as
    bf16 rows or through the folded norm."""
    from .ops import get_ops
    ops = get_ops()
    dev = torch.device("cuda:0")
    T, N, K, mode = args.m, args.n, args.k, args.mode
    copies = max(2, int(300e6 // (N * K * 2)) + 1)
    ws = [(torch.randn(N, K, device=dev) * 0.02).bfloat16() for _ in range(copies)]
    from .engine.context import Workspace
    in_cluster = args.meet == "cluster"
    space = None if in_cluster else Workspace(dev)
    if args.splits:
        ops._few_cache[(N, K, T, mode, in_cluster)] = int(ops.lib("tensorcore").llm_gemm_decode_splits(
            N, K, T, ops._FEW_MODES[mode], args.splits, 1 if in_cluster else 0))
    splits = ops.few_token_splits(N, K, T, mode, in_cluster)
    x = torch.randn(T, K, device=dev).bfloat16()
    h = torch.randn(T, K, device=dev)
    sumsq = (h * h).sum(1, keepdim=True).repeat(1, 16).contiguous() / 16
    nw = torch.ones(K, device=dev)
    norm = (h, sumsq, nw, 1e-5, None) if args.norm else None
    if mode == "residual":
        out = torch.zeros(T, N, device=dev)
        ss = torch.empty(T, ops.residual_sumsq_parts(N, K, T, in_cluster), device=dev)
        fn = lambda i: ops.gemm_few_tokens(ws[i % copies], out, "residual", x=None if norm else x, norm=norm, sumsq_out=ss, ws=space)
    elif mode == "swiglu":
        out = torch.empty(T, N // 2, device=dev, dtype=torch.bfloat16)
        fn = lambda i: ops.gemm_few_tokens(ws[i % copies], out, "swiglu", x=None if norm else x, norm=norm, ws=space)
    else:
        out = torch.empty(T, N, device=dev)
        fn = lambda i: ops.gemm_few_tokens(ws[i % copies], out, "plain", x=None if norm else x, norm=norm, ws=space)
    sec = _time(fn, args.reps)
    assert ops.tensor_core_error() == 0
    nbytes = N * K * 2 + T * K * (4 if norm else 2) + out.numel() * out.element_size()
    return {"kernel": "gemm_decode", "mode": mode, "norm": bool(args.norm), "meet": args.meet, "T": T, "N": N, "K": K, "k_pieces": splits,
            "us": round(sec * 1e6, 2), "gbs": round(nbytes / sec / 1e9, 1)}


class _Batch:
    pass


def run_attention(args) -> dict:
    from .engine.context import Workspace
    from .ops import get_ops
    ops = get_ops()
    dev = torch.device("cuda:0")
    nq, nkv, hd, page = args.heads, args.kv_heads, args.head_dim, args.page
    B, ctx, new = args.batch, args.context, args.new
    if getattr(args, "kernel", "auto") == "mma":
        ops.tcgen05_attention = ops.tma_decode_attention = False
    ops.lib("tensorcore").llm_attention_tc_persistent(1 if getattr(args, "query_tiles", "counter") == "counter" else 0)
    total = ctx + new
    blocks = (total + page - 1) // page
    layers = max(2, int(300e6 // max(B * total * nkv * hd * 4, 1)) + 1)  # caches of several "layers" in turn
    n_pages = B * blocks
    caches = [(torch.randn(n_pages + 1, nkv, page, hd, device=dev).bfloat16(), torch.randn(n_pages + 1, nkv, page, hd, device=dev).bfloat16())
              for _ in range(layers)]
    order = torch.arange(n_pages, device=dev) if args.sequential else torch.randperm(n_pages, device=dev)
    table = order.to(torch.int32).view(B, blocks).contiguous()  # a request's pages: in a row, or anywhere in the pool
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


def run_norm(args) -> dict:
    """RMSNorm with the residual sum folded in: `rows` rows of `dim`, `parts` float32 partial sums to add
    (0: the stream alone); bfloat16 out. Buffers rotate through more than the L2 cache."""
    from .ops import get_ops
    ops = get_ops()
    dev = torch.device("cuda:0")
    n, dim, parts = args.rows, args.dim, args.parts
    per = n * dim * (4 * (2 + parts) + 2)  # bytes a launch touches: stream in and out, the parts, the result
    sets = max(2, int(300e6 // per) + 1)
    w = torch.ones(dim, device=dev)
    hs = [torch.randn(n, dim, device=dev) for _ in range(sets)]
    ds = [torch.randn(parts, n, dim, device=dev) if parts else None for _ in range(sets)]
    outs = [torch.empty(n, dim, device=dev, dtype=torch.bfloat16) for _ in range(sets)]
    sec = _time(lambda i: ops.rmsnorm(hs[i % sets], w, 1e-5, outs[i % sets], delta=ds[i % sets]), args.reps)
    nbytes = n * dim * (4 * (1 + parts) + (4 if parts else 0) + 2)  # the stream is written back only when something was added
    return {"kernel": "rmsnorm", "rows": n, "dim": dim, "parts": parts, "us": round(sec * 1e6, 2), "gbs": round(nbytes / sec / 1e9, 1)}


def run_step_timeline(args) -> dict:
    import collections
    import tempfile
    from torch.profiler import ProfilerActivity, profile
    import llmengine
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=args.hidden, intermediate_size=args.ffn,
               num_hidden_layers=args.layers, num_attention_heads=args.heads, num_key_value_heads=args.kv_heads,
               head_dim=args.head_dim, vocab_size=args.vocab, max_position_embeddings=max(4096, args.context + 512),
               rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=True)
    B, ctx = args.batch, args.context
    from .ops import get_ops
    get_ops().few_token_products = args.few_token_products == "on"
    get_ops().meet_products = args.meet_products == "on"
    get_ops().add_into_stream = args.add_into_stream == "on"
    gen = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, args.vocab, (B, ctx), generator=gen).tolist()
    with tempfile.TemporaryDirectory() as tmp:
        llmengine.write_random_model(tmp, cfg, seed=0, dtype=torch.bfloat16)
        eng = llmengine.Engine(tmp, "bf16", block_size=args.page, num_blocks=B * ((ctx + 256) // args.page + 2),
                               max_concurrent=B)
        eng._ensure_model()  # the folder is read here; it may go afterwards
    sch = llmengine.ContinuousBatchScheduler(eng, None, max_concurrent=B, max_prefill_tokens_per_step=ctx)

    if args.prefill:  # one round of prompts as warm-up, then the first step of the next round
        for p in prompts:
            sch.enqueue(p, 1)
        sch.run_until_idle()
        sch.clear_results()
        for p in prompts:
            sch.enqueue(p, 1)
    else:
        for p in prompts:
            sch.enqueue(p, 200)
        while sch.core.num_running < B:
            sch.step()
        for _ in range(5):
            sch.step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        sch.step()
        torch.cuda.synchronize()
    ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "memcpy" not in e.name.lower()
                 and "memset" not in e.name.lower()), key=lambda e: e.time_range.start)
    t0, prev_end = ev[0].time_range.start, ev[0].time_range.start
    agg = collections.OrderedDict()
    for e in ev:
        end = e.time_range.end
        name = e.name.replace("(anonymous namespace)::", "").replace("<unnamed>::", "")
        name = name[5:] if name.startswith("void ") else name
        name = name.split("(")[0].split("<")[0].split("::")[-1]
        a = agg.setdefault(name, [0, 0.0, 0.0])
        a[0] += 1
        a[1] += max(end - prev_end, 0)
        a[2] += end - e.time_range.start
        prev_end = max(prev_end, end)
    rows = [{"kernel": k, "launches": v[0], "critical_us": round(v[1], 1), "mean_duration_us": round(v[2] / v[0], 2)}
            for k, v in sorted(agg.items(), key=lambda kv: -kv[1][1])]
    assert eng.ops.tensor_core_error() == 0
    return {"step": "prefill" if args.prefill else "decode", "batch": B, "context": ctx, "layers": args.layers,
            "step_us": round(prev_end - t0, 1), "kernels": rows}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m llmengine.kernel_bench", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8); g.add_argument("--n", type=int, default=16384); g.add_argument("--k", type=int, default=2048)
    g.add_argument("--reps", type=int, default=20)
    g.add_argument("--pairs", choices=["auto", "on", "off"], default="off",
                   help="products of more than 128 tokens on CTA pairs (tcgen05 cta_group::2): where estimated faster, always, never")
    g.add_argument("--out", choices=["partials", "bf16", "swiglu"], default="partials",
                   help="what the product writes: float32 partial sums, bfloat16, or silu(gate)*up in bfloat16")
    f = sub.add_parser("gemm_few")
    f.add_argument("--m", type=int, default=8); f.add_argument("--n", type=int, default=2048); f.add_argument("--k", type=int, default=2048)
    f.add_argument("--mode", choices=["plain", "residual", "swiglu"], default="plain")
    f.add_argument("--norm", action="store_true", help="activations through the folded norm instead of bf16 rows")
    f.add_argument("--splits", type=int, default=0, help="K pieces wanted (0: the engine's choice)")
    f.add_argument("--meet", choices=["global", "cluster"], default="global",
                   help="where the K pieces are added: in global memory by the CTA that arrives last, or in the shared memory of a cluster")
    f.add_argument("--reps", type=int, default=20)
    a = sub.add_parser("attention")
    a.add_argument("--batch", type=int, default=8); a.add_argument("--context", type=int, default=2048); a.add_argument("--new", type=int, default=1)
    a.add_argument("--heads", type=int, default=32); a.add_argument("--kv-heads", type=int, default=8); a.add_argument("--head-dim", type=int, default=64)
    a.add_argument("--page", type=int, default=16); a.add_argument("--reps", type=int, default=20)
    a.add_argument("--kernel", choices=["auto", "mma"], default="auto",
                   help="mma: the mma.sync kernels also where the tcgen05 / TMA kernels would run")
    a.add_argument("--query-tiles", choices=["counter", "cta"], default="counter",
                   help="prompt portions on tcgen05: CTAs that stay and take query tiles from a counter (the default), or a CTA a query tile")
    a.add_argument("--sequential", action="store_true", help="each request's pages lie in a row (default: scattered over the pool)")
    nm = sub.add_parser("norm")
    nm.add_argument("--rows", type=int, default=8); nm.add_argument("--dim", type=int, default=2048)
    nm.add_argument("--parts", type=int, default=16, help="float32 partial sums of the product before, added into the stream (0: none)")
    nm.add_argument("--reps", type=int, default=20)
    t = sub.add_parser("step")
    t.add_argument("--batch", type=int, default=8); t.add_argument("--context", type=int, default=2048)
    t.add_argument("--prefill", action="store_true")
    t.add_argument("--few-token-products", choices=["on", "off"], default="off",
                   help="decode steps: products that add their K pieces inside a cluster, norms and SiLU folded in (off, the "
                        "engine's default: partial sums in memory, added by norm and activation kernels)")
    t.add_argument("--meet-products", choices=["on", "off"], default="off",
                   help="decode steps: o and down add their K splits and the residual themselves and leave the next norm's input; "
                        "the norms are no kernels of their own (off: the engine's default)")
    t.add_argument("--add-into-stream", choices=["on", "off"], default="off",
                   help="prompt steps: o and down add into the residual stream in their epilogue (off: the engine's default)")
    t.add_argument("--hidden", type=int, default=2048); t.add_argument("--ffn", type=int, default=8192)
    t.add_argument("--layers", type=int, default=16); t.add_argument("--heads", type=int, default=32)
    t.add_argument("--kv-heads", type=int, default=8); t.add_argument("--head-dim", type=int, default=64)
    t.add_argument("--vocab", type=int, default=128256); t.add_argument("--page", type=int, default=16)
    args = ap.parse_args(argv)
    if args.what == "step":
        r = run_step_timeline(args)
        kernels = r.pop("kernels")
        print(json.dumps(r))
        for k in kernels:
            print(f"{k['critical_us']:9.1f} us critical  x{k['launches']:4d}  mean {k['mean_duration_us']:8.2f} us  {k['kernel']}")
        return 0
    print(json.dumps({"gemm": run_gemm, "gemm_few": run_gemm_few, "attention": run_attention, "norm": run_norm}[args.what](args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
