#!/usr/bin/env python3
"""Serving benchmark on one B200: decode tokens a second of the Llama 3.2 1B geometry.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of a continuous batch: one new token for each of `batch` requests that
each hold `context` tokens in the paged cache. The default run has the layer sizes of the 1B
geometry with random bfloat16 weights (written as a model folder by the engine's random-weights
mode and read back through its loader), a batch of 8 and contexts of 2,048 tokens.

One JSON line is printed:
  value        decoded tokens a second, device time (CUDA events around K steps, host running ahead); the
               K-step region is timed --reps times (default 5) and the median is reported, with the
               fastest and slowest region in `spread`
  e2e          the same through the Python entry point (ContinuousBatchScheduler.step): every step
               copies that step's batch from pinned host memory and reads the sampled tokens back
  prefill      one 2,048-token prompt as one step: tokens a second, ms, fraction of the tensor peak
  roofline     decode step: bytes it must read (every weight once + the cache of the live requests)
               / step time, against the measured copy bandwidth
  points       decode tokens a second at batch 1 and 64 (with ms a step and the fraction of the copy
               bandwidth), and at batch 8 through the true 32-bit path (CUDA-core kernels)
Peaks come from MEASURED_PEAKS.json beside this file when present, else from the fallback figures
measured earlier on this pool (6.65 TB/s, 1.59 PFLOP/s). For --gpus > 1 one line says that this
engine is single-GPU and the exit code is 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "llm-inference-engine-v6_b200"))

# Llama 3.2 1B geometry
GEOMETRY = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
                num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=128256,
                max_position_embeddings=8192, rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=True,
                rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192))
FULL_LAYERS = 16
# Further sizes for --geometry (the default, and what the headline is quoted on, stays the 1B one):
# Llama 3.2 3B and Llama 3.1 8B layer sizes.
GEOMETRIES = {
    "1b": (GEOMETRY, 16, "llama-3.2-1b-geometry", "Llama 3.2 1B"),
    "3b": (dict(GEOMETRY, hidden_size=3072, num_attention_heads=24, head_dim=128, num_hidden_layers=28), 28, "llama-3.2-3b-geometry", "Llama 3.2 3B"),
    "8b": (dict(GEOMETRY, hidden_size=4096, intermediate_size=14336, num_attention_heads=32, head_dim=128, num_hidden_layers=32,
                tie_word_embeddings=False,
                rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192)), 32, "llama-3.1-8b-geometry", "Llama 3.1 8B"),
}
CONTEXT, CONTEXT_LIMIT, PREFILL_TOKENS, BLOCK_SIZE = 2048, 4096, 2048, 16
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                j = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(j.get(k), (int, float)) and j[k] > 0:
                    out[k] = float(j[k])
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.path = tempfile.mktemp(prefix="clocks_", suffix=".csv")
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:  # (a query stuck in the driver: do not wait for it)
            self.proc.kill()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                pass
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 6:
                    continue
                try:
                    mhz.append(float(parts[0]))
                    mx = float(parts[1])
                except ValueError:
                    continue
                for n, v in zip(names, parts[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        os.remove(self.path)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons)}


def flops_of_prefill(g, layers, T):
    H, FF, V = g["hidden_size"], g["intermediate_size"], g["vocab_size"]
    dq, dkv = g["num_attention_heads"] * g["head_dim"], g["num_key_value_heads"] * g["head_dim"]
    linear = 2 * T * (H * (dq + 2 * dkv) + dq * H + 3 * H * FF) * layers
    attention = layers * 2 * 2 * dq * T * (T + 1) // 2
    return linear + attention + 2 * H * V  # the head runs for the last row only


def decode_bytes(g, layers, batch, context, el=2):
    H, FF, V = g["hidden_size"], g["intermediate_size"], g["vocab_size"]
    dq, dkv = g["num_attention_heads"] * g["head_dim"], g["num_key_value_heads"] * g["head_dim"]
    weights = layers * (H * (dq + 2 * dkv) + dq * H + 3 * H * FF) * el + V * H * el + (2 * layers + 1) * H * 4
    kv = batch * context * layers * 2 * dkv * el
    return weights + kv


def run_ours(args):
    import torch
    import llmengine
    from llmengine.cache import host_module

    torch.cuda.set_device(0)
    base, full_layers, model_name, model_label = GEOMETRIES[args.geometry]
    layers = args.layers if args.layers > 0 else full_layers
    g = dict(base, num_hidden_layers=layers)
    pk = peaks()
    K, W = args.steps, args.warmup
    tmp = tempfile.TemporaryDirectory(prefix="llmengine_bench_")
    t0 = time.time()
    llmengine.write_random_model(tmp.name, g, seed=0, dtype=torch.bfloat16)
    max_batch = max(args.batch, 64 if args.points else args.batch, 1)
    R = max(1, args.reps)
    room = CONTEXT + 2 * (K * R + W) + max_batch + 64
    num_blocks = max_batch * (room + BLOCK_SIZE - 1) // BLOCK_SIZE + PREFILL_TOKENS // BLOCK_SIZE + 8
    skip = set(x for x in args.skip.split(",") if x)
    if "points" in skip:
        args.points = False
    eng = main_eng = llmengine.Engine(tmp.name, "bf16", block_size=BLOCK_SIZE, num_blocks=num_blocks, max_concurrent=max_batch,
                                      cuda_graphs=args.graphs)
    eng.configure_cache()
    sys.stderr.write(f"[bench] model written and loaded in {time.time() - t0:.1f}s; {num_blocks} pages\n")
    gen = torch.Generator().manual_seed(1)
    H = host_module()

    def prompts(n, length):
        return torch.randint(0, g["vocab_size"], (n, length), generator=gen).tolist()

    def check(phase):
        """A kernel whose bounded wait gave up leaves a code and returns; every launch after it may do
        the same, a second at a time. Better to stop at once and say where."""
        code = main_eng.ops.tensor_core_error()
        if code:
            raise RuntimeError(f"a tensor-core kernel gave up a wait (code {code}) during: {phase}")
        sys.stderr.write(f"[bench] {phase}: done at {time.time() - t0:.1f}s\n")
        sys.stderr.flush()

    def decode_run(batch, k_steps, w_steps, e2e, reps=1, eng=None):
        """-> (median seconds per step over `reps` timed regions of k_steps, kernel launches per step,
        h2d bytes, d2h bytes, [seconds per step of every region])."""
        eng = eng or main_eng
        sch = llmengine.ContinuousBatchScheduler(eng, None, max_concurrent=batch, max_prefill_tokens_per_step=PREFILL_TOKENS)
        for p in prompts(batch, CONTEXT):
            sch.enqueue(p, 2 * (k_steps * reps + w_steps) + batch + 8)  # early requests decode while later prompts prefill
        for _ in range(2 * batch + 8):  # prefill (untimed): one prompt a step
            if sch.core.num_running == batch:
                break
            sch.step()
        assert sch.core.num_running == batch, "the contexts could not be filled"
        check(f"prompts of batch {batch}")
        launches = 0

        def one_step():
            if e2e:
                sch.step()
                return
            entries = sch.core.plan()
            if eng.cuda_graphs:
                if eng.graphs is None:
                    from llmengine.engine.graphs import DecodeGraphs
                    eng.graphs = DecodeGraphs(eng)
                eng.graphs.run_device(entries)
            else:
                ctx, logits = eng.step(entries)
                eng.sampler.sample_device(logits, ctx, ctx.n_rows)
            sch.core.commit([1] * len(entries))  # timing only: the token values do not matter

        for _ in range(w_steps):
            one_step()
        torch.cuda.synchronize()
        check(f"warm-up steps of batch {batch}")
        eng.ops.launches = 0
        regions = []
        for _ in range(reps):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t_wall = time.perf_counter()
            start.record()
            for _ in range(k_steps):
                one_step()
            stop.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - t_wall
            dev = start.elapsed_time(stop) / 1e3
            regions.append((max(dev, wall) if e2e else dev) / k_steps)
        launches = eng.ops.launches / (k_steps * reps)
        check(f"timed steps of batch {batch}" + (" through the scheduler" if e2e else ""))
        if e2e and eng.cuda_graphs and eng.graphs is not None:
            h2d, d2h = eng.graphs.h2d_bytes, eng.graphs.d2h_bytes
        else:
            h2d, d2h = eng.buffers.h2d_bytes, 4 * batch
        # drain: finish the requests and give their pages back
        for r in list(sch._cm.request_ids()):
            sch._cm.release(r)
        return statistics.median(regions), launches, h2d, d2h, regions

    def prefill_run(k_steps, w_steps):
        times = []
        for i in range(w_steps + k_steps):
            ids = prompts(1, PREFILL_TOKENS)[0]
            e = H.StepEntries()
            rid = 10 ** 9 + i
            eng = main_eng
            eng.cm.add_request(rid)
            assert eng.cm.reserve(rid, PREFILL_TOKENS)
            e.add(rid, ids, [PREFILL_TOKENS - 1])
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            eng.step(e)
            b.record()
            torch.cuda.synchronize()
            eng.cm.release(rid)
            if i >= w_steps:
                times.append(a.elapsed_time(b) / 1e3)
            if i == 0:
                check(f"first prompt step of {PREFILL_TOKENS} tokens")
        return statistics.median(times)

    clocks = ClockSampler()
    clocks.start()
    if "decode" in skip:  # profiling runs of the prefill alone
        sec, launches, regions = float("inf"), 0, [float("inf")]
    else:
        sec, launches, _, _, regions = decode_run(args.batch, K, W, e2e=False, reps=R)
    clock_rec = clocks.stop()
    e2e_sec, h2d, d2h = sec, 0, 0
    if "e2e" not in skip:
        e2e_sec, _, h2d, d2h, _ = decode_run(args.batch, K, W, e2e=True, reps=R)
    pre_sec = prefill_run(max(2, min(K, 5)), max(1, min(W, 3))) if "prefill" not in skip else float("inf")
    points = {}
    if args.points:
        for b in (1, 64):
            s, *_ = decode_run(b, max(4, K // 2), W, e2e=False, reps=min(R, 3))
            points[f"decode_b{b}"] = round(b / s, 1)
            points[f"decode_b{b}_ms"] = round(s * 1e3, 4)
            points[f"decode_b{b}_hbm_frac"] = round(decode_bytes(g, layers, b, CONTEXT + W + K // 2) / s / 1e9 / pk["hbm_gbs"], 4)
        # the true 32-bit path of the same model (CUDA-core products, float32 cache): what the oracle costs
        fp32_blocks = args.batch * (CONTEXT + 64) // BLOCK_SIZE + 16
        eng32 = llmengine.Engine(tmp.name, "fp32", block_size=BLOCK_SIZE, num_blocks=fp32_blocks, max_concurrent=args.batch)
        eng32.configure_cache()
        s, *_ = decode_run(args.batch, 4, 3, e2e=False, eng=eng32)
        points[f"decode_b{args.batch}_fp32"] = round(args.batch / s, 1)
        points[f"decode_b{args.batch}_fp32_ms"] = round(s * 1e3, 3)

    value = args.batch / sec
    bytes_step = decode_bytes(g, layers, args.batch, CONTEXT + W + K * R // 2)
    achieved = bytes_step / sec / 1e9 if sec != float("inf") else 0.0
    pf = flops_of_prefill(g, layers, PREFILL_TOKENS)
    rec = {
        "metric": f"decode tok/s at batch {args.batch} ({model_label} geometry, {CONTEXT}-token contexts)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(sec * 1e3, 4) if sec != float("inf") else None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids", "impl": "ours",
        "config": {"model": model_name, "global_batch": args.batch, "seq_len": CONTEXT,
                   "context_limit": CONTEXT_LIMIT, "parallelism": "single-gpu", "layers": layers,
                   "layers_full_config": full_layers, "hidden": g["hidden_size"], "heads": g["num_attention_heads"],
                   "kv_heads": g["num_key_value_heads"], "head_dim": g["head_dim"], "intermediate": g["intermediate_size"],
                   "vocab": g["vocab_size"], "tied_embeddings": bool(g["tie_word_embeddings"]), "kv_block_size": BLOCK_SIZE,
                   "prefill_tokens": PREFILL_TOKENS, "l2": "step reads > 2 GB of weights: inputs larger than L2",
                   "peaks": pk["source"]},
        "spread": ({"reps": R, "min_ms": round(min(regions) * 1e3, 4), "max_ms": round(max(regions) * 1e3, 4)}
                   if sec != float("inf") else None),
        "e2e": {"value": round(args.batch / e2e_sec, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(round(launches * K)),
        "prefill": {"value": round(PREFILL_TOKENS / pre_sec, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_sec * 1e3, 3),
                    "frac": round(pf / pre_sec / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_rec,
    }
    print(json.dumps(rec), flush=True)
    return 0


def run_workload(args):
    """The serving workloads that go with the larger geometries: `serve` = 32 requests with prompts of
    16 to 2,048 random tokens and 256 new tokens each through the continuous-batching scheduler;
    `long` = one prompt of 16,384 tokens in portions of 2,048, then 512 decoded tokens. Prints one JSON
    line of its own (not the contract's line): tokens a second over the whole run, and `host_wait_share`: the part of the wall
    time that the host spent blocked, waiting for the device to finish a step. While it waits the host
    is no bound; the rest (`host_busy_share`: planning, batch building, launching the kernels of prompt
    and mixed steps one by one, most of it beside a busy device) is the most that the host can cost."""
    import torch
    import llmengine

    torch.cuda.set_device(0)
    base, full_layers, model_name, _ = GEOMETRIES[args.geometry]
    layers = args.layers if args.layers > 0 else full_layers
    gen = torch.Generator().manual_seed(2)
    if args.workload == "serve":
        lens = torch.randint(16, 2049, (32,), generator=gen).tolist()
        new, budget, conc, max_pos = 256, args.budget, 32, 8192
    else:
        lens, new, budget, conc, max_pos = [16384], 512, 2048, 1, 32768
    g = dict(base, num_hidden_layers=layers, max_position_embeddings=max_pos)
    tmp = tempfile.TemporaryDirectory(prefix="llmengine_bench_")
    llmengine.write_random_model(tmp.name, g, seed=0, dtype=torch.bfloat16)
    pages = sum((n + new + BLOCK_SIZE - 1) // BLOCK_SIZE + 1 for n in lens) + 8
    eng = llmengine.Engine(tmp.name, "bf16", block_size=BLOCK_SIZE, num_blocks=pages, max_concurrent=conc)
    eng.configure_cache()
    prompts = [torch.randint(0, g["vocab_size"], (n,), generator=gen).tolist() for n in lens]

    def run():
        sch = llmengine.ContinuousBatchScheduler(eng, None, max_concurrent=conc, max_prefill_tokens_per_step=budget)
        for p in prompts:
            sch.enqueue(p, new)
        steps = 0
        torch.cuda.synchronize()
        waited0 = eng.sampler.wait_seconds
        t_all = time.perf_counter()
        while sch.step():
            steps += 1
        torch.cuda.synchronize()
        total = time.perf_counter() - t_all
        waited = eng.sampler.wait_seconds - waited0
        sch.core.finalize()
        out = sum(len(r.token_ids) - r.prompt_len for r in sch.results)
        assert all(r.finish_reason == "length" for r in sch.results)
        return total, waited, steps + 1, out

    run()  # warm-up: kernels loaded, graphs captured, workspaces sized
    total, waited, steps, out = run()
    code = eng.ops.tensor_core_error()
    if code:
        raise RuntimeError(f"a tensor-core kernel gave up a wait (code {code})")
    print(json.dumps({"workload": args.workload, "model": model_name, "layers": layers, "requests": len(lens),
                      "prompt_tokens": sum(lens), "new_tokens": out, "budget": budget, "steps": steps,
                      "seconds": round(total, 4), "tokens_per_s": round((sum(lens) + out) / total, 1),
                      "decoded_tokens_per_s": round(out / total, 1),
                      "host_wait_share": round(waited / total, 4), "host_busy_share": round(1 - waited / total, 4)}), flush=True)
    return 0


def run_reference(args):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0

    if not os.path.isdir(os.path.join(ref_dir, "llmengine")):
        return unavailable("baseline/_ref holds no installed reference package (pip builds its wheel without the compiled module)")
    # the model folder is written by this repo's random-weights mode in a child process, so that the
    # reference's `llmengine` and this repo's `llmengine` never share an interpreter
    tmp = tempfile.TemporaryDirectory(prefix="llmengine_bench_ref_")
    g = dict(GEOMETRY, num_hidden_layers=args.layers if args.layers > 0 else FULL_LAYERS)
    code = ("import sys, json, torch; sys.path.insert(0, %r); import llmengine; "
            "llmengine.write_random_model(%r, json.loads(%r), seed=0, dtype=torch.bfloat16)"
            % (os.path.join(ROOT, "llm-inference-engine-v6_b200"), tmp.name, json.dumps(g)))
    subprocess.run([sys.executable, "-c", code], check=True)
    sys.path.insert(0, ref_dir)
    try:
        import llmengine as ref
        assert hasattr(ref, "StaticBatchScheduler")
    except Exception as e:
        return unavailable(f"reference does not import: {type(e).__name__}: {e}"[:200])
    import numpy as np
    K, W, B = args.steps, args.warmup, args.batch
    eng = ref.Engine(tmp.name, "fp32")
    rng = np.random.default_rng(1)
    # probe: the reference prefills one token at a time on the CPU
    t0 = time.perf_counter()
    eng.generate(rng.integers(0, g["vocab_size"], 16).tolist(), 0)
    per_tok = (time.perf_counter() - t0) / 16
    projected = per_tok * B * CONTEXT
    if projected > args.reference_setup_limit:
        return unavailable(f"reference is a CPU engine: filling {B} contexts of {CONTEXT} tokens would take "
                           f"~{projected / 60:.0f} min ({per_tok * 1e3:.0f} ms a token)")
    cfg = eng.cfg
    need = B * ((CONTEXT + K + W + 2 + BLOCK_SIZE) // BLOCK_SIZE + 1)
    mgr = ref.BlockManager(need, BLOCK_SIZE, cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.head_dim)
    sch = ref.ContinuousBatchScheduler(eng, mgr, max_concurrent=B, max_prefill_tokens_per_step=256)
    for _ in range(B):
        sch.enqueue(rng.integers(0, g["vocab_size"], CONTEXT).tolist(), K + W + 2)
    for _ in range((B * CONTEXT + 255) // 256):
        sch.step()
    for _ in range(W):
        sch.step()
    t0 = time.perf_counter()
    for _ in range(K):
        sch.step()
    sec = (time.perf_counter() - t0) / K
    print(json.dumps({
        "metric": "decode tok/s at batch 8 (Llama 3.2 1B geometry, 2048-token contexts)", "impl": "reference",
        "value": round(B / sec, 3), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(sec * 1e3, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32 (the reference's stock path; it has no bf16 engine)", "data": "synthetic: same random model folder",
        "config": {"model": "llama-3.2-1b-geometry", "global_batch": B, "seq_len": CONTEXT, "layers": args.layers if args.layers > 0 else FULL_LAYERS,
                   "parallelism": "cpu threads (the reference has no GPU code)"},
        "gpu_launches": 0}), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--reps", type=int, default=5, help="how many times the K-step region is timed (the median is reported)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the full configuration (named in `config`); 0: all")
    ap.add_argument("--geometry", choices=sorted(GEOMETRIES), default="1b", help="layer sizes: Llama 3.2 1B (default), 3.2 3B, 3.1 8B")
    ap.add_argument("--no-points", dest="points", action="store_false", help="skip the batch 1 and 64 points")
    ap.add_argument("--skip", default="", help="comma list of parts to leave out: decode,e2e,prefill,points (for profiling runs)")
    ap.add_argument("--no-cuda-graphs", dest="graphs", action="store_false", help="launch decode steps kernel by kernel")
    ap.add_argument("--workload", choices=["decode", "serve", "long"], default="decode",
                    help="decode: the contract's line (default). serve / long: the workloads of the 3B and 8B configurations, a line of their own")
    ap.add_argument("--budget", type=int, default=2048, help="serve: prompt tokens a step (max_prefill_tokens_per_step)")
    ap.add_argument("--reference-setup-limit", type=float, default=900.0, help="seconds the reference arm may spend filling contexts")
    args = ap.parse_args()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py: this engine runs on ONE GPU; --gpus {args.gpus} is not supported", flush=True)
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    if args.workload != "decode":
        return run_workload(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
