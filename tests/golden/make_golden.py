"""Makes tests/golden/*.npz from the reference's own compiled model code (CPU).

Run once, by hand, where the reference module `llmengine` (built from its unmodified C++ sources)
is importable:

    PYTHONPATH=<dir holding the reference's llmengine package> python tests/golden/make_golden.py

For two tiny Llama configurations (one plain RoPE / GQA / untied, one llama3-scaled RoPE / MQA /
tied) it writes a checkpoint from `golden_weights` (a formula, so the test can rebuild exactly the
same tensors without a random-number library), runs the reference's `Engine.forward_logits` and
`Engine.generate`, and stores the token ids, the logits and the generated ids. The test
tests/test_plain_vs_reference.py rebuilds the checkpoints and checks tests/plain_llama.py against
these files; it needs no reference module.

Two more records reach what `Engine` of the reference refuses or does not show:
  * golden_b_long.npz: configuration b at 150 and 255 tokens. The reference's engine stops at
    min(max_position_embeddings, original_max_position_embeddings) = 64 positions for b, so here its
    EXPORTED KERNELS (src/bindings.cpp:338-412: embed_lookup_f32, rmsnorm_f32, matmul_f32,
    llama3_inv_freq, build_rope_tables with max_pos = 256, apply_rope_f32, attention_f32, silu_f32)
    are composed in the order of its layer loop (src/engine.cpp:105-261), token by token with a
    growing key/value list as its engine does. Logits at a few positions on both sides of 64 are kept.
  * golden_scheduler.json: token streams and finish reasons of the reference's
    ContinuousBatchScheduler (src/scheduler.cpp:136-319) for both configurations: budget 4 with
    max_new_tokens 0, 1, 2 and 5, a batch with an end-of-sequence id among the outputs, and the
    capacity case of its own test (tests/test_scheduler.py:285-307).
"""
from __future__ import annotations

import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

GOLDEN_CONFIGS = {
    # sequences stay within the reference's position cap min(max_pos, original_max_pos)
    "a": dict(hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, vocab_size=256, max_position_embeddings=128,
              rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=False,
              architectures=["LlamaForCausalLM"], eos_token_id=7),
    "b": dict(hidden_size=96, intermediate_size=200, num_hidden_layers=3, num_attention_heads=6,
              num_key_value_heads=1, head_dim=32, vocab_size=509, max_position_embeddings=256,
              rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=True,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                high_freq_factor=4.0, original_max_position_embeddings=64),
              architectures=["LlamaForCausalLM"], eos_token_id=[3, 5]),
}
GOLDEN_SEQ_LENS = {"a": [1, 5, 17], "b": [2, 23, 58]}


def _hash_unit(n: int, salt: int) -> np.ndarray:
    """n values in (0,1) from an integer hash of (index, salt)."""
    with np.errstate(over="ignore"):
        x = np.arange(n, dtype=np.uint64) + np.full(1, salt, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)
        x ^= x >> np.uint64(30)
        x *= np.uint64(0xBF58476D1CE4E5B9)
        x ^= x >> np.uint64(27)
        x *= np.uint64(0x94D049BB133111EB)
        x ^= x >> np.uint64(31)
    return ((x >> np.uint64(11)).astype(np.float64) + 0.5) / float(1 << 53)


def _hash_normal(shape, salt: int) -> np.ndarray:
    n = int(np.prod(shape))
    u1 = _hash_unit(n, 2 * salt + 1)
    u2 = _hash_unit(n, 2 * salt + 2)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return z.reshape(shape)


def golden_weights(cfg: dict) -> dict:
    """Linear and embedding weights ~N(0, 0.05), norm weights ~N(1, 0.1), float32, by formula.
    The spread is wider than a trained checkpoint's so that logits are well apart."""
    H, FF, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    shapes = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    if not cfg.get("tie_word_embeddings", False):
        shapes["lm_head.weight"] = (V, H)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        shapes[p + "input_layernorm.weight"] = (H,)
        shapes[p + "post_attention_layernorm.weight"] = (H,)
        shapes[p + "self_attn.q_proj.weight"] = (nq * hd, H)
        shapes[p + "self_attn.k_proj.weight"] = (nkv * hd, H)
        shapes[p + "self_attn.v_proj.weight"] = (nkv * hd, H)
        shapes[p + "self_attn.o_proj.weight"] = (H, nq * hd)
        shapes[p + "mlp.gate_proj.weight"] = (FF, H)
        shapes[p + "mlp.up_proj.weight"] = (FF, H)
        shapes[p + "mlp.down_proj.weight"] = (H, FF)
    out = {}
    for salt, (name, shape) in enumerate(sorted(shapes.items())):
        z = _hash_normal(shape, salt + 1)
        if name.endswith("norm.weight") or "layernorm" in name:
            out[name] = (1.0 + 0.1 * z).astype(np.float32)
        else:
            out[name] = (0.05 * z).astype(np.float32)
    return out


def golden_ids(name: str, n: int, vocab: int) -> list:
    u = _hash_unit(n, 1000 + n + (0 if name == "a" else 500))
    return [int(v) for v in np.minimum((u * vocab).astype(np.int64), vocab - 1)]


def write_model_dir(path: str, cfg: dict, weights: dict) -> None:
    from safetensors.numpy import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(weights, os.path.join(path, "model.safetensors"))


LONG_LENS = [150, 255]
LONG_ROWS = {150: [0, 1, 31, 62, 63, 64, 65, 100, 127, 128, 148, 149],
             255: [0, 63, 64, 65, 129, 191, 192, 200, 253, 254]}


def compose_reference_kernels(k, cfg: dict, w: dict, ids, rows) -> np.ndarray:
    """Logits at `rows` of one sequence from the reference's exported kernels, composed as its layer
    loop composes them (src/engine.cpp:105-261): one token at a time, keys (after rotation) and
    values appended to per-layer lists, attention of the token over all of them."""
    H, nq, nkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = float(np.float32(cfg["rms_norm_eps"]))
    rs = cfg.get("rope_scaling")
    inv = k.llama3_inv_freq(hd, float(np.float32(cfg["rope_theta"])), rs is not None,
                            float(rs["factor"]) if rs else 1.0, float(rs["low_freq_factor"]) if rs else 1.0,
                            float(rs["high_freq_factor"]) if rs else 1.0,
                            int(rs["original_max_position_embeddings"]) if rs else 0)
    cos, sin = k.build_rope_tables(inv, cfg["max_position_embeddings"], hd)
    L = cfg["num_hidden_layers"]
    keys = [[] for _ in range(L)]
    vals = [[] for _ in range(L)]
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    out = {}
    for pos, tok in enumerate(ids):
        h = np.asarray(k.embed_lookup_f32(w["model.embed_tokens.weight"], int(tok)), dtype=np.float32)
        for l in range(L):
            p = f"model.layers.{l}."
            x = np.asarray(k.rmsnorm_f32(h, w[p + "input_layernorm.weight"], eps))[None, :]
            q = np.asarray(k.matmul_f32(x, w[p + "self_attn.q_proj.weight"])).reshape(nq, hd)
            kk = np.asarray(k.matmul_f32(x, w[p + "self_attn.k_proj.weight"])).reshape(nkv, hd)
            v = np.asarray(k.matmul_f32(x, w[p + "self_attn.v_proj.weight"])).reshape(nkv, hd)
            q = np.stack([np.asarray(k.apply_rope_f32(q[i], cos[pos], sin[pos])) for i in range(nq)])
            kk = np.stack([np.asarray(k.apply_rope_f32(kk[i], cos[pos], sin[pos])) for i in range(nkv)])
            keys[l].append(kk)
            vals[l].append(v)
            a = np.asarray(k.attention_f32(q.astype(np.float32), np.stack(keys[l]).astype(np.float32),
                                           np.stack(vals[l]).astype(np.float32), nq, nkv, hd)).reshape(1, nq * hd)
            h = h + np.asarray(k.matmul_f32(a, w[p + "self_attn.o_proj.weight"]))[0]
            x = np.asarray(k.rmsnorm_f32(h, w[p + "post_attention_layernorm.weight"], eps))[None, :]
            g = np.asarray(k.silu_f32(np.asarray(k.matmul_f32(x, w[p + "mlp.gate_proj.weight"]))[0]))
            u = np.asarray(k.matmul_f32(x, w[p + "mlp.up_proj.weight"]))[0]
            h = h + np.asarray(k.matmul_f32((g * u).astype(np.float32)[None, :], w[p + "mlp.down_proj.weight"]))[0]
        if pos in rows:
            x = np.asarray(k.rmsnorm_f32(h.astype(np.float32), w["model.norm.weight"], eps))[None, :]
            out[pos] = np.asarray(k.matmul_f32(x, head))[0]
    return np.stack([out[r] for r in rows]).astype(np.float32)


SCHEDULER_CASES = [
    # (name, configuration, prompt lengths, max_new_tokens per prompt, budget, max_concurrent, pages, page size)
    ("a_budget4", "a", [5, 11, 3, 17], [5, 0, 1, 2], 4, 8, 64, 4),
    ("b_budget4", "b", [2, 23, 9, 40], [5, 1, 0, 2], 4, 3, 32, 16),
    ("a_wide", "a", [1, 3, 7, 2], [12, 12, 12, 12], 64, 4, 64, 4),
    ("a_capacity", "a", [4, 4], [12, 12], 4, 2, 4, 4),
]


def reference_scheduler_streams(ref) -> dict:
    out = {}
    for name, which, lens, news, budget, conc, pages, page in SCHEDULER_CASES:
        cfg = GOLDEN_CONFIGS[which]
        with tempfile.TemporaryDirectory() as d:
            write_model_dir(d, cfg, golden_weights(cfg))
            eng = ref.Engine(d, "fp32")
            mgr = ref.BlockManager(pages, page, cfg["num_hidden_layers"], cfg["num_key_value_heads"], cfg["head_dim"])
            sch = ref.ContinuousBatchScheduler(eng, mgr, max_concurrent=conc, max_prefill_tokens_per_step=budget)
            prompts = [golden_ids(which, n, cfg["vocab_size"]) for n in lens]
            for p, n in zip(prompts, news):
                sch.enqueue(p, n)
            sch.run_until_idle()
            res = sorted(sch.results, key=lambda r: r.seq_id)
            out[name] = dict(config=which, prompt_lens=lens, max_new=news, budget=budget, max_concurrent=conc, pages=pages,
                             page_size=page, token_ids=[list(map(int, r.token_ids)) for r in res],
                             finish=[r.finish_reason for r in res], free_after=int(mgr.free_blocks))
    # requests that end at an end-of-sequence id (not appended): prompts of configuration a whose greedy
    # stream meets id 7 within 40 tokens, found by trying lengths, run beside two that end by length
    cfg = GOLDEN_CONFIGS["a"]
    with tempfile.TemporaryDirectory() as d:
        write_model_dir(d, cfg, golden_weights(cfg))
        eng = ref.Engine(d, "fp32")
        stops = [n for n in range(1, 80) if eng.generate(golden_ids("a", n, cfg["vocab_size"]), 40)[1] == "stop"][:2]
        if stops:
            lens, news = stops + [6, 9], [40] * len(stops) + [3, 7]
            mgr = ref.BlockManager(64, 4, cfg["num_hidden_layers"], cfg["num_key_value_heads"], cfg["head_dim"])
            sch = ref.ContinuousBatchScheduler(eng, mgr, max_concurrent=3, max_prefill_tokens_per_step=5)
            for n, k in zip(lens, news):
                sch.enqueue(golden_ids("a", n, cfg["vocab_size"]), k)
            sch.run_until_idle()
            res = sorted(sch.results, key=lambda r: r.seq_id)
            out["a_stop"] = dict(config="a", prompt_lens=lens, max_new=news, budget=5, max_concurrent=3, pages=64, page_size=4,
                                 token_ids=[list(map(int, r.token_ids)) for r in res], finish=[r.finish_reason for r in res],
                                 free_after=int(mgr.free_blocks))
    return out


def main() -> None:
    import llmengine as ref  # the reference's module, not the package under test
    from llmengine._llmengine import kernels as ref_kernels  # its exported kernels (src/bindings.cpp:338-412)
    cfg = GOLDEN_CONFIGS["b"]
    w = golden_weights(cfg)
    rec = {}
    for n in LONG_LENS:
        ids = golden_ids("b", n, cfg["vocab_size"])
        rec[f"ids_{n}"] = np.array(ids, dtype=np.int32)
        rec[f"rows_{n}"] = np.array(LONG_ROWS[n], dtype=np.int32)
        rec[f"logits_{n}"] = compose_reference_kernels(ref_kernels, cfg, w, ids, LONG_ROWS[n])
    np.savez_compressed(os.path.join(HERE, "golden_b_long.npz"), **rec)
    print("b_long", {k_: v.shape for k_, v in rec.items()})
    with open(os.path.join(HERE, "golden_scheduler.json"), "w") as f:
        json.dump(reference_scheduler_streams(ref), f, indent=0)
    for name, cfg in GOLDEN_CONFIGS.items():
        w = golden_weights(cfg)
        with tempfile.TemporaryDirectory() as d:
            write_model_dir(d, cfg, w)
            eng = ref.Engine(d, "fp32")
            rec = {}
            for n in GOLDEN_SEQ_LENS[name]:
                ids = golden_ids(name, n, cfg["vocab_size"])
                rec[f"ids_{n}"] = np.array(ids, dtype=np.int32)
                rec[f"logits_{n}"] = np.asarray(eng.forward_logits(ids), dtype=np.float32)
                toks, reason = eng.generate(ids, 6)
                rec[f"gen_{n}"] = np.array(toks, dtype=np.int32)
                rec[f"reason_{n}"] = np.array([reason])
            np.savez_compressed(os.path.join(HERE, f"golden_{name}.npz"), **rec)
            print(name, {k: v.shape for k, v in rec.items()})


if __name__ == "__main__":
    sys.exit(main())
