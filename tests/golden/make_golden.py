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


def main() -> None:
    import llmengine as ref  # the reference's module, not the package under test
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
