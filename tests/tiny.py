"""Shared helpers of the tests: tiny Llama configurations that differ in every size and option,
model folders with random weights in a temporary place, and builders of replay traces.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")

# A: 2 layers, GQA 4:2, head 16, FF 176 (no power of two), vocab 256, theta 1e4, plain RoPE,
#    eps 1e-6, untied head, 128 positions; pages of 4.
TINY_A = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=176, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256,
              max_position_embeddings=128, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=False)
# B: 3 layers, MQA 6:1, head 32, hidden 192, FF 512, vocab 509 (odd), theta 5e5 with llama3 scaling
#    (factor 8, low 1, high 4, original 64), eps 1e-5, tied head, 256 positions; pages of 16.
TINY_B = dict(architectures=["LlamaForCausalLM"], hidden_size=192, intermediate_size=512, num_hidden_layers=3,
              num_attention_heads=6, num_key_value_heads=1, head_dim=32, vocab_size=509,
              max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=True,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=64))
# C: sizes that fit nothing: multi-head (5:5), head 48 (so heads * head_dim != hidden), hidden 120,
#    FF 100 (not a multiple of 8: the tensor-core product refuses it), vocab 1001, one layer, large eps.
TINY_C = dict(architectures=["LlamaForCausalLM"], hidden_size=120, intermediate_size=100, num_hidden_layers=1,
              num_attention_heads=5, num_key_value_heads=5, head_dim=48, vocab_size=1001,
              max_position_embeddings=300, rms_norm_eps=1e-3, rope_theta=1000000.0, tie_word_embeddings=False,
              hidden_act="silu", attention_bias=False, mlp_bias=False, rope_scaling=None, torch_dtype="bfloat16")
# D: the shapes the tensor-core kernels are made for: head 64, GQA 8:2, pages of 16, FF a multiple of 128.
TINY_D = dict(architectures=["LlamaForCausalLM"], hidden_size=256, intermediate_size=384, num_hidden_layers=2,
              num_attention_heads=8, num_key_value_heads=2, head_dim=64, vocab_size=2000,
              max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=True,
              rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=128))
# E: head 128 (its own instantiations of the attention kernels), a group of 3, pages of 32.
TINY_E = dict(architectures=["LlamaForCausalLM"], hidden_size=192, intermediate_size=320, num_hidden_layers=2,
              num_attention_heads=3, num_key_value_heads=1, head_dim=128, vocab_size=777,
              max_position_embeddings=400, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False)
TINY = {"a": (TINY_A, 4), "b": (TINY_B, 16), "c": (TINY_C, 16), "d": (TINY_D, 16), "e": (TINY_E, 32)}  # name -> (config.json, page size)

# Weights are wider than a trained model's (std 0.05) so that logits are well apart and a wrong
# key, page or position shows as a large error.
WEIGHT_STD = 0.05


def make_model_dir(path: str, cfg: dict, dtype: torch.dtype, seed: int = 11) -> str:
    import llmengine
    return llmengine.write_random_model(path, cfg, seed=seed, dtype=dtype, std=WEIGHT_STD)


def random_ids(n: int, vocab: int, seed: int) -> List[int]:
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


# ------------------------------------------------------------------------------------ traces
def round64(n: int) -> int:
    return (n + 63) // 64 * 64


class Trace:
    """Steps for bin/trace_run plus, for every written row, which (request, position) it is."""

    def __init__(self):
        self.steps: List[dict] = []
        self.rows: Dict[int, List[Tuple[str, int]]] = {}

    def add(self, entries: Sequence[Tuple[str, Sequence[int], Sequence[int], int]], end: Sequence[str] = ()) -> None:
        """entries: (request name, tokens, wanted places, position of the first token)."""
        k = len(self.steps)
        self.steps.append({"step": k, "entries": [{"id": n, "tokens": list(map(int, t)), "want": list(map(int, w))}
                                                  for n, t, w, _ in entries], "end": list(end)})
        rows = [(n, start + w) for n, t, ws, start in entries for w in ws]
        if rows:
            self.rows[k] = rows

    def keep_only(self, wanted) -> "Trace":
        """Asks only for the logits at the positions wanted(request name) -> set of positions (for
        models whose head is too large to compare at every position)."""
        self.rows = {}
        pos: Dict[str, int] = {}
        for k, s in enumerate(self.steps):
            rows = []
            for e in s["entries"]:
                start = pos.get(e["id"], 0)
                keep = wanted(e["id"])
                e["want"] = [w for w in range(len(e["tokens"])) if start + w in keep]
                rows += [(e["id"], start + w) for w in e["want"]]
                pos[e["id"]] = start + len(e["tokens"])
            for name in s["end"]:
                pos.pop(name, None)
            if rows:
                self.rows[k] = rows
        return self

    def extend(self, other: "Trace") -> None:
        off = len(self.steps)
        for s in other.steps:
            s2 = dict(s)
            s2["step"] = s["step"] + off
            self.steps.append(s2)
        for k, v in other.rows.items():
            self.rows[k + off] = v


def trace_whole(reqs: Dict[str, List[int]]) -> Trace:
    """Each request alone and whole, logits at every position."""
    t = Trace()
    for name, ids in reqs.items():
        t.add([(name, ids, range(len(ids)), 0)], end=[name])
    return t


def trace_tail(reqs: Dict[str, List[int]], tail: int = 32) -> Trace:
    """Most of it in one step, then the last `tail` tokens one by one."""
    t = Trace()
    for name, ids in reqs.items():
        head = max(len(ids) - tail, 1)
        t.add([(name, ids[:head], range(head), 0)])
        for p in range(head, len(ids)):
            t.add([(name, ids[p:p + 1], [0], p)], end=[name] if p == len(ids) - 1 else [])
        if head == len(ids):
            t.add([], end=[name])
    return t


def trace_portions(reqs: Dict[str, List[int]], sizes=(7, 2, 13, 2, 5, 3, 16, 2, 9, 4, 17, 2)) -> Trace:
    """In portions of changing size, down to two tokens."""
    t = Trace()
    for name, ids in reqs.items():
        p, k = 0, 0
        while p < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - p)
            if len(ids) - p - n == 1:  # never leave a single token: portions are at least two
                n += 1
            t.add([(name, ids[p:p + n], range(n), p)], end=[name] if p + n == len(ids) else [])
            p += n
            k += 1
    return t


MIXED_SIZES = (2, 3, 5, 8, 13, 21)
# ... and portions long enough for the kernels that serve a scheduler's real mixed steps (a long
# prompt portion beside single decoded tokens): tensor-core attention of portions, token-tile products
MIXED_SIZES_LONG = MIXED_SIZES + (40, 70, 130)


def trace_mixed(reqs: Dict[str, List[int]], max_tokens: int, seed: int = 0, max_live: int = 4,
                sizes: Sequence[int] = MIXED_SIZES) -> Trace:
    """Up to `max_live` live requests; portions of some (of the given sizes) beside single (decoded)
    tokens of others; a request starts only when the pool (max_tokens, each request rounded up to
    64) has room, so later requests reuse the pages of finished ones."""
    rng = np.random.default_rng(seed)
    t = Trace()
    waiting = list(reqs.items())
    live: Dict[str, dict] = {}
    while waiting or live:
        while waiting and len(live) < max_live:
            name, ids = waiting[0]
            used = sum(round64(len(v["ids"])) for v in live.values())
            if used + round64(len(ids)) > max_tokens:
                break
            waiting.pop(0)
            # the prompt part is cut into portions; the rest comes token by token
            live[name] = {"ids": ids, "pos": 0, "prompt": int(len(ids) * rng.uniform(0.4, 0.8))}
        assert live, "max_tokens is too small for the next request"
        entries, end = [], []
        for name, st in live.items():
            if rng.uniform() < 0.2 and len(live) > 1:
                continue  # a request may sit out a step
            ids, p = st["ids"], st["pos"]
            if p < st["prompt"]:
                n = int(min(rng.choice(list(sizes)), st["prompt"] - p))
                if st["prompt"] - p - n == 1:
                    n += 1
            else:
                n = 1
            n = min(n, len(ids) - p)
            entries.append((name, ids[p:p + n], range(n), p))
            st["pos"] = p + n
            if st["pos"] == len(ids):
                end.append(name)
        t.add(entries, end=end)
        for name in end:
            del live[name]
    return t


def run_trace(model_dir: str, dtype: str, trace: Trace, out_dir: str, max_tokens: int, block_size: int,
              vocab: int) -> Dict[Tuple[str, int], np.ndarray]:
    """Runs bin/trace_run as a user would and returns {(request, position): logits row}."""
    text = "".join(json.dumps(s) + "\n" for s in trace.steps)
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens), "--block-size", str(block_size)]
    r = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, f"trace_run failed ({r.returncode}):\n{r.stderr[-3000:]}"
    done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == list(range(len(trace.steps))), "a `done` line is missing or out of order"
    out: Dict[Tuple[str, int], np.ndarray] = {}
    for k, rows in trace.rows.items():
        a = np.fromfile(os.path.join(out_dir, f"{k}.f32"), dtype="<f4").reshape(len(rows), vocab)
        for i, key in enumerate(rows):
            assert key not in out, f"{key} written twice"
            out[key] = a[i]
    return out
