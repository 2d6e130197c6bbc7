"""Properties of the plain implementation itself (it is the oracle of every GPU test)."""
import tempfile

import numpy as np
import torch

import plain_llama as P
from tiny import TINY_A, TINY_B, make_model_dir, random_ids


def _model(cfg):
    with tempfile.TemporaryDirectory() as d:
        make_model_dir(d, cfg, torch.float32)
        return P.read_model(d)


def test_causal_prefix_property():
    """Logits at position t depend on tokens 0..t only."""
    for cfg in (TINY_A, TINY_B):
        pc, pw = _model(cfg)
        ids = random_ids(40, cfg["vocab_size"], 1)
        full = P.forward_logits(pc, pw, ids)
        part = P.forward_logits(pc, pw, ids[:23])
        np.testing.assert_allclose(full[:23], part, atol=2e-5, rtol=1e-5)  # BLAS blocks differ with the shape


def test_rope_tables_against_direct_formula():
    pc, _ = _model(TINY_B)
    inv = P.llama3_inv_freq(32, pc["rope_theta"], True, pc["rope_factor"], pc["rope_low_freq_factor"],
                            pc["rope_high_freq_factor"], pc["rope_original_max_pos"])
    assert inv.dtype == np.float32 and inv.shape == (16,)
    base = 1.0 / (500000.0 ** (np.arange(16) * 2 / 32))
    # highest frequencies unchanged, lowest divided by the factor
    assert abs(inv[0] - base[0]) < 1e-7 and abs(inv[-1] - base[-1] / 8.0) < 1e-9
    cos, sin = P.rope_tables(inv, 200, 32)
    p = 137
    np.testing.assert_allclose(cos[p, :16], np.cos(p * inv.astype(np.float64)), atol=1e-7)
    np.testing.assert_allclose(sin[p, 16:], np.sin(p * inv.astype(np.float64)), atol=1e-7)


def test_attention_single_key_is_value():
    q = np.random.default_rng(0).standard_normal((1, 4, 16)).astype(np.float32)
    k = np.random.default_rng(1).standard_normal((1, 2, 16)).astype(np.float32)
    v = np.random.default_rng(2).standard_normal((1, 2, 16)).astype(np.float32)
    out = P.causal_gqa_attention(q, k, v).reshape(4, 16)
    np.testing.assert_allclose(out[0], v[0, 0], atol=1e-6)
    np.testing.assert_allclose(out[3], v[0, 1], atol=1e-6)


def test_greedy_tie_takes_first_index():
    assert P.argmax_first(np.array([1.0, 3.0, 3.0, 2.0], dtype=np.float32)) == 1


def test_temperature_draws_follow_softmax():
    logits = np.array([0.0, 1.0, 2.0, -1.0], dtype=np.float32)
    counts = np.zeros(4)
    n = 4000
    for d in range(n):
        counts[P.sample_token(logits, 1.0, seed=123, draw_index=d)] += 1
    p = np.exp(logits) / np.exp(logits).sum()
    assert np.abs(counts / n - p).max() < 0.03
    assert P.sample_token(logits, 0.0, 1, 1) == 2
    # same (seed, draw) -> same token; the draw does not depend on anything else
    assert P.sample_token(logits, 0.7, 9, 4) == P.sample_token(logits, 0.7, 9, 4)


def test_generate_stops_at_eos_without_appending():
    pc, pw = _model(TINY_A)
    ids = random_ids(6, 256, 3)
    out, reason = P.generate(pc, pw, ids, 5)
    assert reason == "length" and len(out) == 11
    pc2 = dict(pc, eos_token_ids={out[8]})
    out2, reason2 = P.generate(pc2, pw, ids, 5)
    assert reason2 == "stop" and out2 == out[:out.index(out[8], 6)]
