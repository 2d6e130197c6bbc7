"""The plain C++ twins of the kernels (csrc/ref/kernels_ref.cpp) against the plain Python
implementation, part by part and as a whole small model (no GPU): two restatements of the
reference's formulas, in two languages, that share no code."""
import math

import numpy as np
import pytest

import cpp_twins as C
import plain_llama as P
from tiny import TINY_A, TINY_B


def rnd(*shape, seed=0, std=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * std).astype(np.float32)


def test_norm_product_activation_and_embedding():
    h, w = rnd(5, 70, seed=1), 1.0 + rnd(70, seed=2, std=0.1)
    out, _ = C.rmsnorm(h, w, 1e-5)
    np.testing.assert_allclose(out, P.rmsnorm(h, w, 1e-5), atol=2e-6, rtol=2e-6)
    delta = rnd(3, 5, 70, seed=3)
    out, h2 = C.rmsnorm(h, w, 1e-6, delta=delta)
    np.testing.assert_allclose(h2, h + delta.sum(0), atol=1e-6)
    np.testing.assert_allclose(out, P.rmsnorm(h + delta.sum(0), w, 1e-6), atol=2e-6, rtol=2e-6)
    a, m = rnd(7, 50, seed=4), rnd(13, 50, seed=5)
    np.testing.assert_allclose(C.gemm(a, m), P.linear(a, m), atol=2e-5, rtol=2e-5)
    g, u = rnd(4, 33, seed=6, std=3.0), rnd(4, 33, seed=7)
    np.testing.assert_allclose(C.silu_mul(g, u), P.silu(g) * u, atol=1e-6, rtol=1e-6)
    table = rnd(20, 9, seed=8)
    np.testing.assert_array_equal(C.embed(table, [3, 19, 0, 3]), P.embed(table, [3, 19, 0, 3]))


@pytest.mark.parametrize("hd,theta,scaling", [(16, 10000.0, None), (32, 500000.0, (8.0, 1.0, 4.0, 64)), (128, 500000.0, (32.0, 1.0, 4.0, 8192))])
def test_rotation_tables(hd, theta, scaling):
    cos, sin = C.rope_tables(hd, theta, 300, scaling)
    inv = P.llama3_inv_freq(hd, np.float32(theta), scaling is not None, *(np.float32(v) for v in (scaling or (1, 1, 1))[:3]),
                            (scaling or (0, 0, 0, 0))[3])
    pc, ps = P.rope_tables(inv, 300, hd)
    np.testing.assert_array_equal(cos, pc[:, :hd // 2])
    np.testing.assert_array_equal(sin, ps[:, :hd // 2])


@pytest.mark.parametrize("nq,nkv,hd,page,window", [(4, 2, 16, 4, 0), (6, 1, 32, 16, 0), (3, 3, 8, 8, 5)])
def test_rotation_cache_write_and_attention(nq, nkv, hd, page, window):
    """One request of T tokens through rotation, the paged cache (pages scattered) and attention,
    against the plain implementation on the whole sequence."""
    T = 37
    q, k, v = rnd(T, nq, hd, seed=1), rnd(T, nkv, hd, seed=2), rnd(T, nkv, hd, seed=3)
    cos, sin = C.rope_tables(hd, 10000.0, T)
    n_pages = (T + page - 1) // page
    table = np.random.default_rng(5).permutation(n_pages + 3)[:n_pages].astype(np.int32)[None, :]
    kc = np.zeros((n_pages + 3, nkv, page, hd), dtype=np.float32)
    vc = np.zeros_like(kc)
    qkv = np.concatenate([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], axis=1)
    pos = np.arange(T, dtype=np.int32)
    qkv2, kc, vc = C.rope_kv_write(qkv, pos, np.zeros(T, np.int32), table, cos, sin, kc, vc, nq, nkv, hd)
    full_c, full_s = np.concatenate([cos, cos], 1), np.concatenate([sin, sin], 1)
    q_rot, k_rot = P.apply_rope(q, full_c, full_s), P.apply_rope(k, full_c, full_s)
    np.testing.assert_allclose(qkv2[:, :nq * hd].reshape(T, nq, hd), q_rot, atol=1e-6)
    for t in (0, page - 1, page, T - 1):  # the cache rows at page edges
        np.testing.assert_allclose(kc[table[0, t // page], :, t % page, :], k_rot[t], atol=1e-6)
        np.testing.assert_array_equal(vc[table[0, t // page], :, t % page, :], v[t])
    out = C.paged_attention(qkv2[:, :nq * hd], kc, vc, pos, np.zeros(T, np.int32), table, nq, nkv, hd, 1.0 / math.sqrt(hd), window)
    if window == 0:
        ref = P.causal_gqa_attention(q_rot, k_rot, v)
    else:
        ref = np.stack([P.causal_gqa_attention(q_rot[max(0, t - window + 1):t + 1], k_rot[max(0, t - window + 1):t + 1],
                                               v[max(0, t - window + 1):t + 1])[-1] for t in range(T)])
    np.testing.assert_allclose(out, ref, atol=3e-6, rtol=1e-5)


def test_token_choice():
    logits = rnd(6, 1000, seed=9, std=2.0)
    logits[0, 17] = logits[0, 900] = 50.0  # a tie: the first index wins
    assert C.sample(logits).tolist() == [P.argmax_first(r) for r in logits] and C.sample(logits)[0] == 17
    temps = np.array([0.0, 0.7, 1.0, 1.3, 0.0, 2.0], dtype=np.float32)
    seeds, draws = np.arange(6) + 40, np.arange(6) * 3
    got = C.sample(logits, temps, seeds, draws)
    assert got.tolist() == [P.sample_token(logits[r], float(temps[r]), int(seeds[r]), int(draws[r])) for r in range(6)]


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B], ids=["a", "b"])
def test_a_whole_model_from_the_twins(cfg, tmp_path):
    """The layer loop of the reference (src/engine.cpp:105-261) put together from the C++ twins, with
    a paged cache, against the plain implementation's logits."""
    import torch

    from tiny import make_model_dir, random_ids
    d = str(tmp_path / "m")
    make_model_dir(d, cfg, torch.float32)
    pc, w = P.read_model(d)
    T, page = 21, 4
    ids = random_ids(T, cfg["vocab_size"], 3)
    nq, nkv, hd, eps = pc["num_attention_heads"], pc["num_key_value_heads"], pc["head_dim"], float(pc["rms_norm_eps"])
    sc = (float(pc["rope_factor"]), float(pc["rope_low_freq_factor"]), float(pc["rope_high_freq_factor"]), pc["rope_original_max_pos"]) \
        if pc["rope_has_scaling"] else None
    cos, sin = C.rope_tables(hd, float(pc["rope_theta"]), T, sc)
    n_pages = (T + page - 1) // page
    table = np.arange(n_pages, dtype=np.int32)[::-1].copy()[None, :]
    pos, seq = np.arange(T, dtype=np.int32), np.zeros(T, np.int32)
    h = C.embed(w["model.embed_tokens.weight"], ids)
    for l in range(pc["num_hidden_layers"]):
        p = f"model.layers.{l}."
        x, _ = C.rmsnorm(h, w[p + "input_layernorm.weight"], eps)
        qkv = np.concatenate([C.gemm(x, w[p + f"self_attn.{n}_proj.weight"]) for n in "qkv"], axis=1)
        kc = np.zeros((n_pages, nkv, page, hd), dtype=np.float32)
        vc = np.zeros_like(kc)
        qkv, kc, vc = C.rope_kv_write(qkv, pos, seq, table, cos, sin, kc, vc, nq, nkv, hd)
        a = C.paged_attention(qkv[:, :nq * hd], kc, vc, pos, seq, table, nq, nkv, hd, 1.0 / math.sqrt(hd))
        h = h + C.gemm(a, w[p + "self_attn.o_proj.weight"])
        x, _ = C.rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps)
        act = C.silu_mul(C.gemm(x, w[p + "mlp.gate_proj.weight"]), C.gemm(x, w[p + "mlp.up_proj.weight"]))
        h = h + C.gemm(act, w[p + "mlp.down_proj.weight"])
    x, _ = C.rmsnorm(h, w["model.norm.weight"], eps)
    logits = C.gemm(x, w["lm_head.weight"])
    ref = P.forward_logits(pc, w, ids)
    np.testing.assert_allclose(logits, ref, atol=2e-5, rtol=2e-5)
    assert (logits.argmax(-1) == ref.argmax(-1)).all()
