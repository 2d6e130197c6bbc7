"""Each part of a layer alone (norm, position encoding, attention mixer, feed-forward, block) on the
GPU against the plain implementation's function for it, in 32-bit and in bfloat16, at sizes that are
not the tiny models'."""

import numpy as np
import pytest
import torch

import plain_llama as P
from gpu_helpers import DEV, Harness
from llmengine.parts import (AttentionSpec, BlockSpec, GatedMLPSpec, NormSpec, PositionSpec, Residual, build_part)

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def tol(dt, scale=1.0):
    return dict(atol=3e-5 * scale, rtol=3e-5) if dt == torch.float32 else dict(atol=2e-2 * scale, rtol=2e-2)


def rnd(*shape, seed=0, std=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * std


def as_dev(t, dt):
    return t.to(dt).to(DEV)


def whole(delta):
    """A part's delta may come as partial sums [parts, tokens, hidden]."""
    return delta if delta.dim() == 2 else delta.sum(0)


def bf(t, dt):
    """The value a tensor has after being stored in dtype dt (as float32, on the CPU)."""
    return t.to(dt).float()


@pytest.mark.parametrize("dt", DTYPES)
def test_norm_part(dt):
    h = Harness(dt)
    spec = NormSpec("rmsnorm", 200, 3e-6, "w")
    norm = build_part("norm", spec, h.env)
    assert [(n.name, n.shape, n.precision) for n in norm.tensor_needs(spec)] == [("w", (200,), "float32")]
    w = 1 + 0.1 * rnd(200, seed=1)
    norm.load({"w": w.to(DEV)})
    ctx = h.ctx([(1, 9, [])])
    x, d = rnd(9, 200, seed=2), rnd(9, 200, seed=3)
    res = Residual(x.to(DEV).clone())
    res.pending = d.to(DEV)
    out = norm.forward(res, ctx)
    assert res.pending is None
    torch.testing.assert_close(res.h.cpu(), x + d, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(out.float().cpu(), torch.from_numpy(P.rmsnorm((x + d).numpy(), w.numpy(), 3e-6)), **tol(dt, 4))


@pytest.mark.parametrize("dt", DTYPES)
def test_position_part_matches_reference_tables(dt):
    spec = PositionSpec(kind="rope", head_dim=48, theta=500000.0, max_positions=400, scaling_factor=8.0,
                        low_freq_factor=1.0, high_freq_factor=4.0, original_max_positions=64)
    h = Harness(dt, nkv=2, hd=48)
    pos = build_part("position", spec, h.env)
    inv = P.llama3_inv_freq(48, np.float32(500000.0), True, np.float32(8), np.float32(1), np.float32(4), 64)
    cos, sin = P.rope_tables(inv, 400, 48)
    assert np.array_equal(pos.cos.cpu().numpy(), cos[:, :24]) and np.array_equal(pos.sin.cpu().numpy(), sin[:, :24])
    plain = build_part("position", PositionSpec(kind="rope", head_dim=48, theta=10000.0, max_positions=50), h.env)
    c2, _ = P.rope_tables(P.llama3_inv_freq(48, np.float32(10000.0), False, 1, 1, 1, 0), 50, 48)
    assert np.array_equal(plain.cos.cpu().numpy(), c2[:, :24])


def _attention_spec(hidden, nq, nkv, hd, window=0, max_pos=300):
    pos = PositionSpec(kind="rope", head_dim=hd, theta=10000.0, max_positions=max_pos)
    return AttentionSpec(kind="attention", hidden=hidden, num_heads=nq, num_kv_heads=nkv, head_dim=hd, position=pos,
                         q_weight="q", k_weight="k", v_weight="v", o_weight="o", window=window)


def _plain_attention(x, w, nq, nkv, hd, window=0):
    T = x.shape[0]
    inv = P.llama3_inv_freq(hd, np.float32(10000.0), False, 1, 1, 1, 0)
    cos, sin = P.rope_tables(inv, T, hd)
    q = P.apply_rope(P.linear(x, w["q"]).reshape(T, nq, hd), cos, sin)
    k = P.apply_rope(P.linear(x, w["k"]).reshape(T, nkv, hd), cos, sin)
    v = P.linear(x, w["v"]).reshape(T, nkv, hd)
    if window == 0:
        a = P.causal_gqa_attention(q, k, v)
    else:  # the plain implementation has no window: restrict the keys here
        a = np.zeros((T, nq * hd), dtype=np.float32)
        for t in range(T):
            lo = max(0, t - window + 1)
            a[t] = _one_query(q[t], k[lo:t + 1], v[lo:t + 1], nq, nkv, hd)
    return P.linear(a, w["o"])


def _one_query(q, k, v, nq, nkv, hd):
    out = np.zeros((nq, hd), dtype=np.float32)
    for hh in range(nq):
        s = (k[:, hh // (nq // nkv)] @ q[hh]) / np.sqrt(np.float32(hd))
        p = np.exp(s - s.max())
        out[hh] = (p / p.sum()) @ v[:, hh // (nq // nkv)]
    return out.reshape(-1)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("hidden,nq,nkv,hd,window,page", [(96, 6, 2, 16, 0, 4), (80, 5, 1, 32, 0, 16), (64, 4, 4, 48, 11, 8)])
def test_attention_mixer_in_portions(dt, hidden, nq, nkv, hd, window, page):
    """The mixer alone, fed one request in portions (and a second request in between), equals plain
    attention over the whole sequence."""
    T = 45
    h = Harness(dt, page=page, pages=40, windows=(window,), nkv=nkv, hd=hd)
    spec = _attention_spec(hidden, nq, nkv, hd, window)
    mixer = build_part("mixer", spec, h.env)
    assert mixer.cache_needs()[0].window == window and mixer.cache_needs()[0].num_kv_heads == nkv
    w = {"q": rnd(nq * hd, hidden, seed=1, std=0.15), "k": rnd(nkv * hd, hidden, seed=2, std=0.15),
         "v": rnd(nkv * hd, hidden, seed=3, std=0.15), "o": rnd(hidden, nq * hd, seed=4, std=0.15)}
    w = {k: bf(v, dt) for k, v in w.items()}
    mixer.load({k: as_dev(v, dt) for k, v in w.items()})
    x = bf(rnd(T, hidden, seed=5), dt)
    other = bf(rnd(7, hidden, seed=6), dt)
    ref = _plain_attention(x.numpy(), {k: v.numpy() for k, v in w.items()}, nq, nkv, hd, window)
    got = torch.empty(T, hidden)
    p = 0
    for n in (5, 2, 13, 1, 1, 16, 7):
        batch = [(1, n, [])] + ([(2, 7, [])] if p == 7 else [])
        ctx = h.ctx(batch)
        xin = torch.cat([x[p:p + n]] + ([other] if p == 7 else []))
        delta = mixer.forward(as_dev(xin, dt), ctx, h.cache)
        assert delta.dtype == torch.float32
        got[p:p + n] = whole(delta)[:n].cpu()
        p += n
    torch.testing.assert_close(got, torch.from_numpy(ref), **tol(dt, 3))


@pytest.mark.parametrize("dt", DTYPES)
def test_feed_forward_part(dt):
    h = Harness(dt)
    spec = GatedMLPSpec(kind="gated_mlp", hidden=72, intermediate=200, gate_weight="g", up_weight="u", down_weight="d")
    ff = build_part("feed_forward", spec, h.env)
    assert sorted((n.name, n.shape) for n in ff.tensor_needs(spec)) == [("d", (72, 200)), ("g", (200, 72)), ("u", (200, 72))]
    w = {"g": bf(rnd(200, 72, seed=1, std=0.2), dt), "u": bf(rnd(200, 72, seed=2, std=0.2), dt), "d": bf(rnd(72, 200, seed=3, std=0.2), dt)}
    ff.load({k: as_dev(v, dt) for k, v in w.items()})
    x = bf(rnd(11, 72, seed=4), dt)
    ctx = h.ctx([(1, 11, [])])
    out = whole(ff.forward(as_dev(x, dt), ctx))
    ref = P.swiglu_mlp(x.numpy(), w["g"].numpy(), w["u"].numpy(), w["d"].numpy())
    torch.testing.assert_close(out.cpu(), torch.from_numpy(ref), **tol(dt, 3))
    with pytest.raises(ValueError, match="activation"):
        build_part("feed_forward", GatedMLPSpec("gated_mlp", 8, 8, "g", "u", "d", activation="gelu"), h.env)


@pytest.mark.parametrize("dt", DTYPES)
def test_block_part(dt):
    hidden, nq, nkv, hd, T = 64, 4, 2, 16, 19
    h = Harness(dt, page=4, pages=16, nkv=nkv, hd=hd)
    spec = BlockSpec(kind="pre_norm", norm1=NormSpec("rmsnorm", hidden, 1e-5, "n1"), mixer=_attention_spec(hidden, nq, nkv, hd),
                     norm2=NormSpec("rmsnorm", hidden, 1e-5, "n2"),
                     feed_forward=GatedMLPSpec("gated_mlp", hidden, 176, "g", "u", "d"))
    block = build_part("block", spec, h.env)
    assert len(block.tensor_needs(spec)) == 9
    w = {"q": rnd(64, 64, seed=1, std=0.1), "k": rnd(32, 64, seed=2, std=0.1), "v": rnd(32, 64, seed=3, std=0.1),
         "o": rnd(64, 64, seed=4, std=0.1), "g": rnd(176, 64, seed=5, std=0.1), "u": rnd(176, 64, seed=6, std=0.1),
         "d": rnd(64, 176, seed=7, std=0.1)}
    w = {k: bf(v, dt) for k, v in w.items()}
    n1, n2 = 1 + 0.1 * rnd(64, seed=8), 1 + 0.1 * rnd(64, seed=9)
    tensors = {k: as_dev(v, dt) for k, v in w.items()}
    tensors.update(n1=n1.to(DEV), n2=n2.to(DEV))
    block.load(tensors)
    x = rnd(T, hidden, seed=10)
    wn = {k: v.numpy() for k, v in w.items()}
    hh = x.numpy()
    hh = hh + _plain_attention(P.rmsnorm(hh, n1.numpy(), 1e-5), wn, nq, nkv, hd)
    hh = hh + P.swiglu_mlp(P.rmsnorm(hh, n2.numpy(), 1e-5), wn["g"], wn["u"], wn["d"])
    ctx = h.ctx([(1, T, [])])
    res = block.forward(Residual(x.to(DEV).clone()), ctx, h.cache)
    h.env.ops.residual_add(res.h, res.pending)
    torch.testing.assert_close(res.h.cpu(), torch.from_numpy(hh), **tol(dt, 3))
