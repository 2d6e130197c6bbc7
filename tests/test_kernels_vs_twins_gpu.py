"""Each CUDA kernel against its plain C++ twin (llmengine/csrc/ref/kernels_ref.cpp through
tests/cpp_twins.py): the twin is a scalar loop on the host that restates the reference's formula;
the kernel gets the same inputs on the device. Sizes differ from those of the tiny models and of
test_kernels_gpu.py: odd widths, head sizes 48 and 80, a vocabulary of 50,021."""
import math

import numpy as np
import pytest
import torch

import cpp_twins as C
from test_kernels_gpu import Batch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from llmengine.ops import get_ops
    return get_ops()


def rnd(*shape, dtype=torch.float32, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


def host(t):
    return t.detach().float().cpu().numpy()


def close(got, want, dt, scale=1.0):
    a = 2e-5 * scale if dt == torch.float32 else 1.6e-2 * scale
    np.testing.assert_allclose(host(got), want, atol=a, rtol=2e-5 if dt == torch.float32 else 1.6e-2)


@pytest.mark.parametrize("dt", DTYPES)
def test_embedding(ops, dt):
    table = rnd(777, 136, dtype=dt, seed=1)
    ids = torch.tensor([776, 0, 3, 3, 500, 1], dtype=torch.int32)
    out = torch.empty(6, 136, dtype=torch.float32, device=DEV)
    sumsq = torch.zeros(6, dtype=torch.float32, device=DEV)
    ops.embed(table.to(DEV), ids.to(DEV), out, sumsq=sumsq)
    want = C.embed(host(table), ids.numpy())
    np.testing.assert_array_equal(host(out), want)
    np.testing.assert_allclose(host(sumsq), (want.astype(np.float64) ** 2).sum(1), rtol=1e-5)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("n,dim,eps", [(3, 72, 1e-5), (33, 1000, 1e-6), (130, 3080, 1e-5)])
def test_norm_with_the_residual_sum(ops, dt, n, dim, eps):
    h, w, delta = rnd(n, dim, seed=2), 1.0 + rnd(dim, seed=3, std=0.2), rnd(4, n, dim, seed=4, std=0.5)
    want, h_after = C.rmsnorm(host(h), host(w), eps, delta=host(delta), round_bf16=dt == torch.bfloat16)
    hd_, out = h.to(DEV), torch.empty(n, dim, dtype=dt, device=DEV)
    ops.rmsnorm(hd_, w.to(DEV), eps, out, delta=delta.to(DEV))
    np.testing.assert_allclose(host(hd_), h_after, atol=2e-6, rtol=1e-6)
    close(out, want, dt, 4)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("M,N,K", [(2, 11, 24), (19, 333, 136), (150, 520, 264), (5, 3080, 1000)])
def test_product(ops, dt, M, N, K):
    a, w = rnd(M, K, dtype=dt, seed=5), rnd(N, K, dtype=dt, seed=6, std=0.1)
    want = C.gemm(host(a), host(w))
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.gemm(a.to(DEV), w.to(DEV), out)
    close(out, want, torch.float32 if dt == torch.float32 else dt, math.sqrt(K) * 0.1 * (1.0 if dt == torch.float32 else 0.1))


@pytest.mark.parametrize("dt", DTYPES)
def test_activation(ops, dt):
    n, ff = 9, 1336
    gu = rnd(n, 2 * ff, dtype=dt, seed=7, std=2.5)
    out = torch.empty(n, ff, dtype=dt, device=DEV)
    ops.silu_mul(gu.to(DEV), out)
    close(out, C.silu_mul(host(gu[:, :ff]), host(gu[:, ff:])), dt, 4)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,page", [(5, 1, 48, 8), (6, 3, 80, 16), (8, 2, 64, 32)])
def test_rotation_and_cache_write(ops, dt, nq, nkv, hd, page):
    """Two requests, one a portion from the middle of a page, the other a single token; the rotation
    table from the twin with the scaled frequencies (the device gets the same table, so what is
    compared is the rotation and the placement in the pages)."""
    cos, sin = C.rope_tables(hd, 500000.0, 400, (8.0, 1.0, 4.0, 128))
    b = Batch([(page + 3, 2 * page + 5), (390, 1)])
    n, width = b.n_tokens, (nq + 2 * nkv) * hd
    n_pages = 400 // page + 8
    table = torch.full((2, 400 // page + 1), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(8)).int()
    table[0, :5], table[1, :400 // page + 1] = perm[:5], perm[5:5 + 400 // page + 1]
    qkv = rnd(n, width, dtype=dt, seed=9)
    kc0 = rnd(n_pages, nkv, page, hd, dtype=dt, seed=10)
    vc0 = rnd(n_pages, nkv, page, hd, dtype=dt, seed=11)
    want_qkv, want_k, want_v = C.rope_kv_write(host(qkv), host(b.positions).astype(np.int32), host(b.token_seq).astype(np.int32),
                                               table.numpy(), cos, sin, host(kc0), host(vc0), nq, nkv, hd, round_bf16=dt == torch.bfloat16)
    q_dev, kc, vc = qkv.to(DEV), kc0.to(DEV), vc0.to(DEV)
    ops.rope_kv_write(q_dev, b.positions, b.token_seq, table.to(DEV), torch.from_numpy(cos).to(DEV), torch.from_numpy(sin).to(DEV),
                      kc, vc, n, nq, nkv, hd)
    close(q_dev[:, :nq * hd], want_qkv[:, :nq * hd], dt, 2)
    close(kc, want_k, dt, 2)   # rows that no token wrote keep their old values on both sides
    np.testing.assert_array_equal(host(vc), want_v)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,page,window", [(5, 1, 48, 8, 0), (6, 3, 80, 16, 0), (8, 2, 64, 32, 0), (4, 2, 128, 16, 75), (9, 3, 32, 4, 0)])
def test_attention_over_pages(ops, dt, nq, nkv, hd, page, window):
    """A prompt portion of 90 tokens that starts at position 210 beside two decoded tokens; pages in
    a shuffled order; one far key per request scaled so that it carries the softmax if it is read."""
    lens = [300, 41, 1000]
    n_pages = sum((L + page - 1) // page for L in lens) + 2
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(12)).int()
    table = torch.full((3, (1000 + page - 1) // page), -1, dtype=torch.int32)
    at = 0
    for s, L in enumerate(lens):
        nb = (L + page - 1) // page
        table[s, :nb] = perm[at:at + nb]
        at += nb
    kc, vc = rnd(n_pages, nkv, page, hd, dtype=dt, seed=13), rnd(n_pages, nkv, page, hd, dtype=dt, seed=14)
    b = Batch([(210, 90), (40, 1), (999, 1)])
    q = rnd(b.n_tokens, nq * hd, dtype=dt, seed=15)
    if window == 0:  # key 3 of request 2 (997 places back) in line with the decoded token's first head
        kc[int(table[2, 3 // page]), 0, 3 % page] = (q[-1, :hd].float() * 3.0).to(dt)
    scale = 1.0 / math.sqrt(hd)
    want = C.paged_attention(host(q), host(kc), host(vc), host(b.positions).astype(np.int32), host(b.token_seq).astype(np.int32),
                             table.numpy(), nq, nkv, hd, scale, window)
    out = torch.full((b.n_tokens, nq * hd), float("nan"), dtype=dt, device=DEV)
    ops.paged_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), b, table.to(DEV), out, nq, nkv, hd, scale, window)
    close(out, want, dt, 2)
    assert ops.tensor_core_error() == 0


def test_token_choice(ops):
    n, vocab = 24, 50021
    logits = rnd(n, vocab, seed=16, std=2.0)
    logits[1, 7] = logits[1, vocab - 1] = 30.0  # a tie in a greedy row: the first index wins
    temps = torch.tensor([0.0, 0.0, 0.6, 1.0, 1.7, 0.3] * 4)
    seeds = torch.arange(n, dtype=torch.int32) * 7 + 1
    draws = torch.arange(n, dtype=torch.int32) % 5
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV), out)
    greedy = C.sample(host(logits))
    assert out.cpu().tolist() == greedy.tolist() and greedy[1] == 7
    ops.sample(logits.to(DEV), out, temps.to(DEV), seeds.to(DEV), draws.to(DEV))
    want = C.sample(host(logits), temps.numpy(), seeds.numpy(), draws.numpy())
    got = out.cpu().numpy()
    # a sampled row is the argmax of logit / temperature + Gumbel noise from a counter-based hash: the
    # device's logarithm may round otherwise than the host's, which can turn a near-tie in one row
    differ = np.nonzero(got != want)[0]
    assert len(differ) <= 1 and all(temps[r] > 0 for r in differ), (got, want)
