"""The products of a step with few tokens that finish their K splits themselves (the CTA of each
tile of outputs that arrives last adds them, adds the sum into the residual stream and leaves the
next norm's input prepared), and the consumers that multiply a norm's 1/rms in where partial sums
are added: each against plain float64 arithmetic, at sizes with tails, twice in a row (the
counters must be left at zero)."""
import math

import pytest
import torch

from test_kernels_gpu import Batch, _paged_setup

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from llmengine.ops import get_ops
    o = get_ops()
    before, o.meet_products, o.add_into_stream = (o.meet_products, o.add_into_stream), True, True  # options that are off by default
    yield o
    o.meet_products, o.add_into_stream = before


def rnd(*shape, dtype=torch.float32, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype).to(DEV)


def rms_scale(sumsq, dim, eps):
    return 1.0 / torch.sqrt(sumsq.double().sum(1) / dim + eps)


@pytest.mark.parametrize("M,N,K", [(1, 2048, 2048), (8, 2048, 8192), (64, 3072, 1024), (5, 384, 192), (17, 200, 64), (33, 1000, 520)])
@pytest.mark.parametrize("with_next", [True, False])
def test_product_that_adds_itself_into_the_stream(ops, M, N, K, with_next):
    from llmengine.engine.context import Workspace
    ws = Workspace(torch.device(DEV))
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, std=0.05)
    h0 = rnd(M + 3, N, seed=3, std=2.0)  # rows beyond the step's tokens stay as they are
    next_w = 1.0 + rnd(N, seed=4, std=0.2)
    tiles = (N + 127) // 128
    assert ops.can_meet(a, w)
    want_h = h0[:M].double() + a.double() @ w.double().t()
    for _ in range(2):
        h = h0.clone()
        sumsq = torch.full((M + 3, tiles), float("nan"), device=DEV)
        scaled = torch.full((M + 3, N), float("nan"), dtype=torch.bfloat16, device=DEV) if with_next else None
        ops.gemm_meet(a, w, h, ws, "t.parts", next_w=next_w if with_next else None, scaled=scaled, sumsq=sumsq)
        torch.testing.assert_close(h[:M].double(), want_h, atol=2e-5 * math.sqrt(K), rtol=2e-5)
        assert torch.equal(h[M:], h0[M:])
        torch.testing.assert_close(sumsq[:M].double().sum(1), (want_h ** 2).sum(1), rtol=1e-4, atol=1e-4)
        if with_next:
            torch.testing.assert_close(scaled[:M].double(), (h[:M] * next_w).double(), rtol=8e-3, atol=1e-6)  # bfloat16 rounding
        assert ops.tensor_core_error() == 0
    assert int(ws.get_zeroed("gemm.meet_counters", (tiles,), torch.int32).abs().sum()) == 0
    # the same sums in the same order as the partial-sum path: equal bit for bit
    parts = ops.gemm_partials(a, w, Workspace(torch.device(DEV)), "t.parts2")
    delta = parts[0].clone()
    for z in range(1, parts.shape[0]):
        delta += parts[z]
    assert torch.equal(h[:M], h0[:M] + delta)


@pytest.mark.parametrize("M,N,K", [(1, 1000, 256), (8, 128256, 2048), (40, 509, 192)])
def test_product_divided_by_the_rows_root_mean_square(ops, M, N, K):
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=5), rnd(N, K, dtype=torch.bfloat16, seed=6, std=0.05)
    sumsq = rnd(M, 7, seed=7).abs() * 100.0
    eps, dim = 1e-5, 300
    out = torch.full((M, N), float("nan"), device=DEV)
    ops.gemm_scaled(a, w, out, ops.row_scale(sumsq, dim, eps))
    want = (a.double() @ w.double().t()) * rms_scale(sumsq, dim, eps)[:, None]
    torch.testing.assert_close(out.double(), want, atol=2e-5 * math.sqrt(K), rtol=2e-5)
    assert ops.tensor_core_error() == 0


def test_activation_from_partial_sums_with_a_row_scale(ops):
    n, ff, p = 7, 384, 5
    parts = rnd(p, n, 2 * ff, seed=8)
    sumsq = rnd(n, 3, seed=9).abs() * 50.0
    sc = rms_scale(sumsq, 64, 1e-6)
    for block in (0, 128):
        out = torch.empty(n, ff, dtype=torch.bfloat16, device=DEV)
        ops.silu_mul_partials(parts, out, block=block, row_scale=ops.row_scale(sumsq, 64, 1e-6))
        plain = torch.empty(n, ff, dtype=torch.float32, device=DEV)
        scaled_parts = (parts.double().sum(0) * sc[:, None]).float()[None].contiguous()
        ops.silu_mul_partials(scaled_parts, plain, block=block)
        torch.testing.assert_close(out.float(), plain, atol=2e-2, rtol=1.6e-2)


def test_embedding_leaves_the_first_norms_input(ops):
    table = rnd(300, 200, dtype=torch.bfloat16, seed=10)
    ids = torch.tensor([299, 0, 17, 17], dtype=torch.int32, device=DEV)
    w = 1.0 + rnd(200, seed=11, std=0.3)
    out, sumsq = torch.empty(4, 200, device=DEV), torch.empty(4, 1, device=DEV)
    scaled = torch.empty(4, 200, dtype=torch.bfloat16, device=DEV)
    ops.embed(table, ids, out, sumsq=sumsq, next_w=w, scaled=scaled)
    rows = table[ids.long()].float()
    assert torch.equal(out, rows) and torch.equal(scaled, (rows * w).to(torch.bfloat16))
    torch.testing.assert_close(sumsq[:, 0], (rows ** 2).sum(1), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("nq,nkv,hd,page,window", [(32, 8, 64, 16, 0), (24, 8, 128, 16, 0), (8, 2, 64, 8, 100)])
@pytest.mark.parametrize("n_parts", [1, 6])
def test_decoding_attention_and_rotation_take_the_row_scale(ops, nq, nkv, hd, page, window, n_parts):
    """q|k|v partial sums with a 1/rms per token still owed: the one-kernel decoding path and the
    rotation kernel against the same kernels on sums that were multiplied beforehand."""
    dt = torch.bfloat16
    seq_lens = [1, 17, 64, 321, 700]
    n_pages = sum((L + page - 1) // page for L in seq_lens) + 3
    kc0, vc0, table, _ = _paged_setup(dt, nkv, hd, page, seq_lens, n_pages, seed=12)
    b = Batch([(L - 1, 1) for L in seq_lens])
    n, width = b.n_tokens, (nq + 2 * nkv) * hd
    parts = rnd(n_parts, n, width, seed=13) / math.sqrt(n_parts) * 3.0
    sumsq = rnd(n, 16, seed=14).abs() * 40.0
    dim, eps = 2048, 1e-5
    sc = rms_scale(sumsq, dim, eps)
    pre = (parts.double().sum(0) * sc[:, None]).float()[None].contiguous()  # one part, already scaled
    ang = torch.arange(800, dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(hd // 2, dtype=torch.float64) / (hd // 2)))[None]
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    scale = 1.0 / math.sqrt(hd)
    rs = ops.row_scale(sumsq, dim, eps)
    outs, caches = [], []
    for p_, extra in ((parts, {"row_scale": rs}), (pre, {})):
        kc, vc = kc0.clone(), vc0.clone()
        out = torch.full((n, nq * hd), float("nan"), dtype=dt, device=DEV)
        assert ops.decode_attention_fusable(b, kc, nq, nkv, hd, out)
        ops.paged_attention_decode_fused(p_, cos, sin, kc, vc, b, table, out, nq, nkv, hd, scale, window, **extra)
        outs.append(out.float()); caches.append((kc.float(), vc.float()))
    torch.testing.assert_close(outs[0], outs[1], atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(caches[0][0], caches[1][0], atol=4e-2, rtol=1.6e-2)  # keys and values: one bfloat16 rounding apart at most
    torch.testing.assert_close(caches[0][1], caches[1][1], atol=4e-2, rtol=1.6e-2)
    assert ops.tensor_core_error() == 0
    qs = []
    for p_, extra in ((parts, {"row_scale": rs}), (pre, {})):
        kc, vc = kc0.clone(), vc0.clone()
        qkv = torch.zeros(n, width, dtype=dt, device=DEV)
        ops.rope_kv_write(qkv, b.positions, b.token_seq, table, cos, sin, kc, vc, n, nq, nkv, hd, parts=p_, **extra)
        qs.append((qkv[:, :nq * hd].float(), kc.float(), vc.float()))
    for x, y in zip(qs[0], qs[1]):
        torch.testing.assert_close(x, y, atol=4e-2, rtol=1.6e-2)


@pytest.mark.parametrize("M,N,K", [(300, 2048, 192), (129, 130, 64), (2048, 3072, 128), (1100, 8704, 256), (65, 509, 520)])
def test_prompt_sized_product_that_adds_into_the_stream(ops, M, N, K):
    """One tile a CTA and the persistent kernels (tiles of 256 and of 192 outputs): every element of
    the stream is read, added to and written once, the same float32 sum as adding the product
    afterwards (bit for bit); rows beyond the step's tokens stay as they are."""
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=20), rnd(N, K, dtype=torch.bfloat16, seed=21, std=0.05)
    h0 = rnd(M + 2, N, seed=22, std=2.0)
    assert ops.can_add_into(a, w)
    h = h0.clone()
    ops.gemm_add_into(a, w, h)
    out = torch.empty(M, N, device=DEV)
    ops.gemm(a, w, out)
    assert torch.equal(h[:M], h0[:M] + out) and torch.equal(h[M:], h0[M:])
    rows = torch.tensor(sorted({0, min(127, M - 1), min(128, M - 1), M - 1})).to(DEV)
    torch.testing.assert_close(h[rows].double(), h0[rows].double() + a[rows].double() @ w.double().t(), atol=2e-5 * math.sqrt(K), rtol=2e-5)
    assert ops.tensor_core_error() == 0
