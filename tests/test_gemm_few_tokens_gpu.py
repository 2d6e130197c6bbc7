"""The product of a step with few tokens (csrc/kernels/gemm_decode.cu) alone, against float64 sums of
the same bf16 values: K pieces that meet inside a cluster (up to 8) or in global memory (up to 32),
activations fetched as bf16
rows or produced by the folded norm (with and without a row list), and the three endings: plain
(float32 / bf16), added into the residual stream with the rows' sums of squares, and SiLU(gate) * up.
Sizes with tails in every dimension."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    """The kernel library with these products switched on (the engine leaves them off by default:
    a decode step measured slower with them than with partial sums that the norm kernels add)."""
    from llmengine.ops import get_ops
    o = get_ops()
    before, o.few_token_products = o.few_token_products, True
    yield o
    o.few_token_products = before


@pytest.fixture(params=["global", "cluster"])
def space(request):
    """Where the K pieces meet: scratch of a workspace (global memory), or None (inside a cluster)."""
    from llmengine.engine.context import Workspace
    return Workspace(torch.device(DEV)) if request.param == "global" else None


def rnd(*shape, dtype=torch.float32, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype).to(DEV)


SHAPES = [(3072, 2048), (2048, 8192), (509, 200), (130, 64), (5120, 3072), (1000, 1024)]


@pytest.mark.parametrize("T", [1, 8, 17, 33, 64])
@pytest.mark.parametrize("N,K", SHAPES)
def test_plain_and_residual_from_bf16_rows(ops, space, T, N, K):
    x, w = rnd(T, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, std=0.1)
    ref = x.double() @ w.double().t()
    scale = math.sqrt(K) * 0.1
    in_cluster = space is None
    assert ops.few_token_splits(N, K, T, "plain", in_cluster) >= 1
    for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1.6e-2)):
        out = torch.full((T, N), float("nan"), dtype=dt, device=DEV)
        ops.gemm_few_tokens(w, out, "plain", x=x, ws=space)
        torch.testing.assert_close(out.double(), ref, atol=tol * scale, rtol=tol)
    # twice the same launch gives the same bits (the K pieces are added in index order)
    a = torch.empty(T, N, dtype=torch.float32, device=DEV)
    b = torch.empty(T, N, dtype=torch.float32, device=DEV)
    ops.gemm_few_tokens(w, a, "plain", x=x, ws=space)
    ops.gemm_few_tokens(w, b, "plain", x=x, ws=space)
    assert torch.equal(a, b)
    # added into the residual stream, with the parts of the new rows' sums of squares
    if ops.few_token_splits(N, K, T, "residual", in_cluster) >= (2 if in_cluster else 1):
        h0 = rnd(T, N, seed=3)
        h = h0.clone()
        parts = ops.residual_sumsq_parts(N, K, T, in_cluster)
        ss = torch.full((T, parts), float("nan"), device=DEV)
        ops.gemm_few_tokens(w, h, "residual", x=x, sumsq_out=ss, ws=space)
        want = h0.double() + ref
        torch.testing.assert_close(h.double(), want, atol=2e-5 * scale, rtol=2e-5)
        torch.testing.assert_close(ss.double().sum(1), (h.double() ** 2).sum(1), atol=1e-3, rtol=1e-5)
    assert ops.tensor_core_error() == 0


@pytest.mark.parametrize("T", [1, 8, 40, 64])
@pytest.mark.parametrize("N,K", [(3072, 2048), (509, 200), (1024, 328), (128256, 2048)])
def test_the_folded_norm(ops, space, T, N, K):
    """Activations = RMSNorm of float32 rows, computed inside the product from the rows' sums of
    squares given in parts; with a row list, the rows are picked from a larger stream."""
    rows_total = T + 5
    h = rnd(rows_total, K, seed=4)
    nw = 1.0 + rnd(K, seed=5, std=0.1)
    eps = 1e-5
    parts = 7
    true_ss = (h.double() ** 2).sum(1)
    frac = torch.softmax(rnd(rows_total, parts, seed=6).double(), dim=1)
    sumsq = (true_ss[:, None] * frac).float().contiguous()  # any split of the sum into parts
    w = rnd(N, K, dtype=torch.bfloat16, seed=7, std=0.1)
    scale = math.sqrt(K) * 0.1
    for row_list in (None, torch.tensor([(3 * i + 1) % rows_total for i in range(T)], dtype=torch.int32, device=DEV)):
        src = h[:T] if row_list is None else h[row_list.long()]
        ssr = sumsq[:T] if row_list is None else sumsq[row_list.long()]
        inv = 1.0 / torch.sqrt(ssr.sum(1) / K + eps)
        xn = ((nw * src) * inv[:, None]).bfloat16()  # (w * x) * inv, rounded as the norm kernel rounds
        ref = xn.double() @ w.double().t()
        out = torch.full((T, N), float("nan"), device=DEV)
        ops.gemm_few_tokens(w, out, "plain", norm=(h if row_list is not None else h[:T], sumsq, nw, eps, row_list), n_tokens=T, ws=space)
        # a reciprocal root that differs in its last bit moves a few activations by one bf16 step
        torch.testing.assert_close(out.double(), ref, atol=4e-3 * scale, rtol=4e-3)
    assert ops.tensor_core_error() == 0


@pytest.mark.parametrize("T", [1, 8, 33, 64])
@pytest.mark.parametrize("FF,K", [(8192, 2048), (384, 192), (1024, 512), (14336, 4096)])
def test_silu_gate_times_up(ops, space, T, FF, K):
    x = rnd(T, K, dtype=torch.bfloat16, seed=8)
    g, u = rnd(FF, K, dtype=torch.bfloat16, seed=9, std=0.1), rnd(FF, K, dtype=torch.bfloat16, seed=10, std=0.1)
    blocked = torch.stack([g.view(-1, 128, K), u.view(-1, 128, K)], dim=1).reshape(2 * FF, K).contiguous()
    gd, ud = x.double() @ g.double().t(), x.double() @ u.double().t()
    ref = gd / (1.0 + torch.exp(-gd)) * ud
    out = torch.full((T, FF), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_few_tokens(blocked, out, "swiglu", x=x, ws=space)
    scale = K * 0.01
    torch.testing.assert_close(out.double(), ref, atol=1.6e-2 * scale, rtol=1.6e-2)
    # and with the norm folded in front, as the feed-forward of a decode step runs
    h, nw = rnd(T, K, seed=11), 1.0 + rnd(K, seed=12, std=0.1)
    sumsq = ((h.double() ** 2).sum(1)[:, None] * torch.tensor([0.25, 0.75], device=DEV, dtype=torch.float64)).float().contiguous()
    inv = 1.0 / torch.sqrt((h.double() ** 2).sum(1).float() / K + 1e-6)
    xn = ((nw * h) * inv[:, None]).bfloat16()
    gd, ud = xn.double() @ g.double().t(), xn.double() @ u.double().t()
    ref = gd / (1.0 + torch.exp(-gd)) * ud
    ops.gemm_few_tokens(blocked, out, "swiglu", norm=(h, sumsq, nw, 1e-6, None), ws=space)
    torch.testing.assert_close(out.double(), ref, atol=2e-2 * scale, rtol=2e-2)
    assert ops.tensor_core_error() == 0
