"""Each CUDA kernel alone against a plain float32 reference of the same op, at sizes other than
the engine's tiny models use (non powers of two, tails, strided views)."""
import math

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from llmengine.ops import get_ops
    return get_ops()


def tol(dt, scale=1.0):
    return dict(atol=2e-5 * scale, rtol=2e-5) if dt == torch.float32 else dict(atol=1.6e-2 * scale, rtol=1.6e-2)


def rnd(*shape, dtype=torch.float32, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype).to(DEV)


@pytest.mark.parametrize("dt", DTYPES)
def test_embed(ops, dt):
    table = rnd(301, 200, dtype=dt)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 200, dtype=torch.float32, device=DEV)
    ops.embed(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("dim", [16, 257, 2048, 5000])
@pytest.mark.parametrize("n", [7, 70])  # few rows: a cluster of CTAs shares a row; many: one CTA a row
def test_rmsnorm_variants(ops, dt, dim, n):
    eps = 1e-5
    h = rnd(n, dim, seed=1)
    w = rnd(dim, seed=2) * 0.1 + 1.0
    ref = torch.from_numpy(P.rmsnorm(h.cpu().numpy(), w.cpu().numpy(), eps)).to(DEV)
    out = torch.empty(n, dim, dtype=dt, device=DEV)
    ops.rmsnorm(h, w, eps, out)
    torch.testing.assert_close(out.float(), ref, **tol(dt, 4))
    # fused residual sum: h += delta, then norm; also a stack of partial sums added in order
    for delta in (rnd(n, dim, seed=3), rnd(3, n, dim, seed=4)):
        h2 = h.clone()
        dsum = delta if delta.dim() == 2 else delta[0] + delta[1] + delta[2]
        ops.rmsnorm(h2, w, eps, out, delta=delta)
        torch.testing.assert_close(h2, h + dsum, atol=1e-6, rtol=1e-6)
        ref2 = torch.from_numpy(P.rmsnorm((h + dsum).cpu().numpy(), w.cpu().numpy(), eps)).to(DEV)
        torch.testing.assert_close(out.float(), ref2, **tol(dt, 4))
    # chosen rows only (the logits rows): h stays as it is
    rows = torch.tensor([6, 0, 6], dtype=torch.int32, device=DEV)
    h3, d3 = h.clone(), rnd(n, dim, seed=5)
    out3 = torch.empty(3, dim, dtype=dt, device=DEV)
    ops.rmsnorm(h3, w, eps, out3, delta=d3, rows=rows)
    assert torch.equal(h3, h)
    ref3 = torch.from_numpy(P.rmsnorm((h + d3)[rows.long()].cpu().numpy(), w.cpu().numpy(), eps)).to(DEV)
    torch.testing.assert_close(out3.float(), ref3, **tol(dt, 4))


@pytest.mark.parametrize("dt", DTYPES)
def test_silu_mul_and_residual_add(ops, dt):
    n, ff = 5, 1000
    gu = rnd(n, 2 * ff, dtype=dt, seed=6, std=2.0)
    out = torch.empty(n, ff, dtype=dt, device=DEV)
    ops.silu_mul(gu, out)
    g, u = gu[:, :ff].float().cpu().numpy(), gu[:, ff:].float().cpu().numpy()
    torch.testing.assert_close(out.float().cpu(), torch.from_numpy(P.silu(g) * u), **tol(dt, 4))
    h, d = rnd(n, 333, seed=7), rnd(2, n, 333, seed=8)
    want = h + d[0] + d[1]
    ops.residual_add(h, d)
    torch.testing.assert_close(h, want, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 130, 257), (65, 64, 64), (128, 509, 192), (200, 176, 1000), (9, 2048, 96)])
def test_gemm(ops, dt, M, N, K):
    a, w = rnd(M, K, dtype=dt, seed=9), rnd(N, K, dtype=dt, seed=10, std=0.1)
    ref = a.double() @ w.double().t()
    for out_dt in {dt, torch.float32}:
        out = torch.empty(M, N, dtype=out_dt, device=DEV)
        ops.gemm(a, w, out)
        t = tol(out_dt, math.sqrt(K) * 0.1)
        torch.testing.assert_close(out.double(), ref, **t)
    # strided rows (views into wider buffers), as the engine passes the q part of qkv
    wide_a = rnd(M, K + 13, dtype=dt, seed=11)
    wide_out = torch.zeros(M, N + 5, dtype=torch.float32, device=DEV)
    ops.gemm(wide_a[:, 3:3 + K], w, wide_out[:, 2:2 + N])
    torch.testing.assert_close(wide_out[:, 2:2 + N].double(), wide_a[:, 3:3 + K].double() @ w.double().t(),
                               **tol(torch.float32 if dt == torch.float32 else dt, math.sqrt(K) * 0.1))
    assert float(wide_out[:, :2].abs().max()) == 0 and float(wide_out[:, 2 + N:].abs().max()) == 0


@pytest.mark.parametrize("M", [1, 8, 17, 64, 65, 128, 300])
@pytest.mark.parametrize("N,K", [(16, 64), (130, 192), (509, 200), (3072, 2048), (176, 1024)])
def test_gemm_tensor_cores(ops, M, N, K):
    """The tcgen05/TMA kernel in both forms (few tokens: weights on the accumulator lanes, K cut in
    splits; many tokens: 128-token tiles), with tails in every dimension."""
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=50), rnd(N, K, dtype=torch.bfloat16, seed=51, std=0.1)
    assert ops._tc_usable(a, w)
    ref = a.double() @ w.double().t()
    scale = math.sqrt(K) * 0.1
    for out_dt in (torch.float32, torch.bfloat16):
        from llmengine.engine.context import Workspace
        for ws in (None, Workspace(torch.device(DEV))):  # with a workspace the product may be cut along K
            out = torch.full((M, N), float("nan"), dtype=out_dt, device=DEV)
            ops.gemm(a, w, out, ws)
            torch.testing.assert_close(out.double(), ref, **tol(out_dt, scale))
    parts = ops.gemm_partials(a, w, Workspace(torch.device(DEV)), "t")
    assert parts.dtype == torch.float32 and parts.shape[1:] == (M, N)
    if M <= 64 and N <= 3072 and K >= 256:
        assert parts.shape[0] > 1  # few tokens, few output tiles, long K: cut along K
    torch.testing.assert_close(parts.double().sum(0), ref, **tol(torch.float32, scale))
    red = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.reduce_partials(parts, red)
    torch.testing.assert_close(red.double(), ref, **tol(torch.bfloat16, scale))
    assert ops.tensor_core_error() == 0
    # operands the kernel cannot take (K not a multiple of 8) go to the CUDA-core kernel
    a2, w2 = rnd(M, 100, dtype=torch.bfloat16, seed=52)[:, :99], rnd(N, 99, dtype=torch.bfloat16, seed=53)
    assert not ops._tc_usable(a2, w2)


@pytest.mark.parametrize("M", [5, 64, 65, 300])
@pytest.mark.parametrize("FF,K", [(128, 64), (384, 192), (1024, 512)])
def test_gemm_with_fused_swiglu(ops, M, FF, K):
    """silu(gate) * up from the product's epilogue (many tokens) and from its partial sums (few)."""
    from llmengine.engine.context import Workspace
    a = rnd(M, K, dtype=torch.bfloat16, seed=60)
    g, u = rnd(FF, K, dtype=torch.bfloat16, seed=61, std=0.1), rnd(FF, K, dtype=torch.bfloat16, seed=62, std=0.1)
    blocked = torch.stack([g.view(-1, 128, K), u.view(-1, 128, K)], dim=1).reshape(2 * FF, K).contiguous()
    out = torch.full((M, FF), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_swiglu(a, blocked, out, Workspace(torch.device(DEV)))
    gf, uf = (a.float() @ g.float().t()).cpu().numpy(), (a.float() @ u.float().t()).cpu().numpy()
    ref = torch.from_numpy(P.silu(gf) * uf)
    torch.testing.assert_close(out.float().cpu(), ref, **tol(torch.bfloat16, math.sqrt(K) * 0.1))
    assert ops.tensor_core_error() == 0


@pytest.fixture
def one_cta_products(ops):
    """No CTA pairs during the test: it is about the kernels that give a tile to one CTA."""
    ops.use_cta_pairs(False)
    yield
    ops.use_cta_pairs(None)


@pytest.mark.parametrize("M,N,K", [(300, 25617, 192), (129, 76000, 64), (1100, 8704, 256), (2048, 3072, 128), (1500, 5120, 64),
                                   (2048, 3000, 64)])  # the last three: tiles of 192 outputs shorten the last round
def test_gemm_persistent_form(ops, one_cta_products, M, N, K):
    """Enough output tiles that every SM gets several: the persistent kernel (two accumulators in
    tensor memory, epilogue beside the next tile's products) against float64, tails in every
    dimension, and against the one-tile-per-CTA kernel bit for bit (same products in the same order)."""
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=70), rnd(N, K, dtype=torch.bfloat16, seed=71, std=0.1)
    lib = ops.lib("tensorcore")
    scale = math.sqrt(K) * 0.1
    outs = {}
    for out_dt in (torch.float32, torch.bfloat16):
        for persistent in (1, 0):
            lib.llm_gemm_tc_persistent(persistent)
            try:
                out = torch.full((M, N), float("nan"), dtype=out_dt, device=DEV)
                ops.gemm(a, w, out)
            finally:
                lib.llm_gemm_tc_persistent(1)
            outs[(out_dt, persistent)] = out
        assert torch.equal(outs[(out_dt, 1)], outs[(out_dt, 0)])
        rows = torch.tensor([0, 1, 127, 128, M - 1])
        ref = a[rows.to(DEV)].double() @ w.double().t()
        torch.testing.assert_close(outs[(out_dt, 1)][rows.to(DEV)].double(), ref, **tol(out_dt, scale))
    assert ops.tensor_core_error() == 0


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (300, 25617, 192), (1100, 8704, 256), (129, 512, 2048), (700, 1024, 4160)])
def test_gemm_on_cta_pairs(ops, M, N, K):
    """The cta_group::2 kernel (two CTAs of a cluster on one 256 x 256 tile, one MMA stream, each CTA
    loading half of the weight tile): same products in the same order as the one-CTA kernels, so the
    float32 results are equal bit for bit; tails in every dimension; an odd number of 128-row tiles."""
    from llmengine.engine.context import Workspace
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=75), rnd(N, K, dtype=torch.bfloat16, seed=76, std=0.1)
    outs = {}
    for out_dt in (torch.float32, torch.bfloat16):
        for pairs in (True, False):
            ops.use_cta_pairs(pairs)
            try:
                out = torch.full((M, N), float("nan"), dtype=out_dt, device=DEV)
                ops.gemm(a, w, out)
            finally:
                ops.use_cta_pairs(None)
            outs[(out_dt, pairs)] = out
        assert torch.equal(outs[(out_dt, True)], outs[(out_dt, False)])
    rows = torch.tensor([0, 127, 128, M - 1]).to(DEV)
    torch.testing.assert_close(outs[(torch.float32, True)][rows].double(), a[rows].double() @ w.double().t(),
                               **tol(torch.float32, math.sqrt(K) * 0.1))
    if N % 256 == 0:  # silu(gate) * up from the pair kernel's epilogue
        FF = N // 2
        acts = []
        for pairs in (True, False):
            ops.use_cta_pairs(pairs)
            try:
                act = torch.full((M, FF), float("nan"), dtype=torch.bfloat16, device=DEV)
                ops.gemm_swiglu(a, w, act, Workspace(torch.device(DEV)))
            finally:
                ops.use_cta_pairs(None)
            acts.append(act)
        assert torch.equal(acts[0], acts[1])
    assert ops.tensor_core_error() == 0


def test_gemm_persistent_form_with_swiglu(ops, one_cta_products):
    from llmengine.engine.context import Workspace
    M, FF, K = 300, 12800, 128
    a = rnd(M, K, dtype=torch.bfloat16, seed=72)
    g, u = rnd(FF, K, dtype=torch.bfloat16, seed=73, std=0.1), rnd(FF, K, dtype=torch.bfloat16, seed=74, std=0.1)
    blocked = torch.stack([g.view(-1, 128, K), u.view(-1, 128, K)], dim=1).reshape(2 * FF, K).contiguous()
    lib = ops.lib("tensorcore")
    outs = []
    for persistent in (1, 0):
        lib.llm_gemm_tc_persistent(persistent)
        try:
            out = torch.full((M, FF), float("nan"), dtype=torch.bfloat16, device=DEV)
            ops.gemm_swiglu(a, blocked, out, Workspace(torch.device(DEV)))
        finally:
            lib.llm_gemm_tc_persistent(1)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    gf, uf = (a.float() @ g.float().t()).cpu().numpy(), (a.float() @ u.float().t()).cpu().numpy()
    torch.testing.assert_close(outs[0].float().cpu(), torch.from_numpy(P.silu(gf) * uf), **tol(torch.bfloat16, math.sqrt(K) * 0.1))
    assert ops.tensor_core_error() == 0


def test_silu_mul_partials(ops):
    parts = rnd(3, 5, 2 * 176, seed=54)
    out = torch.empty(5, 176, dtype=torch.bfloat16, device=DEV)
    ops.silu_mul_partials(parts, out)
    s = parts.sum(0).cpu().numpy()
    torch.testing.assert_close(out.float().cpu(), torch.from_numpy(P.silu(s[:, :176]) * s[:, 176:]), **tol(torch.bfloat16, 4))


def test_gemm_float32_rows_do_not_depend_on_the_batch(ops):
    """A row's result is bit-identical whether it is computed alone or among others."""
    a, w = rnd(77, 300, seed=12), rnd(190, 300, seed=13)
    full = torch.empty(77, 190, device=DEV)
    ops.gemm(a, w, full)
    for r in (0, 40, 76):
        one = torch.empty(1, 190, device=DEV)
        ops.gemm(a[r:r + 1], w, one)
        assert torch.equal(one[0], full[r])


def _paged_setup(dt, nkv, hd, page, seq_lens, n_pages, seed=0):
    """Random K,V for each request, scattered into shuffled pages. -> caches, tables, dense K/V."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g).tolist()
    kc = torch.zeros(n_pages + 1, nkv, page, hd, dtype=dt, device=DEV)
    vc = torch.zeros_like(kc)
    max_blocks = max((L + page - 1) // page for L in seq_lens)
    table = torch.full((len(seq_lens), max_blocks), -1, dtype=torch.int32)
    dense = []
    for s, L in enumerate(seq_lens):
        K = (torch.randn(L, nkv, hd, generator=g)).to(dt)
        V = (torch.randn(L, nkv, hd, generator=g)).to(dt)
        dense.append((K, V))
        for b in range((L + page - 1) // page):
            pg = perm.pop()
            table[s, b] = pg
            n = min(page, L - b * page)
            kc[pg, :, :n] = K[b * page:b * page + n].transpose(0, 1).to(DEV)
            vc[pg, :, :n] = V[b * page:b * page + n].transpose(0, 1).to(DEV)
    return kc, vc, table.to(DEV), dense


def _attention_ref(q, K, V, pos, nq, nkv, hd, scale, window):
    lo = max(0, pos - window + 1) if window > 0 else 0
    K, V = K[lo:pos + 1].float(), V[lo:pos + 1].float()
    out = torch.empty(nq, hd)
    for h in range(nq):
        s = (K[:, h // (nq // nkv)] @ q[h].float()) * scale
        out[h] = torch.softmax(s, 0) @ V[:, h // (nq // nkv)]
    return out.reshape(-1)


class Batch:
    """The fields of a step context that the attention kernels read."""

    def __init__(self, seqs):
        """seqs: [(first position, number of tokens)] for batch rows 0, 1, ..."""
        from llmengine.engine.context import Workspace
        pos, tseq, qoff = [], [], [0]
        for i, (start, n) in enumerate(seqs):
            pos += list(range(start, start + n))
            tseq += [i] * n
            qoff.append(qoff[-1] + n)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        self.positions, self.token_seq, self.seq_qoff = i32(pos), i32(tseq), i32(qoff)
        self.seq_start, self.seq_ntok = i32([s for s, _ in seqs]), i32([n for _, n in seqs])
        self.n_tokens, self.n_seqs = len(pos), len(seqs)
        self.max_new_tokens = max(n for _, n in seqs)
        self.max_seq_len = max(s + n for s, n in seqs)
        self.ws = Workspace(torch.device(DEV))
        self.tokens = list(zip(tseq, pos))


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,page,window", [(8, 2, 64, 16, 0), (6, 1, 32, 4, 0), (5, 5, 48, 8, 0), (4, 2, 16, 4, 9),
                                                   (8, 4, 128, 16, 40), (2, 1, 256, 16, 0), (3, 3, 80, 64, 0), (32, 8, 64, 16, 0),
                                                   (12, 2, 64, 16, 100)])
def test_paged_attention(ops, dt, nq, nkv, hd, page, window):
    seq_lens = [1, 37, 130, 64, 700]
    kc, vc, table, dense = _paged_setup(dt, nkv, hd, page, seq_lens, sum((L + page - 1) // page for L in seq_lens) + 3)
    scale = 1.0 / math.sqrt(hd)
    batches = [
        # a prompt portion that starts in the middle of a page beside single decoded tokens
        Batch([(0, 1), (36, 1), (101, 29), (63, 1), (650, 50)]),
        # whole prompts from position 0, one longer than a tile of query tokens
        Batch([(0, 1), (0, 37), (0, 130), (0, 2), (0, 3)]),
        # decoding only: one token each (long contexts are cut into key splits on the tensor-core path)
        Batch([(0, 1), (36, 1), (129, 1), (15, 1), (699, 1)]),
    ]
    for b in batches:
        q = rnd(b.n_tokens, nq * hd, dtype=dt, seed=20)
        out = torch.full((b.n_tokens, nq * hd), float("nan"), dtype=dt, device=DEV)
        ops.paged_attention(q, kc, vc, b, table, out, nq, nkv, hd, scale, window)
        for i, (s, p) in enumerate(b.tokens):
            ref = _attention_ref(q[i].cpu().view(nq, hd), dense[s][0], dense[s][1], p, nq, nkv, hd, scale, window)
            torch.testing.assert_close(out[i].float().cpu(), ref, **tol(dt, 2))


@pytest.mark.parametrize("hd,page", [(64, 16), (128, 16), (128, 32), (64, 64)])
@pytest.mark.parametrize("nq,nkv,window", [(32, 8, 0), (8, 2, 0), (4, 4, 0), (16, 1, 0), (8, 2, 150), (6, 2, 0), (5, 1, 70)])
def test_paged_attention_tcgen05(ops, nq, nkv, window, hd, page):
    """The tcgen05 kernel for prompt portions (head sizes 64 and 128): portions that start in the
    middle of a page and of a key tile, span several tiles, stand beside single tokens."""
    dt = torch.bfloat16
    lib = ops.lib("tensorcore")
    from ctypes import c_int, c_longlong
    assert lib.llm_attention_tc_supported(c_int(nq), c_int(nkv), c_int(hd), c_int(page), c_longlong(nq * hd), c_longlong(nq * hd))
    seq_lens = [300, 1, 129, 700, 128]
    kc, vc, table, dense = _paged_setup(dt, nkv, hd, page, seq_lens, sum((L + page - 1) // page for L in seq_lens) + 3, seed=9)
    scale = 1.0 / math.sqrt(hd)
    from llmengine.ops import KernelError
    for b in (Batch([(0, 300), (0, 1), (0, 129), (0, 50), (0, 128)]), Batch([(251, 49), (0, 1), (100, 29), (310, 390), (127, 1)])):
        assert b.max_new_tokens >= ops.TC_ATTENTION_MIN_TOKENS
        q = rnd(b.n_tokens, nq * hd, dtype=dt, seed=23)
        out = torch.full((b.n_tokens, nq * hd), float("nan"), dtype=dt, device=DEV)
        ops.paged_attention(q, kc, vc, b, table, out, nq, nkv, hd, scale, window)
        assert ops.tensor_core_error() == 0
        rows = list(range(0, b.n_tokens, 7)) + [b.n_tokens - 1]
        for i in rows:
            s_, p_ = b.tokens[i]
            ref = _attention_ref(q[i].cpu().view(nq, hd), dense[s_][0], dense[s_][1], p_, nq, nkv, hd, scale, window)
            torch.testing.assert_close(out[i].float().cpu(), ref, **tol(dt, 2))
        assert not torch.isnan(out.float()).any()


@pytest.mark.parametrize("nq,nkv,hd,page,window", [(32, 8, 64, 16, 0), (24, 8, 128, 16, 0), (8, 2, 64, 32, 150), (6, 2, 128, 8, 0),
                                                   (5, 1, 64, 16, 70), (7, 1, 64, 64, 0), (16, 1, 128, 16, 0)])
def test_paged_attention_tcgen05_both_forms(ops, nq, nkv, hd, page, window):
    """The CTAs that stay and take query tiles from a counter (query rows by TMA, a box a head; tiles of
    a multiple of 8 tokens) against a CTA a query tile: the same sums in the same order for every
    (token, head), so equal bit for bit; many more query tiles than CTAs, requests that end inside a
    tile, portions that start in the middle of a context, groups that do not divide 128, and the same
    launch three times (the work counters must be left at zero)."""
    dt = torch.bfloat16
    lib = ops.lib("tensorcore")
    seq_lens = [1500, 1, 129, 700, 128, 40, 333, 2]
    kc, vc, table, dense = _paged_setup(dt, nkv, hd, page, seq_lens, sum((L + page - 1) // page for L in seq_lens) + 3, seed=31)
    scale = 1.0 / math.sqrt(hd)
    for b in (Batch([(0, 1500), (0, 1), (0, 129), (0, 700), (0, 128), (0, 40), (0, 333), (0, 2)]),
              Batch([(1200, 300), (0, 1), (100, 29), (310, 390), (127, 1), (7, 33), (300, 33), (1, 1)])):
        q = rnd(b.n_tokens, nq * hd, dtype=dt, seed=32)
        outs = []
        for form in (1, 1, 1, 0):
            lib.llm_attention_tc_persistent(form)
            try:
                out = torch.full((b.n_tokens, nq * hd), float("nan"), dtype=dt, device=DEV)
                ops.paged_attention(q, kc, vc, b, table, out, nq, nkv, hd, scale, window)
            finally:
                lib.llm_attention_tc_persistent(1)
            assert ops.tensor_core_error() == 0
            outs.append(out)
        assert not torch.isnan(outs[0].float()).any()
        for o in outs[1:]:
            assert torch.equal(outs[0], o)
        for i in list(range(0, b.n_tokens, 97)) + [b.n_tokens - 1]:
            s_, p_ = b.tokens[i]
            ref = _attention_ref(q[i].cpu().view(nq, hd), dense[s_][0], dense[s_][1], p_, nq, nkv, hd, scale, window)
            torch.testing.assert_close(outs[0][i].float().cpu(), ref, **tol(dt, 2))


@pytest.mark.parametrize("cluster_merge", [True, False])
@pytest.mark.parametrize("target_ctas", [1, 592, 100000])  # no split, the usual splits, a split every 64 keys
@pytest.mark.parametrize("nq,nkv,hd,page,window", [(32, 8, 64, 16, 0), (8, 2, 64, 8, 0), (4, 4, 64, 32, 0), (16, 1, 64, 64, 0),
                                                   (8, 2, 64, 16, 150), (8, 4, 128, 16, 0), (2, 2, 128, 32, 70), (6, 2, 128, 8, 0)])
def test_paged_attention_decode_by_tma(ops, monkeypatch, nq, nkv, hd, page, window, target_ctas, cluster_merge):
    """The decoding kernel that fetches keys and values by TMA (head sizes 64 and 128): contexts that
    end at a tile's, a page's and a split's edge, a window whose pages behind it were given back
    (their table entries are -1), requests of very different lengths in one batch, and every
    split policy, merged inside a cluster and through global memory; the same call twice, since
    the split counters must be left at zero."""
    dt = torch.bfloat16
    if not cluster_merge and target_ctas == 1:
        pytest.skip("nothing to merge without splits")
    monkeypatch.setattr(type(ops), "ATTENTION_TARGET_CTAS", target_ctas)
    if target_ctas > 1000:
        monkeypatch.setattr(type(ops), "ATTENTION_MIN_SPLIT_KEYS", 64)
    seq_lens = [1, 32, 33, 64, 257, 700, 1024, 16]
    kc, vc, table, dense = _paged_setup(dt, nkv, hd, page, seq_lens, sum((L + page - 1) // page for L in seq_lens) + 3, seed=5)
    if window:  # pages wholly behind the window are no longer the request's
        for s_, L in enumerate(seq_lens):
            for b_ in range(max(0, L - window) // page):
                kc[int(table[s_, b_])].fill_(float("nan"))  # whoever reads them shows
                vc[int(table[s_, b_])].fill_(float("nan"))
                table[s_, b_] = -1
    scale = 1.0 / math.sqrt(hd)
    b = Batch([(L - 1, 1) for L in seq_lens])
    q = rnd(b.n_tokens, nq * hd, dtype=dt, seed=24)
    ops.merge_splits_in_cluster(cluster_merge)
    try:
        for _ in range(2):
            out = torch.full((b.n_tokens, nq * hd), float("nan"), dtype=dt, device=DEV)
            ops.paged_attention(q, kc, vc, b, table, out, nq, nkv, hd, scale, window)
            assert ops.tensor_core_error() == 0
            for i, (s_, p_) in enumerate(b.tokens):
                ref = _attention_ref(q[i].cpu().view(nq, hd), dense[s_][0], dense[s_][1], p_, nq, nkv, hd, scale, window)
                torch.testing.assert_close(out[i].float().cpu(), ref, **tol(dt, 2))
    finally:
        ops.merge_splits_in_cluster(True)


@pytest.mark.parametrize("nq,nkv,hd,page,window,rotate", [(32, 8, 64, 16, 0, True), (8, 2, 64, 8, 100, True), (16, 1, 64, 32, 0, False),
                                                          (8, 4, 128, 16, 0, True), (2, 2, 128, 64, 90, True)])
@pytest.mark.parametrize("n_parts", [1, 11])
def test_decode_attention_with_rotation_and_cache_write_folded_in(ops, nq, nkv, hd, page, window, rotate, n_parts):
    """One kernel from the q|k|v partial sums against the two-kernel path (rotation + cache write,
    then attention) on the same inputs: the same sums in the same order, so the outputs and the
    caches are equal bit for bit. Positions at the first slot of a fresh page and at a split's edge."""
    dt = torch.bfloat16
    seq_lens = [1, 17, 64, 65, 321, 1025, 700]  # the token is the last of each
    n_pages = sum((L + page - 1) // page for L in seq_lens) + 3
    kc, vc, table, dense = _paged_setup(dt, nkv, hd, page, seq_lens, n_pages, seed=7)
    b = Batch([(L - 1, 1) for L in seq_lens])
    n, width = b.n_tokens, (nq + 2 * nkv) * hd
    parts = rnd(n_parts, n, width, dtype=torch.float32, seed=26) / math.sqrt(n_parts)
    max_pos = 1100
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(hd // 2, dtype=torch.float64) / (hd // 2)))[None]
    cos, sin = (ang.cos().float().to(DEV), ang.sin().float().to(DEV)) if rotate else (None, None)
    scale = 1.0 / math.sqrt(hd)
    # two kernels
    k1, v1 = kc.clone(), vc.clone()
    qkv = torch.empty(n, width, dtype=dt, device=DEV)
    ops.rope_kv_write(qkv, b.positions, b.token_seq, table, cos, sin, k1, v1, n, nq, nkv, hd, parts=parts)
    out1 = torch.empty(n, nq * hd, dtype=dt, device=DEV)
    ops.paged_attention(qkv[:, :nq * hd], k1, v1, b, table, out1, nq, nkv, hd, scale, window)
    # one kernel
    k2, v2 = kc.clone(), vc.clone()
    out2 = torch.full((n, nq * hd), float("nan"), dtype=dt, device=DEV)
    assert ops.decode_attention_fusable(b, k2, nq, nkv, hd, out2)
    ops.paged_attention_decode_fused(parts, cos, sin, k2, v2, b, table, out2, nq, nkv, hd, scale, window)
    assert ops.tensor_core_error() == 0
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    assert torch.equal(out1, out2)
    # and both are right: the new key/value count
    summed = parts.sum(0).cpu()
    for i, (s_, p_) in enumerate(b.tokens):
        K, V = dense[s_][0].clone(), dense[s_][1].clone()
        pg, off = int(table[s_, p_ // page]), p_ % page
        K[p_], V[p_] = k2[pg, :, off].cpu(), v2[pg, :, off].cpu()
        q = qkv[i, :nq * hd].cpu().view(nq, hd)
        ref = _attention_ref(q, K, V, p_, nq, nkv, hd, scale, window)
        torch.testing.assert_close(out2[i].float().cpu(), ref, **tol(dt, 2))
        torch.testing.assert_close(v2[pg, :, off].float().cpu().reshape(-1), summed[i, (nq + nkv) * hd:], atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("hd,n_req", [(64, 80), (128, 40), (64, 20), (128, 12)])
def test_decode_attention_many_requests(ops, hd, n_req):
    """Enough (request, kv head) pairs that the short ring is used (four CTAs an SM), and few enough
    for the long one; contexts of dozens of tiles, so that every stage of the ring is used many
    times over by different warps (the ring lengths 6, 5 and 3 are no multiples of the four warps)."""
    nq, nkv, page, dt = 16, 8, 16, torch.bfloat16
    g = torch.Generator().manual_seed(hd + n_req)
    seq_lens = torch.randint(900, 1600, (n_req,), generator=g).tolist()
    kc, vc, table, dense = _paged_setup(dt, nkv, hd, page, seq_lens, sum((L + page - 1) // page for L in seq_lens) + 3, seed=8)
    b = Batch([(L - 1, 1) for L in seq_lens])
    q = rnd(b.n_tokens, nq * hd, dtype=dt, seed=27)
    scale = 1.0 / math.sqrt(hd)
    outs = []
    for _ in range(3):  # timing differs from launch to launch; the result must not
        out = torch.full((b.n_tokens, nq * hd), float("nan"), dtype=dt, device=DEV)
        ops.paged_attention(q, kc, vc, b, table, out, nq, nkv, hd, scale)
        outs.append(out)
    assert ops.tensor_core_error() == 0
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    for i in list(range(0, n_req, max(1, n_req // 6))) + [n_req - 1]:
        s_, p_ = b.tokens[i]
        ref = _attention_ref(q[i].cpu().view(nq, hd), dense[s_][0], dense[s_][1], p_, nq, nkv, hd, scale, 0)
        torch.testing.assert_close(outs[0][i].float().cpu(), ref, **tol(dt, 2))


def test_decode_attention_kernels_agree(ops):
    """The TMA decoding kernel against the general mma.sync kernel (cp.async, tiles of 64 keys, a
    second kernel merging the splits) on the same inputs: equal up to the order of float32 sums."""
    nq, nkv, hd, page = 32, 8, 64, 16
    seq_lens = [2048, 100, 777, 1500]
    kc, vc, table, dense = _paged_setup(torch.bfloat16, nkv, hd, page, seq_lens, sum((L + page - 1) // page for L in seq_lens) + 3, seed=6)
    b = Batch([(L - 1, 1) for L in seq_lens])
    q = rnd(b.n_tokens, nq * hd, dtype=torch.bfloat16, seed=25)
    outs = []
    for tma in (True, False):
        ops.tma_decode_attention = tma
        try:
            out = torch.empty(b.n_tokens, nq * hd, dtype=torch.bfloat16, device=DEV)
            ops.paged_attention(q, kc, vc, b, table, out, nq, nkv, hd, 0.125)
            outs.append(out.float())
        finally:
            ops.tma_decode_attention = True
    assert ops.tensor_core_error() == 0
    torch.testing.assert_close(outs[0], outs[1], atol=2e-3, rtol=2e-2)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("special", [0, 15, 16, 31, 32, 63, 64, 127, 128, 255, 256, 499])
@pytest.mark.parametrize("n_new", [1, 3, 40])
def test_attention_finds_one_far_key_among_hundreds(ops, dt, special, n_new):
    """Random values hide a skipped key (its weight is ~1/500). Here one key is made to match the
    query, so that the output must be that key's value: a key lost at a page's edge, at a tile's or
    a split's edge, at the start or at the end of the range shows as an error of order one."""
    nq, nkv, hd, page, L = 4, 2, 64, 16, 500
    kc, vc, table, dense = _paged_setup(dt, nkv, hd, page, [L], 40, seed=special)
    b = Batch([(L - n_new, n_new)])
    q = rnd(n_new, nq * hd, dtype=dt, seed=21)
    K, V = dense[0]
    pg, off = int(table[0, special // page]), special % page
    for h in range(nkv):  # both kv heads: key `special` := 4 * (a query of that group), others stay random
        K[special, h] = (q[n_new - 1].cpu().view(nq, hd)[h * 2].float() * 4).to(dt)
        kc[pg, h, off] = K[special, h].to(DEV)
    out = torch.empty(n_new, nq * hd, dtype=dt, device=DEV)
    ops.paged_attention(q, kc, vc, b, table, out, nq, nkv, hd, 1.0, 0)
    for i in range(n_new):
        ref = _attention_ref(q[i].cpu().view(nq, hd), K, V, L - n_new + i, nq, nkv, hd, 1.0, 0)
        torch.testing.assert_close(out[i].float().cpu(), ref, **tol(dt, 2))
    if special <= L - n_new:
        o = out[n_new - 1].float().cpu().view(nq, hd)
        for h in (0, 2):  # the matching heads return (almost exactly) the special key's value
            assert (o[h] - V[special, h // 2].float()).abs().max() < 0.05


@pytest.mark.parametrize("nq,nkv,hd", [(32, 8, 64), (24, 8, 128)])
@pytest.mark.parametrize("special", [0, 63, 64, 340, 341, 342, 1023, 1024, 2040])
@pytest.mark.parametrize("n_new", [1, 40])
def test_attention_finds_one_far_key_at_real_head_counts(ops, nq, nkv, hd, special, n_new):
    """The same at the head counts and context lengths of real checkpoints (Llama 3.2 1B and 3B: 32
    and 24 query heads over 8 key/value heads of 64 and 128, 2,048 keys, bfloat16): single tokens go
    through the TMA decoding kernel with its key splits merged inside a cluster, portions of 40
    through the tcgen05 kernel; the special key sits at the start, at tile and split edges and near
    the end. Among 2,048 random keys a lost one would weigh 1/2048 and pass any tolerance."""
    dt, page, L = torch.bfloat16, 16, 2048
    g = nq // nkv
    kc, vc, table, dense = _paged_setup(dt, nkv, hd, page, [L], L // page + 3, seed=special)
    b = Batch([(L - n_new, n_new)])
    q = rnd(n_new, nq * hd, dtype=dt, seed=27)
    K, V = dense[0]
    pg, off = int(table[0, special // page]), special % page
    qs = q[n_new - 1].cpu().view(nq, hd).float()
    for h in range(nkv):  # key `special` of every kv head: along the first query of its group, with a score of 16
        K[special, h] = (qs[h * g] * (16.0 * math.sqrt(hd) / float((qs[h * g] ** 2).sum()))).to(dt)
        kc[pg, h, off] = K[special, h].to(DEV)
    out = torch.full((n_new, nq * hd), float("nan"), dtype=dt, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ops.paged_attention(q, kc, vc, b, table, out, nq, nkv, hd, scale, 0)
    assert ops.tensor_core_error() == 0
    for i in (0, n_new - 1):
        ref = _attention_ref(q[i].cpu().view(nq, hd), K, V, L - n_new + i, nq, nkv, hd, scale, 0)
        torch.testing.assert_close(out[i].float().cpu(), ref, **tol(dt, 2))
    o = out[n_new - 1].float().cpu().view(nq, hd)
    for h in range(nkv):  # a score of 16 against 2,047 of ~N(0, 1): that key carries the row
        assert (o[h * g] - V[special, h].float()).abs().max() < 0.05


@pytest.mark.parametrize("dt", DTYPES)
def test_attention_window_edge(ops, dt):
    """The key just outside the window must not count, the one just inside must."""
    nq, nkv, hd, page, L, W = 2, 1, 32, 8, 100, 24
    for special, inside in ((L - W, True), (L - W - 1, False)):
        kc, vc, table, dense = _paged_setup(dt, nkv, hd, page, [L], 20, seed=3)
        q = rnd(1, nq * hd, dtype=dt, seed=22)
        K, V = dense[0]
        K[special, 0] = (q[0].cpu().view(nq, hd)[0].float() * 4).to(dt)
        kc[int(table[0, special // page]), 0, special % page] = K[special, 0].to(DEV)
        out = torch.empty(1, nq * hd, dtype=dt, device=DEV)
        ops.paged_attention(q, kc, vc, Batch([(L - 1, 1)]), table, out, nq, nkv, hd, 1.0, W)
        ref = _attention_ref(q[0].cpu().view(nq, hd), K, V, L - 1, nq, nkv, hd, 1.0, W)
        torch.testing.assert_close(out[0].float().cpu(), ref, **tol(dt, 2))
        hit = (out[0].float().cpu()[:hd] - V[special, 0].float()).abs().max() < 0.05
        assert bool(hit) == inside


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,page", [(4, 2, 16, 4), (6, 1, 32, 16), (3, 3, 80, 8)])
def test_rope_and_cache_write(ops, dt, nq, nkv, hd, page):
    inv = P.llama3_inv_freq(hd, 500000.0, True, 8.0, 1.0, 4.0, 64)
    cos, sin = P.rope_tables(inv, 300, hd)
    cos_d = torch.from_numpy(cos[:, :hd // 2].copy()).to(DEV)
    sin_d = torch.from_numpy(sin[:, :hd // 2].copy()).to(DEV)
    toks = [(0, 0), (0, 1), (1, 163), (1, 150), (2, 17)]
    n = len(toks)
    qkv = rnd(n, (nq + 2 * nkv) * hd, dtype=dt, seed=30)
    orig = qkv.clone()
    table = torch.tensor([[3, 1] + [-1] * 40, [(5 + i) for i in range(42)], [50, 51, 52, 53, 54] + [-1] * 37], dtype=torch.int32, device=DEV)
    kc = torch.zeros(60, nkv, page, hd, dtype=dt, device=DEV)
    vc = torch.zeros_like(kc)
    positions = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    token_seq = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    ops.rope_kv_write(qkv, positions, token_seq, table, cos_d, sin_d, kc, vc, n, nq, nkv, hd)
    o = orig.float().cpu().numpy()
    pos = positions.cpu().numpy()
    q_ref = P.apply_rope(o[:, :nq * hd].reshape(n, nq, hd), cos[pos], sin[pos])
    k_ref = P.apply_rope(o[:, nq * hd:(nq + nkv) * hd].reshape(n, nkv, hd), cos[pos], sin[pos])
    v_ref = o[:, (nq + nkv) * hd:].reshape(n, nkv, hd)
    torch.testing.assert_close(qkv[:, :nq * hd].float().cpu(), torch.from_numpy(q_ref.reshape(n, -1)), **tol(dt, 4))
    written = torch.zeros(60, page, dtype=torch.bool)
    for i, (s, p) in enumerate(toks):
        pg = int(table[s, p // page])
        written[pg, p % page] = True
        torch.testing.assert_close(kc[pg, :, p % page].float().cpu(), torch.from_numpy(k_ref[i]), **tol(dt, 4))
        assert torch.equal(vc[pg, :, p % page].float().cpu(), torch.from_numpy(v_ref[i]))
    # nothing else was touched
    assert float(kc.float().abs().sum(dim=(1, 3)).cpu()[~written].sum()) == 0
    # the same from K-split partial sums: three float32 parts that add up to the q|k|v rows
    of = orig.float()
    p1, p2 = rnd(n, of.shape[1], seed=31), rnd(n, of.shape[1], seed=32)
    parts = torch.stack([p1, p2, of - p1 - p2]).contiguous()
    summed = (parts[0] + parts[1] + parts[2])
    qkv3 = torch.zeros_like(orig)
    kc3, vc3 = torch.zeros_like(kc), torch.zeros_like(vc)
    ops.rope_kv_write(qkv3, positions, token_seq, table, cos_d, sin_d, kc3, vc3, n, nq, nkv, hd, parts=parts)
    s3 = summed.cpu().numpy()
    q3 = P.apply_rope(s3[:, :nq * hd].reshape(n, nq, hd), cos[pos], sin[pos])
    k3 = P.apply_rope(s3[:, nq * hd:(nq + nkv) * hd].reshape(n, nkv, hd), cos[pos], sin[pos])
    torch.testing.assert_close(qkv3[:, :nq * hd].float().cpu(), torch.from_numpy(q3.reshape(n, -1)), **tol(dt, 4))
    for i, (s_, p_) in enumerate(toks):
        pg = int(table[s_, p_ // page])
        torch.testing.assert_close(kc3[pg, :, p_ % page].float().cpu(), torch.from_numpy(k3[i]), **tol(dt, 4))
        torch.testing.assert_close(vc3[pg, :, p_ % page].float().cpu(), torch.from_numpy(s3[i, (nq + nkv) * hd:].reshape(nkv, hd)), **tol(dt, 4))
    # no tables: q, k stay as they are, k and v are only stored
    qkv2 = orig.clone()
    ops.rope_kv_write(qkv2, positions, token_seq, table, None, None, kc, vc, n, nq, nkv, hd)
    assert torch.equal(qkv2[:, :nq * hd], orig[:, :nq * hd])
    assert torch.equal(kc[int(table[1, 163 // page]), :, 163 % page].reshape(-1), orig[2, nq * hd:(nq + nkv) * hd])


def test_sampling_greedy_and_temperature(ops):
    V = 5003
    logits = rnd(6, V, seed=40)
    logits[0, 100] = logits[0, 4000] = 50.0  # tie: the first index wins
    logits[1, V - 1] = 60.0
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    ops.sample(logits, out)
    assert out.tolist() == [100, V - 1] + logits[2:].argmax(-1).tolist()
    temps = torch.tensor([0.0, 1.0, 0.7, 1.5, 1.0, 1.0], device=DEV)
    seeds = torch.tensor([1, 2, 3, 4, 5, 5], dtype=torch.int32, device=DEV)
    draws = torch.tensor([0, 0, 7, 3, 1, 2], dtype=torch.int32, device=DEV)
    ops.sample(logits, out, temps, seeds, draws)
    host = logits.cpu().numpy()
    want = [P.sample_token(host[r], float(temps[r]), int(seeds[r]), int(draws[r])) for r in range(6)]
    assert out.tolist() == want and out[4] != out[5] or want[4] == want[5]
    # a draw follows softmax(logits / T)
    small = torch.tensor([[0.0, 1.0, 2.0, -1.0]], device=DEV).repeat(4000, 1).contiguous()
    o = torch.empty(4000, dtype=torch.int32, device=DEV)
    ops.sample(small, o, torch.ones(4000, device=DEV), torch.full((4000,), 77, dtype=torch.int32, device=DEV),
               torch.arange(4000, dtype=torch.int32, device=DEV))
    freq = torch.bincount(o.long(), minlength=4).float().cpu() / 4000
    assert (freq - torch.softmax(small[0].cpu(), 0)).abs().max() < 0.03


def test_kernels_refuse_what_they_cannot_take(ops):
    from llmengine.ops import KernelError
    with pytest.raises(KernelError, match="head_dim"):
        ops.paged_attention(rnd(1, 2 * 512), torch.zeros(2, 1, 4, 512, device=DEV), torch.zeros(2, 1, 4, 512, device=DEV),
                            Batch([(0, 1)]), torch.zeros(1, 1, dtype=torch.int32, device=DEV), torch.empty(1, 1024, device=DEV),
                            2, 1, 512, 1.0)
    with pytest.raises(KernelError, match="CUDA tensor"):
        ops.gemm(torch.zeros(2, 2), torch.zeros(2, 2), torch.zeros(2, 2))
    with pytest.raises(KernelError):
        ops.gemm(rnd(2, 2).half(), rnd(2, 2).half(), torch.empty(2, 2, device=DEV))
