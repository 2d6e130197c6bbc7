"""Trace replay through bin/trace_run (a subprocess, as a user runs it) against the plain
implementation: each request alone and whole; most of it in one step and the last 32 tokens one by
one; in portions of changing size down to two tokens; mixed, up to four live requests with so few
pages that they are used again. In true 32-bit and in bfloat16, for both tiny configurations."""
import numpy as np
import pytest
import torch

import plain_llama as P
from tiny import (MIXED_SIZES, MIXED_SIZES_LONG, TINY, make_model_dir, random_ids, round64, run_trace, trace_mixed,
                  trace_portions, trace_tail, trace_whole, Trace)

pytestmark = pytest.mark.gpu

LENS = {"a": [5, 64, 33, 97, 128], "b": [2, 23, 64, 150, 255, 201],  # short ones first: four are live at once
        "c": [3, 40, 64, 130, 299], "d": [7, 50, 64, 200, 511, 300], "e": [4, 33, 60, 399, 260]}
# float32: the engine's own arithmetic is float32 throughout; the plain implementation differs by
# summation order only. bfloat16: weights are the same bf16 values on both sides; the difference is
# the rounding of activations to bf16 between kernels.
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


@pytest.fixture(scope="module", params=[(n, d) for n in ("a", "b", "c", "d", "e") for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def replayed(request, tmp_path_factory):
    name, dtype = request.param
    cfg, page = TINY[name]
    d = str(tmp_path_factory.mktemp(f"model_{name}_{dtype}"))
    make_model_dir(d, cfg, torch.float32 if dtype == "float32" else torch.bfloat16)
    pc, pw = P.read_model(d)
    reqs = {f"r{i}": random_ids(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(LENS[name])}
    plain = {k: P.forward_logits(pc, pw, ids) for k, ids in reqs.items()}
    # one process replays the four cuts one after another; request names are made distinct per cut
    cuts = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}
    full, spans = Trace(), {}
    for cut, fn in cuts.items():
        t = fn({f"{cut}.{k}": v for k, v in reqs.items()})
        spans[cut] = (len(full.steps), len(full.steps) + len(t.steps))
        full.extend(t)
    longest = max(round64(len(v)) for v in reqs.values())
    max_tokens = longest + 3 * 64  # room for the longest request and three short ones: pages are reused
    # (configuration a holds 128 positions: its prompts are too short for the long portions)
    t = trace_mixed({f"mixed.{k}": v for k, v in reqs.items()}, max_tokens, seed=5,
                    sizes=MIXED_SIZES if name == "a" else MIXED_SIZES_LONG)
    spans["mixed"] = (len(full.steps), len(full.steps) + len(t.steps))
    full.extend(t)
    out = str(tmp_path_factory.mktemp(f"out_{name}_{dtype}"))
    rows = run_trace(d, dtype, full, out, max_tokens, page, cfg["vocab_size"])
    return dtype, reqs, plain, rows, t, name


@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_cut_matches_plain(replayed, cut):
    dtype, reqs, plain, rows, *_ = replayed
    worst = (0.0, None)
    for k, ids in reqs.items():
        for p in range(len(ids)):
            row = rows[(f"{cut}.{k}", p)]
            err = float(np.abs(row - plain[k][p]).max())
            if err > worst[0]:
                worst = (err, (k, p))
    assert worst[0] < TOL[dtype], f"{cut}: first look at request/position {worst[1]} (max error {worst[0]:.3e})"


def test_cuts_agree_with_one_another(replayed):
    """The logits at a position do not depend on how the tokens were cut into steps, on what else
    was in the batch, or on which pages were used, beyond rounding."""
    dtype, reqs, plain, rows, *_ = replayed
    tol = 2e-5 if dtype == "float32" else 3e-2
    for k, ids in reqs.items():
        for p in range(len(ids)):
            base = rows[(f"whole.{k}", p)]
            for cut in ("tail", "portions", "mixed"):
                err = float(np.abs(rows[(f"{cut}.{k}", p)] - base).max())
                assert err < tol, f"{cut} vs whole differ at request {k} position {p}: {err:.3e}"


def test_mixed_trace_is_really_mixed(replayed):
    """The trace used above has steps with four live requests, prompt portions beside single tokens."""
    *_, t, name = replayed
    assert max(len(s["entries"]) for s in t.steps) == 4
    assert any(len({len(e["tokens"]) == 1 for e in s["entries"]}) == 2 for s in t.steps)
    assert any(len(e["tokens"]) == 2 for s in t.steps for e in s["entries"])
    if name != "a":  # a portion of 32 tokens or more beside single tokens: what a scheduler's mixed steps look like
        assert any(max(len(e["tokens"]) for e in s["entries"]) >= 32 and min(len(e["tokens"]) for e in s["entries"]) == 1
                   for s in t.steps)


def test_requests_that_start_after_others_ended_are_new_requests(tmp_path):
    """Three live requests, the first ends, a fourth starts beside the two that go on, and the first
    one's NAME comes back for other tokens: nobody continues anybody else's cache."""
    cfg, page = TINY["a"]
    d = str(tmp_path / "m")
    make_model_dir(d, cfg, torch.float32)
    pc, pw = P.read_model(d)
    V = cfg["vocab_size"]
    ids = {k: random_ids(n, V, 300 + i) for i, (k, n) in enumerate([("a", 9), ("b", 14), ("c", 12), ("d", 10), ("a2", 7)])}
    plain = {k: P.forward_logits(pc, pw, v) for k, v in ids.items()}
    t = Trace()
    t.add([("a", ids["a"][:5], range(5), 0), ("b", ids["b"][:6], range(6), 0), ("c", ids["c"][:4], range(4), 0)])
    t.add([("a", ids["a"][5:], range(4), 5), ("b", ids["b"][6:8], range(2), 6)], end=["a"])
    t.add([("d", ids["d"][:7], range(7), 0), ("c", ids["c"][4:], range(8), 4), ("b", ids["b"][8:], range(6), 8)], end=["c"])
    t.add([("a", ids["a2"], range(7), 0), ("d", ids["d"][7:], range(3), 7)], end=["a", "b", "d"])  # "a" again: a new request
    t.rows = {}  # read the files by step below: the name "a" stands for two requests
    run_trace(d, "float32", t, str(tmp_path / "out"), 4 * 64, page, V)
    import os
    def step_rows(k):
        return np.fromfile(os.path.join(str(tmp_path / "out"), f"{k}.f32"), dtype="<f4").reshape(-1, V)
    s0, s1, s2, s3 = (step_rows(k) for k in range(4))
    np.testing.assert_allclose(np.concatenate([s0[:5], s1[:4]]), plain["a"], atol=2e-4, rtol=0)
    np.testing.assert_allclose(np.concatenate([s0[5:11], s1[4:6], s2[15:21]]), plain["b"], atol=2e-4, rtol=0)
    np.testing.assert_allclose(np.concatenate([s0[11:15], s2[7:15]]), plain["c"], atol=2e-4, rtol=0)
    np.testing.assert_allclose(np.concatenate([s2[:7], s3[7:10]]), plain["d"], atol=2e-4, rtol=0)
    np.testing.assert_allclose(s3[:7], plain["a2"], atol=2e-4, rtol=0)


@pytest.mark.parametrize("name,dtype,seed", [("a", "float32", 1), ("d", "bfloat16", 2), ("b", "float32", 3), ("d", "float32", 4)])
def test_random_mixed_traces(tmp_path, name, dtype, seed):
    """Other lengths, orders and cuts than the fixture's: ten requests of random length through a
    pool that holds about three of them, so that every page is used several times over."""
    cfg, page = TINY[name]
    d = str(tmp_path / "m")
    make_model_dir(d, cfg, torch.float32 if dtype == "float32" else torch.bfloat16, seed=20 + seed)
    pc, pw = P.read_model(d)
    rng = np.random.default_rng(seed)
    top = min(cfg["max_position_embeddings"], 200)
    lens = [int(n) for n in rng.integers(2, top, 10)]
    reqs = {f"q{i}": random_ids(n, cfg["vocab_size"], 500 + 10 * seed + i) for i, n in enumerate(lens)}
    max_tokens = round64(max(lens)) + 2 * 64
    t = trace_mixed(reqs, max_tokens, seed=seed)
    rows = run_trace(d, dtype, t, str(tmp_path / "out"), max_tokens, page, cfg["vocab_size"])
    assert len(rows) == sum(lens)
    for k, ids in reqs.items():
        ref = P.forward_logits(pc, pw, ids)
        got = np.stack([rows[(k, p)] for p in range(len(ids))])
        np.testing.assert_allclose(got, ref, atol=TOL[dtype], rtol=0, err_msg=f"request {k} of {len(ids)} tokens")
