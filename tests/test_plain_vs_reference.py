"""The plain implementation against outputs of the reference's own compiled model code
(tests/golden/*.npz, made by tests/golden/make_golden.py on the CPU)."""
import os
import tempfile

import numpy as np
import pytest

import make_golden as G
import plain_llama as P

GOLDEN_DIR = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", ["a", "b"])
def test_plain_matches_reference_outputs(name):
    cfg = G.GOLDEN_CONFIGS[name]
    g = np.load(os.path.join(GOLDEN_DIR, f"golden_{name}.npz"))
    with tempfile.TemporaryDirectory() as d:
        G.write_model_dir(d, cfg, G.golden_weights(cfg))
        pc, pw = P.read_model(d)
    for n in G.GOLDEN_SEQ_LENS[name]:
        ids = [int(t) for t in g[f"ids_{n}"]]
        assert ids == G.golden_ids(name, n, cfg["vocab_size"])
        logits = P.forward_logits(pc, pw, ids)
        np.testing.assert_allclose(logits, g[f"logits_{n}"], atol=1e-5, rtol=1e-5)
        assert (logits.argmax(-1) == g[f"logits_{n}"].argmax(-1)).all()
        out, reason = P.generate(pc, pw, ids, 6)
        assert out == [int(t) for t in g[f"gen_{n}"]]
        assert reason == str(g[f"reason_{n}"][0])


def test_plain_matches_the_references_kernels_beyond_its_engines_position_cap():
    """Configuration b at 150 and 255 tokens: the reference's engine stops at 64 positions there, so
    the golden logits are its exported kernels composed in the order of its layer loop
    (make_golden.compose_reference_kernels). They pin the scaled rotation table and the attention
    over long key ranges on both sides of position 64."""
    cfg = G.GOLDEN_CONFIGS["b"]
    g = np.load(os.path.join(GOLDEN_DIR, "golden_b_long.npz"))
    with tempfile.TemporaryDirectory() as d:
        G.write_model_dir(d, cfg, G.golden_weights(cfg))
        pc, pw = P.read_model(d)
    for n in G.LONG_LENS:
        ids = [int(t) for t in g[f"ids_{n}"]]
        rows = [int(r) for r in g[f"rows_{n}"]]
        assert ids == G.golden_ids("b", n, cfg["vocab_size"]) and rows == G.LONG_ROWS[n] and max(rows) > 64
        logits = P.logits_at(pc, pw, P.final_hidden(pc, pw, ids), rows)
        np.testing.assert_allclose(logits, g[f"logits_{n}"], atol=2e-5, rtol=2e-5)
        assert (logits.argmax(-1) == g[f"logits_{n}"].argmax(-1)).all()


def test_scheduler_streams_are_the_references():
    """Token streams and finish reasons of the reference's ContinuousBatchScheduler (recorded by
    make_golden.reference_scheduler_streams) against this engine's scheduler above the step function
    (kernels: the CPU test double): budget 4 with max_new_tokens 0, 1, 2 and 5, a request that ends at
    an end-of-sequence id, and the reference's own capacity case, where the request that cannot get a
    page ends with "capacity" and keeps what it generated."""
    import json

    import torch

    import llmengine
    from cpu_ops import CpuOps
    with open(os.path.join(GOLDEN_DIR, "golden_scheduler.json")) as f:
        cases = json.load(f)
    assert {"a_budget4", "b_budget4", "a_capacity", "a_stop"} <= set(cases)
    assert "stop" in cases["a_stop"]["finish"] and cases["a_capacity"]["finish"] == ["capacity", "length"]
    for name, c in cases.items():
        cfg = G.GOLDEN_CONFIGS[c["config"]]
        with tempfile.TemporaryDirectory() as d:
            G.write_model_dir(d, cfg, G.golden_weights(cfg))
            eng = llmengine.Engine(d, "fp32", device="cpu", ops=CpuOps(), block_size=c["page_size"])
            bm = llmengine.BlockManager(c["pages"], c["page_size"])
            sch = llmengine.ContinuousBatchScheduler(eng, bm, max_concurrent=c["max_concurrent"],
                                                     max_prefill_tokens_per_step=c["budget"])
            for n, k in zip(c["prompt_lens"], c["max_new"]):
                sch.enqueue(G.golden_ids(c["config"], n, cfg["vocab_size"]), k)
            sch.run_until_idle()
            got = sch.results
            assert [r.finish_reason for r in got] == c["finish"], name
            assert [list(r.token_ids) for r in got] == c["token_ids"], name
            assert bm.free_blocks == c["free_after"] == c["pages"], name
