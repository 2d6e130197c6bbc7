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
