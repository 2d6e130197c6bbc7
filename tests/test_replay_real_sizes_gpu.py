"""The four ways of cutting the work, in true 32-bit, at the layer sizes of Llama 3.2 1B (two
layers): each request whole; most of it in one step and the last 32 tokens one by one; in portions
of changing size; mixed with other requests through a pool so small that pages are used again.
Replayed by bin/trace_run as a user runs it and compared with the plain implementation at a subset
of the positions (the head over 128,256 entries is the slow part of the plain side), and with one
another. The same in bfloat16, where the mixed steps run the tensor-core kernels at these sizes."""
import numpy as np
import pytest
import torch

import llmengine
import plain_llama as P
from tiny import (MIXED_SIZES_LONG, Trace, random_ids, round64, run_trace, trace_mixed, trace_portions, trace_tail,
                  trace_whole)

pytestmark = pytest.mark.gpu

SIZES = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=8192, num_hidden_layers=2,
             num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=128256,
             max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=True,
             rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                               original_max_position_embeddings=8192))
LENS = [40, 150, 64, 250, 201]
PAGE = 16


def wanted_positions(n: int):
    """The first and last tokens, the edges of pages and of the tail, and every 23rd position."""
    keep = {0, 1, n - 1, n - 2, max(n - 33, 0), max(n - 32, 0)} | set(range(0, n, 23))
    keep |= {p for p in (15, 16, 17, 63, 64, 65, 127, 128, 129) if p < n}
    return {p for p in keep if 0 <= p < n}


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("sizes_1b"))
    llmengine.write_random_model(d, SIZES, seed=9, dtype=torch.bfloat16, std=0.02)
    pc, pw = P.read_model(d)
    reqs = {f"r{i}": random_ids(n, SIZES["vocab_size"], 200 + i) for i, n in enumerate(LENS)}
    plain = {}
    for k, ids in reqs.items():
        rows = sorted(wanted_positions(len(ids)))
        plain[k] = dict(zip(rows, P.logits_at(pc, pw, P.final_hidden(pc, pw, ids), rows)))
    return d, reqs, plain


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_four_cuts_at_real_layer_sizes(model, tmp_path, dtype):
    d, reqs, plain = model
    full, cuts = Trace(), {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}
    for cut, fn in cuts.items():
        full.extend(fn({f"{cut}.{k}": v for k, v in reqs.items()}))
    max_tokens = round64(max(LENS)) + 3 * 64
    mixed = trace_mixed({f"mixed.{k}": v for k, v in reqs.items()}, max_tokens, seed=3, sizes=MIXED_SIZES_LONG)
    assert any(max(len(e["tokens"]) for e in s["entries"]) >= 32 and min(len(e["tokens"]) for e in s["entries"]) == 1
               for s in mixed.steps)
    full.extend(mixed)
    full.keep_only(lambda name: wanted_positions(len(reqs[name.split(".", 1)[1]])))
    rows = run_trace(d, dtype, full, str(tmp_path / "out"), max_tokens, PAGE, SIZES["vocab_size"])
    # 32-bit: the plain implementation differs by the order of sums only. bfloat16: rounding of
    # activations between kernels; at these sizes its largest of a few million samples is about 0.06
    tol, tol_cuts = (2e-4, 2e-5) if dtype == "float32" else (1e-1, 6e-2)
    for k, ids in reqs.items():
        for p in sorted(wanted_positions(len(ids))):
            for cut in ("whole", "tail", "portions", "mixed"):
                err = float(np.abs(rows[(f"{cut}.{k}", p)] - plain[k][p]).max())
                assert err < tol, f"{cut}: request {k} position {p}: {err:.3e} from the plain implementation"
                if cut != "whole":
                    err = float(np.abs(rows[(f"{cut}.{k}", p)] - rows[(f"whole.{k}", p)]).max())
                    assert err < tol_cuts, f"{cut} vs whole: request {k} position {p}: {err:.3e}"
            if dtype == "float32":  # (among 128,256 bfloat16 logits the two largest may be a rounding step apart)
                assert int(np.argmax(rows[(f"whole.{k}", p)])) == int(np.argmax(plain[k][p]))
