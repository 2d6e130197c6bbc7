"""Decode-only steps replay CUDA graphs over a padded batch (null request, null page, block tables
rounded up to whole buckets of pages, key splits chosen for the widest table the graph may meet).
The other tests see that path through the chosen tokens only; here its LOGITS are compared with the
plain implementation, at capacities 1, 2 and 8 (with and without padded rows), with ragged context
lengths, across a bucket edge of the block table and up to the model's position limit."""
import numpy as np
import pytest
import torch

import llmengine
import plain_llama as P
from llmengine.cache import host_module
from tiny import TINY, TINY_D, make_model_dir, random_ids

pytestmark = pytest.mark.gpu
TOL = {"fp32": 2e-4, "bf16": 6e-2}
# f: the position limit (500) is no multiple of 16 pages of 16 positions: the widest table of a graph
# reaches beyond the rotation tables' last row
CONFIGS = dict(TINY, f=(dict(TINY_D, max_position_embeddings=500), 16))


@pytest.mark.parametrize("name,dtype,folded", [("d", "bf16", False), ("e", "bf16", False), ("f", "bf16", False), ("b", "bf16", False),
                                               ("a", "fp32", False), ("d", "fp32", False), ("d", "bf16", "few"), ("e", "bf16", "few"),
                                               ("d", "bf16", "meet"), ("e", "bf16", "meet"), ("f", "bf16", "meet")])
def test_logits_through_decode_graphs(tmp_path, monkeypatch, name, dtype, folded):
    """folded (options that are off by default; the same logits either way): "few": the products of
    few-token steps add their K pieces themselves and take the norms, the residual sums and SiLU * up in;
    "meet": the last product of a sub-layer adds its K splits and the residual itself and leaves the next
    norm's input, whose 1/rms goes in where the next product's partial sums are consumed."""
    from llmengine.ops import get_ops
    monkeypatch.setattr(get_ops(), "few_token_products", folded == "few")
    monkeypatch.setattr(get_ops(), "meet_products", folded == "meet")
    cfg, page = CONFIGS[name]
    d = str(tmp_path / "m")
    make_model_dir(d, cfg, torch.float32 if dtype == "fp32" else torch.bfloat16)
    pc, pw = P.read_model(d)
    V, limit = cfg["vocab_size"], cfg["max_position_embeddings"]
    steps = 6
    # context lengths: short ones, one that crosses a bucket edge of the block table (16 pages) while
    # it decodes, and one that ends exactly at the position limit
    edge = 16 * page
    lens = [3, limit - steps, edge - 3 if edge + steps < limit else limit // 2, 17, page, page + 1, 2 * page - 2, limit // 3]
    seqs = [random_ids(n + steps, V, 900 + i) for i, n in enumerate(lens)]
    plain = [P.forward_logits(pc, pw, s) for s in seqs]
    pages = sum((len(s) + page - 1) // page for s in seqs) + 4
    eng = llmengine.Engine(d, dtype, block_size=page, num_blocks=pages, max_concurrent=8, cuda_graphs=True)
    H = host_module()
    worst = 0.0
    for live in ([0], [1, 2], [0, 1, 2, 3, 4], list(range(8))):  # capacities 1, 2, 8 (three padded rows), 8
        for i in live:  # the context: one eager prompt step
            eng.run_step([(100 + i, seqs[i][:lens[i]], [])])
        for k in range(steps):
            e = H.StepEntries()
            for i in live:
                assert eng.cm.reserve(100 + i, 1)
                e.add(100 + i, [seqs[i][lens[i] + k]], [0])
            tokens = eng.step_and_sample(e)
            for i in live:
                eng.cm.advance(100 + i, 1)
            g = eng.graphs.last
            assert g is not None and g.pad_to[1] == (1 if len(live) == 1 else 2 if len(live) == 2 else 8)
            logits = g.logits[:len(live)].float().cpu().numpy()
            for r, i in enumerate(live):
                ref = plain[i][lens[i] + k]
                worst = max(worst, float(np.abs(logits[r] - ref).max()))
                assert np.abs(logits[r] - ref).max() < TOL[dtype], \
                    f"{len(live)} live, step {k}, request {i} at position {lens[i] + k}: {np.abs(logits[r] - ref).max():.3e}"
                assert tokens[r] == int(np.argmax(logits[r]))  # greedy rows: the first index of the maximum
        eng.run_step([], end=[100 + i for i in live])
    assert eng.ops.tensor_core_error() == 0
    assert len(eng.graphs.captured) >= 3  # capacities 1, 2, 8 (and more than one table width)
    eng.cm.check()
    assert eng.cm.free_pages(0) == pages


def test_a_recorded_kernel_error_raises_at_the_step_and_the_engine_goes_on(tmp_path):
    """The tensor-core kernels bound their waits; one that gives up leaves a code in a device word.
    Here the HOST writes that word (no kernel has to fail): the step that follows must raise, in the
    eager path and in the graph path, the word must be clear again afterwards, the failed requests
    must give their pages back, and the same prompt must then generate what it generated before."""
    cfg, page = TINY["d"]
    d = str(tmp_path / "m")
    make_model_dir(d, cfg, torch.bfloat16)
    eng = llmengine.Engine(d, "bf16", block_size=page, num_blocks=64, max_concurrent=4)
    prompt = random_ids(40, cfg["vocab_size"], 5)
    before = eng.generate(prompt, 8)
    eng.ops.set_tensor_core_error(22)
    with pytest.raises(llmengine.KernelError, match="code 22"):
        eng.generate(prompt, 8)  # its first step is an eager prompt step
    assert eng.ops.tensor_core_error() == 0 and eng.cm.free_pages(0) == 64
    assert eng.generate(prompt, 8) == before
    # before a graph-replayed decode step, with a request beside it that is not in the failed step
    sch = llmengine.ContinuousBatchScheduler(eng, None, max_concurrent=1, max_prefill_tokens_per_step=64)
    sch.enqueue(prompt, 8)
    sch.enqueue(prompt, 8)
    sch.step()
    sch.step()
    eng.ops.set_tensor_core_error(2)
    with pytest.raises(llmengine.KernelError, match="code 2"):
        sch.step()
    sch.run_until_idle()
    r = sch.results
    assert r[0].finish_reason == "error" and len(r[0].token_ids) == 42
    assert (list(r[1].token_ids), r[1].finish_reason) == before
    assert eng.ops.tensor_core_error() == 0 and eng.cm.free_pages(0) == 64
    eng.cm.check()


def test_an_engine_with_graphs_goes_away_when_it_is_dropped(tmp_path):
    """No reference cycle holds an engine that has recorded decode graphs: dropping it frees the
    graphs and their memory at once, not at some later run of the garbage collector (which might
    be in the middle of another engine's capture, where nothing may be destroyed)."""
    import gc
    import weakref
    cfg, page = CONFIGS["d"]
    d = str(tmp_path / "m")
    make_model_dir(d, cfg, torch.bfloat16)
    gc.collect()
    gc.disable()
    try:
        eng = llmengine.Engine(d, "bf16", block_size=page, num_blocks=40, max_concurrent=4, cuda_graphs=True)
        out, reason = eng.generate(random_ids(9, cfg["vocab_size"], 5), 6)
        assert reason == "length" and len(out) >= 6 and eng.graphs is not None and len(eng.graphs.captured) >= 1
        graphs = weakref.ref(eng.graphs)
        captured = weakref.ref(next(iter(eng.graphs.captured.values())))
        alive = weakref.ref(eng)
        del eng
        assert alive() is None and graphs() is None and captured() is None
    finally:
        gc.enable()
