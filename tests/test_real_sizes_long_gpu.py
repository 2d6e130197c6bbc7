"""The shapes that serving at the Llama 3.2 3B layer sizes reaches and short tests do not: head size
128 with a group of three query heads over 2,048 cached keys. Two layers, so that the plain
implementation can follow on the CPU.

  * a whole prompt of about 2,000 tokens as ONE step (tensor-core attention over 32 key tiles at
    head size 128, token-tile products at M = 2,000, N = 5,120 / 3,072 / 16,384, K = 3,072 / 8,192),
    alone and beside single decoded tokens of other requests, which is how a scheduler fills a batch;
  * decode steps through the CUDA graphs at batch 64 (no key split, the short ring of stages), 8 and
    1 (key splits merged inside thread-block clusters of four and six), with the q|k|v sums, the
    rotation and the cache write folded into the attention kernel.

Every phase ends with the tensor-core kernels' error word still zero: none of their bounded waits
gave up."""
import numpy as np
import pytest
import torch

import llmengine
import plain_llama as P
from llmengine.cache import host_module
from tiny import random_ids

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(420)]  # (the plain side follows 6,300 tokens on the CPU: about a minute)

SIZES_3B = dict(architectures=["LlamaForCausalLM"], hidden_size=3072, intermediate_size=8192, num_hidden_layers=2,
                num_attention_heads=24, num_key_value_heads=8, head_dim=128, vocab_size=128256,
                max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=True,
                rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192))
N_SEQS, SEQ_LEN, BATCH, STEPS = 3, 2100, 64, 3
# bfloat16 against the plain float32 implementation with the same (bf16) weights: rounding noise of
# root mean square about 0.011 at these sizes; a lost key, page or position moves a row by the order
# of the logits themselves (standard deviation about 1.1)
RMS_BOUND, MAX_BOUND = 1.3e-2, 8 * 1.3e-2


def context_len(i: int) -> int:
    return 2000 + (i * 37) % 60  # 2,000 .. 2,059: some cross position 2,048 while they decode


@pytest.fixture(scope="module")
def served(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("sizes_3b"))
    llmengine.write_random_model(d, SIZES_3B, seed=5, dtype=torch.bfloat16, std=0.02)
    pc, pw = P.read_model(d)
    seqs = [random_ids(SEQ_LEN, SIZES_3B["vocab_size"], 70 + s) for s in range(N_SEQS)]
    hidden = [P.final_hidden(pc, pw, ids) for ids in seqs]
    pages = BATCH * 131 + 16  # up to 2,059 + 13 positions a request
    eng = llmengine.Engine(d, "bf16", block_size=16, num_blocks=pages, max_concurrent=BATCH)
    return eng, pc, pw, seqs, hidden, pages


def compare(pc, pw, hidden, got, where):
    """got: [(sequence, position, logits row)]."""
    by_seq = {}
    for s, pos, row in got:
        by_seq.setdefault(s, []).append((pos, row))
    diffs = []
    for s, items in by_seq.items():
        ref = P.logits_at(pc, pw, hidden[s], [p for p, _ in items])
        diffs.append(np.stack([r for _, r in items]) - ref)
    diff = np.concatenate(diffs)
    rms = float(np.sqrt((diff ** 2).mean()))
    assert rms < RMS_BOUND, f"{where}: rms difference {rms}"
    assert np.abs(diff).max() < MAX_BOUND, f"{where}: largest difference per row {np.abs(diff).max(axis=1)}"


def test_prompt_steps_then_decode_at_batch_64_8_and_1(served):
    eng, pc, pw, seqs, hidden, pages = served
    H = host_module()
    # ---- the contexts: one whole-prompt step each; from the fifth on, beside single tokens of the first three
    got, fed = [], {}
    for i in range(BATCH):
        s, L = i % N_SEQS, context_len(i)
        batch = [(i, seqs[s][:L], [0, L - 1])]
        if 4 <= i < 8:
            for j in range(3):
                batch.append((j, [seqs[j % N_SEQS][context_len(j) + fed.get(j, 0)]], [0]))
        lg = eng.run_step(batch).float().cpu().numpy()
        got += [(s, 0, lg[0]), (s, L - 1, lg[1])]
        if 4 <= i < 8:
            for j in range(3):
                got.append((j % N_SEQS, context_len(j) + fed.get(j, 0), lg[2 + j]))
                fed[j] = fed.get(j, 0) + 1
    assert eng.ops.tensor_core_error() == 0
    compare(pc, pw, hidden, got, "whole prompts of about 2,000 tokens")
    # ---- decode steps through the graphs: 64 live requests, then 8, then 1
    live = list(range(BATCH))
    for keep in (BATCH, 8, 1):
        eng.run_step([], end=live[keep:])
        live = live[:keep]
        got = []
        for _ in range(STEPS):
            e = H.StepEntries()
            for i in live:
                assert eng.cm.reserve(i, 1)
                e.add(i, [seqs[i % N_SEQS][context_len(i) + fed.get(i, 0)]], [0])
            eng.step_and_sample(e)
            logits = eng.graphs.last.logits[:len(live)].float().cpu().numpy()
            for r, i in enumerate(live):
                eng.cm.advance(i, 1)
                got.append((i % N_SEQS, context_len(i) + fed.get(i, 0), logits[r]))
                fed[i] = fed.get(i, 0) + 1
        assert eng.ops.tensor_core_error() == 0
        compare(pc, pw, hidden, got, f"decode steps at batch {keep}")
    eng.run_step([], end=live)
    eng.cm.check()
    assert eng.cm.free_pages(0) == pages
