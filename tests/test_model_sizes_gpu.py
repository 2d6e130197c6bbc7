"""The engine at the layer sizes of a real checkpoint (Llama 3.2 1B: hidden 2048, 32 heads over 8
key/value heads of 64, feed-forward 8192, vocabulary 128256, llama3 frequency scaling), cut down to
two layers so that the plain implementation can follow on the CPU. These sizes are where the
tensor-core kernels run in the forms that tiny models never reach: the persistent product, products
cut along K, attention over hundreds of keys with key splits, a vocabulary that is no multiple of
the tile."""
import numpy as np
import pytest
import torch

import llmengine
import plain_llama as P
from tiny import random_ids

pytestmark = pytest.mark.gpu

SIZES = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=8192, num_hidden_layers=2,
             num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=128256,
             max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=True,
             rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                               original_max_position_embeddings=8192))


# Llama 3.2 3B layer sizes: head size 128, a group of three query heads per key/value head
SIZES_3B = dict(SIZES, hidden_size=3072, num_attention_heads=24, head_dim=128)


def _plain_rows(pc, w, ids, rows):
    """Logits of the plain implementation at `rows` only (the head over 128256 entries is the slow part)."""
    T, hd, eps = len(ids), pc["head_dim"], pc["rms_norm_eps"]
    inv = P.llama3_inv_freq(hd, pc["rope_theta"], pc["rope_has_scaling"], pc["rope_factor"], pc["rope_low_freq_factor"],
                            pc["rope_high_freq_factor"], pc["rope_original_max_pos"])
    cos, sin = P.rope_tables(inv, T, hd)
    h = P.embed(w["model.embed_tokens.weight"], ids)
    for l in range(pc["num_hidden_layers"]):
        p = f"model.layers.{l}."
        h = h + P.attention_block(P.rmsnorm(h, w[p + "input_layernorm.weight"], eps), pc, w, l, cos, sin)
        x = P.rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + P.swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return P.linear(P.rmsnorm(h[rows], w["model.norm.weight"], eps), w["lm_head.weight"])


@pytest.mark.parametrize("sizes", [SIZES, SIZES_3B], ids=["1b", "3b"])
def test_real_layer_sizes_prompt_portions_and_decoding(tmp_path, sizes):
    d = str(tmp_path / "m")
    llmengine.write_random_model(d, sizes, seed=3, dtype=torch.bfloat16, std=0.02)
    pc, pw = P.read_model(d)
    T, tail = 1000, 6
    ids = random_ids(T, sizes["vocab_size"], 41)
    rows = [0, 1, 299, 300, 301, T - tail - 1] + list(range(T - tail, T))
    ref = _plain_rows(pc, pw, ids, rows)
    eng = llmengine.Engine(d, "bf16", block_size=16, num_blocks=80, max_concurrent=2)
    got = []
    # a portion of 300 tokens (3 x 64 tiles of gate|up: below the persistent product's threshold), one
    # of 694 (above it), then single tokens over 994..999 keys (key splits, products cut along K)
    lg = eng.run_step([(1, ids[:300], [0, 1, 299])]).clone()
    got.append(lg)
    lg = eng.run_step([(1, ids[300:T - tail], [0, 1, T - tail - 1 - 300])]).clone()
    got.append(lg)
    for t in range(T - tail, T):
        got.append(eng.run_step([(1, ids[t:t + 1], [0])], end=[1] if t == T - 1 else []).clone())
    got = torch.cat(got).cpu().numpy()
    assert eng.ops.tensor_core_error() == 0
    # 12 rows x 128,256 logits of standard deviation ~1.1: the bfloat16 path differs from the plain
    # float32 one by rounding noise of root mean square 0.0107 (both layer sizes, every kernel version
    # so far), whose largest of 1.5 million samples is about 5.3 sigma = 0.057 and moves by +-0.005
    # with any reordering of sums. So the bound on the noise is on its root mean square; the largest
    # difference only has to stay where noise of that size can reach (a lost key, page or position
    # moves a whole row by the order of the logits themselves).
    diff = got - ref
    assert np.sqrt((diff ** 2).mean()) < 1.3e-2, f"rms difference {np.sqrt((diff ** 2).mean())}"
    assert np.abs(diff).max() < 8 * 1.3e-2, f"largest difference per row: {np.abs(diff).max(axis=1)}"
    # the same tokens chosen by both
    assert (got.argmax(1) == ref.argmax(1)).all()

    # generation through the scheduler (decoding steps replay CUDA graphs over a padded batch) chooses
    # the tokens that stepping by hand chooses
    prompt = ids[:333]
    out, reason = eng.generate(prompt, 6)
    assert reason == "length" and out[:333] == prompt
    seq = list(prompt)
    lg = eng.run_step([(7, seq, [len(seq) - 1])])
    for _ in range(6):
        tok = int(lg[0].argmax())
        seq.append(tok)
        lg = eng.run_step([(7, [tok], [0])])
    eng.run_step([], end=[7])
    assert out == seq


def test_float32_path_and_bfloat16_drift_at_real_layer_sizes(tmp_path):
    """A short prompt at the 1B layer sizes through the true 32-bit path (CUDA-core products, no
    reduced-precision matrix mode: equal to the plain implementation to summation order) and through
    bfloat16 with the same weights: the drift between the two precisions stays within the bound
    that the tiny models are held to."""
    d = str(tmp_path / "m")
    llmengine.write_random_model(d, SIZES, seed=4, dtype=torch.bfloat16, std=0.02)
    pc, pw = P.read_model(d)
    ids = random_ids(24, SIZES["vocab_size"], 43)
    ref = _plain_rows(pc, pw, ids, list(range(24)))
    got = {}
    for dtype in ("fp32", "bf16"):
        eng = llmengine.Engine(d, dtype, block_size=16, num_blocks=8, max_concurrent=1)
        a = eng.run_step([(1, ids[:20], range(20))]).clone()
        rest = [eng.run_step([(1, ids[t:t + 1], [0])], end=[1] if t == 23 else []).clone() for t in range(20, 24)]
        got[dtype] = torch.cat([a] + rest).cpu().numpy()
        del eng
        torch.cuda.empty_cache()
    assert np.abs(got["fp32"] - ref).max() < 2e-4
    assert np.abs(got["bf16"] - got["fp32"]).max() < 6e-2
    assert (got["fp32"].argmax(1) == ref.argmax(1)).all()
