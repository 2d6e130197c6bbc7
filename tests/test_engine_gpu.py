"""The engine on the GPU through its Python entry point: greedy and sampled generation, long
decoding, the first tokens of a sequence, the scheduler against each request alone, and a toy mixer
with state of its own that is registered, built and stepped without touching the framework."""
import json
import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import llmengine
import plain_llama as P
from tiny import TINY_A, TINY_B, TINY_D, TINY_E, make_model_dir, random_ids

pytestmark = pytest.mark.gpu
TOL = {"fp32": 2e-4, "bf16": 6e-2}


# f: configuration d with a position limit (500) that is no multiple of 16 pages of 16 positions
TINY_F = dict(TINY_D, max_position_embeddings=500)


@pytest.fixture(scope="module", params=[("a", "fp32"), ("a", "bf16"), ("b", "fp32"), ("b", "bf16"), ("d", "fp32"), ("d", "bf16"),
                                        ("e", "fp32"), ("e", "bf16"), ("f", "bf16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    name, dtype = request.param
    # d: head size 64, pages of 16: the tensor-core attention kernels; e: head size 128, a group of three, pages of 32
    cfg = {"a": TINY_A, "b": TINY_B, "d": TINY_D, "e": TINY_E, "f": TINY_F}[name]
    d = str(tmp_path_factory.mktemp(f"eng_{name}_{dtype}"))
    make_model_dir(d, cfg, torch.float32 if dtype == "fp32" else torch.bfloat16)
    pc, pw = P.read_model(d)
    eng = llmengine.Engine(d, dtype, block_size={"a": 4, "e": 32}.get(name, 16), num_blocks=96, max_concurrent=8)
    return cfg, eng, pc, pw, dtype


def check_stream(pc, pw, prompt, tokens, tol, temperature=0.0, seed=0):
    """Every generated token must be the plain implementation's choice, or differ from it only where
    the plain scores of the two are closer than the tolerance (a near tie that rounding may flip)."""
    logits = P.forward_logits(pc, pw, tokens[:-1]) if len(tokens) > len(prompt) else None
    for k in range(len(prompt), len(tokens)):
        row = logits[k - 1].astype(np.float32)
        if temperature > 0:
            row = row * (np.float32(1.0) / np.float32(temperature)) + P.gumbel_noise(seed, k - len(prompt), row.shape[0])
        best = int(np.argmax(row))
        assert tokens[k] == best or row[best] - row[tokens[k]] < 2 * tol / max(temperature, 1.0) + 2 * tol, \
            f"token {k}: engine chose {tokens[k]}, plain chooses {best} by {row[best] - row[tokens[k]]:.4f}"


def test_forward_logits_and_first_tokens(setup):
    cfg, eng, pc, pw, dtype = setup
    for n in (1, 2, 3, 21):  # the first tokens of a sequence, alone
        ids = random_ids(n, cfg["vocab_size"], 7 + n)
        np.testing.assert_allclose(eng.forward_logits(ids), P.forward_logits(pc, pw, ids), atol=TOL[dtype], rtol=0)
    assert eng.cm.free_pages(0) == 96
    assert eng.dtype == dtype and eng.max_pos == cfg["max_position_embeddings"] and eng.cfg.vocab_size == cfg["vocab_size"]
    assert eng.has_weight("model.norm.weight") and eng.has_weight("lm_head.weight")


def test_greedy_generation_and_long_decoding(setup):
    cfg, eng, pc, pw, dtype = setup
    prompt = random_ids(9, cfg["vocab_size"], 3)
    n_new = cfg["max_position_embeddings"] - 9  # decode up to the position limit
    out, reason = eng.generate(prompt, n_new)
    assert reason == "length" and len(out) == cfg["max_position_embeddings"] and out[:9] == prompt
    check_stream(pc, pw, prompt, out, TOL[dtype])
    if dtype == "fp32":
        assert out[:21] == P.generate(pc, pw, prompt, 12)[0]
    assert eng.generate(prompt, 0) == (prompt, "length")
    with pytest.raises(RuntimeError, match="position limit"):
        eng.generate(prompt, n_new + 1)
    with pytest.raises(ValueError, match="out of range"):
        eng.forward_logits([cfg["vocab_size"]])


def test_eos_stops_generation(setup, tmp_path):
    cfg, eng, pc, pw, dtype = setup
    prompt = random_ids(5, cfg["vocab_size"], 11)
    out, _ = eng.generate(prompt, 6)
    stop_at = out[7]
    d = str(tmp_path / "eos")
    os.makedirs(d)
    with open(os.path.join(eng.model_dir, "config.json")) as f:
        c = json.load(f)
    c["eos_token_id"] = [stop_at]
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(c, f)
    os.symlink(os.path.join(eng.model_dir, "model.safetensors"), os.path.join(d, "model.safetensors"))
    eng2 = llmengine.Engine(d, dtype, block_size=4, num_blocks=32)
    out2, reason2 = eng2.generate(prompt, 6)
    assert reason2 == "stop" and out2 == out[:out.index(stop_at, 5)]


def test_scheduler_equals_each_request_alone(setup):
    cfg, eng, pc, pw, dtype = setup
    lens = [5, 11, 17, 2, 30]
    news = [8, 0, 1, 5, 12]
    prompts = [random_ids(n, cfg["vocab_size"], 60 + n) for n in lens]
    alone = [eng.generate(p, k) for p, k in zip(prompts, news)]
    bm = llmengine.BlockManager(64, eng.cm.page_size)
    sch = llmengine.ContinuousBatchScheduler(eng, bm, max_concurrent=3, max_prefill_tokens_per_step=8)
    for p, k in zip(prompts, news):
        sch.enqueue(p, k)
    sch.run_until_idle()
    assert bm.free_blocks == 64 and sch.idle
    for r, (toks, reason), p in zip(sch.results, alone, prompts):
        assert r.finish_reason == reason and r.prompt_len == len(p)
        if dtype == "fp32":
            assert list(r.token_ids) == toks
        else:  # batching changes bf16 rounding: allow a near tie to flip, then the streams part ways
            check_stream(pc, pw, p, list(r.token_ids), TOL[dtype])
    eng.configure_cache(num_blocks=96, block_size=eng.cm.page_size, num_slots=8)


def test_temperature_sampling(setup):
    cfg, eng, pc, pw, dtype = setup
    prompt = random_ids(6, cfg["vocab_size"], 21)
    a, _ = eng.generate(prompt, 10, temperature=1.0, seed=42)
    b, _ = eng.generate(prompt, 10, temperature=1.0, seed=42)
    c, _ = eng.generate(prompt, 10, temperature=1.0, seed=43)
    assert a == b and a != c
    check_stream(pc, pw, prompt, a, TOL[dtype], temperature=1.0, seed=42)
    if dtype == "fp32":
        assert a == P.generate(pc, pw, prompt, 10, temperature=1.0, seed=42)[0]


# ------------------------------------------------------------------------------------ a toy mixer
@dataclass(frozen=True)
class RunningMeanSpec:
    kind: str
    hidden: int
    weight: str


def _register_toy():
    """A mixer with fixed-size state of its own: out_t = W * mean(x_0..x_t). Its state (the running
    sum, one vector per request) lives in the request's slot. Defined here, in the test; the
    framework's files are not touched."""
    from llmengine.config.registry import Architecture, register_architecture
    from llmengine.config.llama import LlamaConfig
    from llmengine.models.llama import describe_llama
    from llmengine.parts import Mixer, StateNeed, TensorNeed, register_part
    from dataclasses import replace

    class RunningMean(Mixer):
        capturable = False  # its forward reads the batch on the host: no CUDA graph may record it

        @staticmethod
        def tensor_needs(spec):
            return [TensorNeed(spec.weight, (spec.hidden, spec.hidden))]

        def cache_needs(self):
            return (StateNeed("sum", (self.spec.hidden,), torch.float32),)

        def load(self, tensors):
            self.w = tensors[self.spec.weight]

        def forward(self, x, ctx, cache):
            state = cache.states["sum"]
            out = torch.empty(ctx.n_tokens, self.spec.hidden, dtype=torch.float32, device=x.device)
            qoff, start, slot = ctx.seq_qoff.tolist(), ctx.seq_start.tolist(), ctx.seq_slot.tolist()
            for s in range(ctx.n_seqs):
                xs = x[qoff[s]:qoff[s + 1]].float()
                run = state[slot[s]] + torch.cumsum(xs, 0)
                state[slot[s]] = run[-1]
                counts = torch.arange(start[s] + 1, start[s] + 1 + xs.shape[0], device=x.device).unsqueeze(1)
                out[qoff[s]:qoff[s + 1]] = (run / counts) @ self.w.float().t()
            return out

    register_part("mixer", "running_mean", RunningMean, replace=True)

    def describe(cfg):
        spec = describe_llama(cfg)
        layers = list(spec.layers)  # layer 1 keeps attention, layer 0 gets the toy mixer
        layers[0] = replace(layers[0], mixer=RunningMeanSpec("running_mean", cfg.hidden_size, "model.layers.0.toy.weight"))
        return replace(spec, architecture="ToyStateModel", layers=tuple(layers))

    register_architecture(Architecture("ToyStateModel", LlamaConfig.from_dict, describe,
                                       lambda c: dict(c.to_dict(), architectures=["ToyStateModel"])), replace=True)


def _toy_plain(pc, w, ids):
    T = len(ids)
    inv = P.llama3_inv_freq(pc["head_dim"], pc["rope_theta"], False, 1, 1, 1, 0)
    cos, sin = P.rope_tables(inv, T, pc["head_dim"])
    h = P.embed(w["model.embed_tokens.weight"], ids)
    x = P.rmsnorm(h, w["model.layers.0.input_layernorm.weight"], pc["rms_norm_eps"])
    mean = np.cumsum(x, axis=0) / np.arange(1, T + 1, dtype=np.float32)[:, None]
    h = h + P.linear(mean.astype(np.float32), w["model.layers.0.toy.weight"])
    x = P.rmsnorm(h, w["model.layers.0.post_attention_layernorm.weight"], pc["rms_norm_eps"])
    h = h + P.swiglu_mlp(x, w["model.layers.0.mlp.gate_proj.weight"], w["model.layers.0.mlp.up_proj.weight"], w["model.layers.0.mlp.down_proj.weight"])
    x = P.rmsnorm(h, w["model.layers.1.input_layernorm.weight"], pc["rms_norm_eps"])
    h = h + P.attention_block(x, pc, w, 1, cos, sin)
    x = P.rmsnorm(h, w["model.layers.1.post_attention_layernorm.weight"], pc["rms_norm_eps"])
    h = h + P.swiglu_mlp(x, w["model.layers.1.mlp.gate_proj.weight"], w["model.layers.1.mlp.up_proj.weight"], w["model.layers.1.mlp.down_proj.weight"])
    return P.linear(P.rmsnorm(h, w["model.norm.weight"], pc["rms_norm_eps"]), w["lm_head.weight"])


def test_toy_mixer_with_state_can_be_registered_built_and_stepped(tmp_path):
    _register_toy()
    cfg = dict(TINY_A, architectures=["ToyStateModel"])
    d = str(tmp_path / "toy")
    llmengine.write_random_model(d, cfg, seed=5, dtype=torch.float32, std=0.05)
    pc, pw = P.read_model(d)
    assert "model.layers.0.toy.weight" in pw and "model.layers.0.self_attn.q_proj.weight" not in pw
    eng = llmengine.Engine(d, "fp32", block_size=4, num_blocks=24, max_concurrent=2)
    ids_a, ids_b = random_ids(23, 256, 1), random_ids(14, 256, 2)
    ref_a, ref_b = _toy_plain(pc, pw, ids_a), _toy_plain(pc, pw, ids_b)
    np.testing.assert_allclose(eng.forward_logits(ids_a), ref_a, atol=2e-4, rtol=0)
    # two requests interleaved in portions: each one's state stays in its own slot; a slot that is
    # used again starts from zero
    got_a, got_b = [], []
    got_a.append(eng.run_step([(1, ids_a[:5], range(5))]).clone())
    lg = eng.run_step([(1, ids_a[5:7], range(2)), (2, ids_b[:9], range(9))])
    got_a.append(lg[:2].clone()); got_b.append(lg[2:].clone())
    lg = eng.run_step([(2, ids_b[9:], range(5)), (1, ids_a[7:], range(16))], end=[1, 2])
    got_b.append(lg[:5].clone()); got_a.append(lg[5:].clone())
    np.testing.assert_allclose(torch.cat(got_a).cpu().numpy(), ref_a, atol=2e-4, rtol=0)
    np.testing.assert_allclose(torch.cat(got_b).cpu().numpy(), ref_b, atol=2e-4, rtol=0)
    np.testing.assert_allclose(eng.run_step([(3, ids_b, range(14))], end=[3]).cpu().numpy(), ref_b, atol=2e-4, rtol=0)
    out, reason = eng.generate(ids_b[:4], 5)
    assert len(out) == 9 and reason == "length" and eng.cm.free_slots == 2
    # bfloat16 serving replays CUDA graphs for decode steps, unless a part says that it cannot be
    # recorded: then generation and the scheduler run the same steps kernel by kernel
    engb = llmengine.Engine(d, "bf16", block_size=4, num_blocks=24, max_concurrent=2)
    np.testing.assert_allclose(engb.forward_logits(ids_a), ref_a, atol=6e-2, rtol=0)
    assert engb.cuda_graphs is False and engb.graphs is None
    outb, reason = engb.generate(ids_b[:4], 8)
    assert len(outb) == 12 and reason == "length" and engb.graphs is None
    lg = _toy_plain(pc, pw, outb)
    for k in range(4, 12):  # each token is the plain model's choice, or a near tie
        best = int(lg[k - 1].argmax())
        assert outb[k] == best or lg[k - 1][best] - lg[k - 1][outb[k]] < 0.12


# ------------------------------------------------- a toy routed feed-forward, a toy position encoding
@dataclass(frozen=True)
class Top1ExpertsSpec:
    kind: str
    hidden: int
    experts: int
    router: str
    expert_weights: tuple  # tensor names, one [hidden, hidden] matrix each


@dataclass(frozen=True)
class AddedPositionSpec:
    kind: str
    head_dim: int
    max_positions: int
    table: str  # [max_positions, head_dim]: added to every q and k head at its position


def _register_toy_routing_and_position():
    """A feed-forward that routes every token to the best of three experts (router logits and their
    softmax in float32, the step's tokens grouped by expert), and a position encoding that is not a
    rotation: a learned vector per position added to q and k. Both live in this file only."""
    from dataclasses import replace
    from llmengine.config.registry import Architecture, register_architecture
    from llmengine.config.llama import LlamaConfig
    from llmengine.models.llama import describe_llama
    from llmengine.parts import FeedForward, PositionEncoding, TensorNeed, register_part

    class Top1Experts(FeedForward):
        @staticmethod
        def tensor_needs(spec):
            return [TensorNeed(spec.router, (spec.experts, spec.hidden), "float32")] + \
                   [TensorNeed(n, (spec.hidden, spec.hidden)) for n in spec.expert_weights]

        def load(self, tensors):
            self.router = tensors[self.spec.router]
            self.w = [tensors[n] for n in self.spec.expert_weights]

        def forward(self, x, ctx):
            n = ctx.n_tokens
            xf = x[:n].float()
            prob = torch.softmax(xf @ self.router.t(), dim=-1)
            best = prob.argmax(dim=-1)
            out = torch.zeros(n, self.spec.hidden, dtype=torch.float32, device=x.device)
            for e in range(self.spec.experts):  # the step's tokens of expert e, whichever request they are of
                rows = (best == e).nonzero().squeeze(1)
                if rows.numel():
                    out[rows] = prob[rows, e].unsqueeze(1) * (xf[rows] @ self.w[e].float().t())
            return out

    class AddedPosition(PositionEncoding):
        @staticmethod
        def tensor_needs(spec):
            return [TensorNeed(spec.table, (spec.max_positions, spec.head_dim), "float32")]

        def load(self, tensors):
            self.table = tensors[self.spec.table]

        def rotate_and_store(self, qkv, ctx, cache, num_heads, num_kv_heads, head_dim, parts=None):
            assert parts is None  # takes_partial_sums is False: finished values only
            n = ctx.n_tokens
            add = self.table[ctx.positions[:n].long()]  # [n, head_dim]
            qk = qkv[:n, :(num_heads + num_kv_heads) * head_dim].view(n, num_heads + num_kv_heads, head_dim)
            qk.copy_((qk.float() + add.unsqueeze(1)).to(qkv.dtype))
            if cache.writes and cache.k is not None:  # the framework's kernel, without tables, stores k and v
                self.env.ops.rope_kv_write(qkv, ctx.positions, ctx.token_seq, ctx.block_tables[cache.group], None, None,
                                           cache.k, cache.v, n, num_heads, num_kv_heads, head_dim)

    register_part("feed_forward", "top1_experts", Top1Experts, replace=True)
    register_part("position", "added", AddedPosition, replace=True)

    def describe(cfg):
        spec = describe_llama(cfg)
        layers = list(spec.layers)
        pos = AddedPositionSpec("added", cfg.head_dim, cfg.max_position_embeddings, "model.toy_positions.weight")
        layers[0] = replace(layers[0], mixer=replace(layers[0].mixer, position=pos))  # layer 0: added positions, dense MLP
        layers[1] = replace(layers[1], feed_forward=Top1ExpertsSpec(             # layer 1: rotary, routed experts
            "top1_experts", cfg.hidden_size, 3, "model.layers.1.toy.router.weight",
            tuple(f"model.layers.1.toy.experts.{e}.weight" for e in range(3))))
        return replace(spec, architecture="ToyRoutedModel", layers=tuple(layers))

    register_architecture(Architecture("ToyRoutedModel", LlamaConfig.from_dict, describe,
                                       lambda c: dict(c.to_dict(), architectures=["ToyRoutedModel"])), replace=True)


def _toy_routed_plain(pc, w, ids):
    T, hd, nq, nkv, eps = len(ids), pc["head_dim"], pc["num_attention_heads"], pc["num_key_value_heads"], pc["rms_norm_eps"]
    cos, sin = P.rope_tables(P.llama3_inv_freq(hd, pc["rope_theta"], False, 1, 1, 1, 0), T, hd)
    h = P.embed(w["model.embed_tokens.weight"], ids)
    # layer 0: attention with added positions, dense MLP
    p = "model.layers.0."
    x = P.rmsnorm(h, w[p + "input_layernorm.weight"], eps)
    add = w["model.toy_positions.weight"][:T][:, None, :]
    q = P.linear(x, w[p + "self_attn.q_proj.weight"]).reshape(T, nq, hd) + add
    k = P.linear(x, w[p + "self_attn.k_proj.weight"]).reshape(T, nkv, hd) + add
    v = P.linear(x, w[p + "self_attn.v_proj.weight"]).reshape(T, nkv, hd)
    h = h + P.linear(P.causal_gqa_attention(q.astype(np.float32), k.astype(np.float32), v), w[p + "self_attn.o_proj.weight"])
    x = P.rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps)
    h = h + P.swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    # layer 1: rotary attention, top-1 of three experts
    p = "model.layers.1."
    x = P.rmsnorm(h, w[p + "input_layernorm.weight"], eps)
    h = h + P.attention_block(x, pc, w, 1, cos, sin)
    x = P.rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps)
    logits = P.linear(x, w[p + "toy.router.weight"])
    prob = np.exp(logits - logits.max(-1, keepdims=True))
    prob = prob / prob.sum(-1, keepdims=True)
    best = prob.argmax(-1)
    routed = np.stack([prob[t, best[t]] * P.linear(x[t:t + 1], w[p + f"toy.experts.{best[t]}.weight"])[0] for t in range(T)])
    h = h + routed.astype(np.float32)
    top2 = np.sort(prob, axis=-1)[:, -2:]
    return P.linear(P.rmsnorm(h, w["model.norm.weight"], eps), w["lm_head.weight"]), best, top2[:, 1] - top2[:, 0]


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_toy_routed_feed_forward_and_toy_position_encoding(tmp_path, dtype):
    """Parts of other kinds than the architecture's, registered from here: a layer with a position
    encoding that is no rotation beside a rotary one, a routed feed-forward beside a dense one; whole,
    in portions, and two requests mixed in a step (the experts see tokens of both)."""
    _register_toy_routing_and_position()
    cfg = dict(TINY_A, architectures=["ToyRoutedModel"])
    d = str(tmp_path / "routed")
    llmengine.write_random_model(d, cfg, seed=8, dtype=torch.float32, std=0.05)
    pc, pw = P.read_model(d)
    if dtype == "bf16":  # the plain model gets the weights the engine will hold
        pw = {k: (torch.from_numpy(v).bfloat16().float().numpy() if v.ndim == 2 and "toy_positions" not in k and "router" not in k else v)
              for k, v in pw.items()}
    assert "model.layers.1.toy.experts.2.weight" in pw and "model.layers.1.mlp.gate_proj.weight" not in pw
    ids_a, ids_b = random_ids(40, 256, 11), random_ids(27, 256, 12)
    (ref_a, best_a, gap_a), (ref_b, best_b, gap_b) = _toy_routed_plain(pc, pw, ids_a), _toy_routed_plain(pc, pw, ids_b)
    assert len(set(best_a.tolist()) | set(best_b.tolist())) == 3, "the test wants every expert used"
    tol_ = dict(atol=2e-4, rtol=0) if dtype == "fp32" else dict(atol=6e-2, rtol=0)
    # The routed layer is the last one, so a token's choice of expert touches its own logits only.
    # A token whose two best experts are nearly tied may go either way under bfloat16 rounding of
    # the router's input; such rows are left out of the comparison (not of the run).
    min_gap = 1e-4 if dtype == "fp32" else 2e-2
    keep_a, keep_b = gap_a > min_gap, gap_b > min_gap
    assert keep_a.sum() > 30 and keep_b.sum() > 20
    eng = llmengine.Engine(d, dtype, block_size=4, num_blocks=40, max_concurrent=2)
    np.testing.assert_allclose(eng.forward_logits(ids_a)[keep_a], ref_a[keep_a], **tol_)
    got_a, got_b = [], []
    got_a.append(eng.run_step([(1, ids_a[:13], range(13))]).clone())
    lg = eng.run_step([(2, ids_b[:20], range(20)), (1, ids_a[13:15], range(2))])
    got_b.append(lg[:20].clone()); got_a.append(lg[20:].clone())
    for t in range(15, 40):  # request 1 decodes token by token while request 2 ends its prompt
        batch = [(1, ids_a[t:t + 1], [0])]
        if t == 15:
            batch.append((2, ids_b[20:], range(7)))
        lg = eng.run_step(batch, end=([1] if t == 39 else []) + ([2] if t == 15 else []))
        got_a.append(lg[:1].clone())
        if t == 15:
            got_b.append(lg[1:].clone())
    np.testing.assert_allclose(torch.cat(got_a).cpu().numpy()[keep_a], ref_a[keep_a], **tol_)
    np.testing.assert_allclose(torch.cat(got_b).cpu().numpy()[keep_b], ref_b[keep_b], **tol_)
    assert eng.cm.free_slots == 2


def test_layer_order_is_data(tmp_path):
    """The order in which layers run is a list: it may name a layer twice, and a run may read an
    earlier run's cache instead of keeping its own."""
    from dataclasses import replace
    from llmengine.config.registry import Architecture, register_architecture
    from llmengine.config.llama import LlamaConfig
    from llmengine.models.llama import describe_llama
    from llmengine.parts import LayerRun

    def describe(cfg):
        spec = describe_llama(cfg)
        return replace(spec, architecture="LoopedModel", order=(LayerRun(0), LayerRun(1), LayerRun(0), LayerRun(1, cache_from=1)))

    register_architecture(Architecture("LoopedModel", LlamaConfig.from_dict, describe,
                                       lambda c: dict(c.to_dict(), architectures=["LoopedModel"])), replace=True)
    cfg = dict(TINY_A, architectures=["LoopedModel"])
    d = str(tmp_path / "looped")
    llmengine.write_random_model(d, cfg, seed=6, dtype=torch.float32, std=0.05)
    pc, w = P.read_model(d)
    ids = random_ids(19, 256, 4)
    T, hd, nq, nkv = 19, 16, 4, 2
    cos, sin = P.rope_tables(P.llama3_inv_freq(hd, pc["rope_theta"], False, 1, 1, 1, 0), T, hd)

    def mlp(h, l):
        p = f"model.layers.{l}."
        x = P.rmsnorm(h, w[p + "post_attention_layernorm.weight"], pc["rms_norm_eps"])
        return h + P.swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])

    h = P.embed(w["model.embed_tokens.weight"], ids)
    kv1 = None
    for run, (l, borrow) in enumerate([(0, False), (1, False), (0, False), (1, True)]):
        p = f"model.layers.{l}."
        x = P.rmsnorm(h, w[p + "input_layernorm.weight"], pc["rms_norm_eps"])
        q = P.apply_rope(P.linear(x, w[p + "self_attn.q_proj.weight"]).reshape(T, nq, hd), cos, sin)
        if borrow:
            k, v = kv1  # keys and values that run 1 wrote
        else:
            k = P.apply_rope(P.linear(x, w[p + "self_attn.k_proj.weight"]).reshape(T, nkv, hd), cos, sin)
            v = P.linear(x, w[p + "self_attn.v_proj.weight"]).reshape(T, nkv, hd)
            if run == 1:
                kv1 = (k, v)
        h = h + P.linear(P.causal_gqa_attention(q, k, v), w[p + "self_attn.o_proj.weight"])
        h = mlp(h, l)
    ref = P.linear(P.rmsnorm(h, w["model.norm.weight"], pc["rms_norm_eps"]), w["lm_head.weight"])
    eng = llmengine.Engine(d, "fp32", block_size=4, num_blocks=24)
    np.testing.assert_allclose(eng.forward_logits(ids), ref, atol=2e-4, rtol=0)
    first = eng.run_step([(9, ids[:11], range(11))]).clone()  # the logits tensor is scratch of the next step
    second = eng.run_step([(9, ids[11:], range(8))], end=[9])
    np.testing.assert_allclose(torch.cat([first, second]).cpu().numpy(), ref, atol=2e-4, rtol=0)


@pytest.mark.parametrize("which", ["a", "d"])
def test_window_layers_share_the_engine_with_full_layers(tmp_path, which):
    """A model whose first layer reads a window of the last W keys and whose second reads all of
    them: two cache groups with their own pages; the window group gives pages back while a request
    is still running, and they are used again by the next one. Configuration A (head size 16, pages
    of 4, W = 9) and D (head size 64, pages of 16, W = 70: the tensor-core kernels, with block-table
    entries of pages that were given back)."""
    from dataclasses import replace
    from llmengine.config.registry import Architecture, register_architecture
    from llmengine.config.llama import LlamaConfig
    from llmengine.models.llama import describe_llama
    base, page, W, T, cuts = {"a": (TINY_A, 4, 9, 41, (6, 2, 13, 1, 1, 9, 9)),
                              "d": (TINY_D, 16, 70, 300, (40, 2, 90, 1, 1, 100, 33, 1, 1, 1, 30))}[which]
    assert sum(cuts) == T

    def describe(cfg):
        spec = describe_llama(cfg)
        layers = list(spec.layers)
        layers[0] = replace(layers[0], mixer=replace(layers[0].mixer, window=W))
        return replace(spec, architecture="WindowedModel", layers=tuple(layers))

    register_architecture(Architecture("WindowedModel", LlamaConfig.from_dict, describe,
                                       lambda c: dict(c.to_dict(), architectures=["WindowedModel"])), replace=True)
    cfg = dict(base, architectures=["WindowedModel"])
    hd, nq, nkv, V = base["head_dim"], base["num_attention_heads"], base["num_key_value_heads"], base["vocab_size"]
    n_pages = (T + page - 1) // page + 2
    for dtype, wdt, tol in (("fp32", torch.float32, 2e-4), ("bf16", torch.bfloat16, 6e-2)):
        d = str(tmp_path / f"windowed_{dtype}")
        llmengine.write_random_model(d, cfg, seed=8, dtype=wdt, std=0.05)
        pc, w = P.read_model(d)
        ids = random_ids(T, V, 12)
        inv = P.llama3_inv_freq(hd, pc["rope_theta"], pc["rope_has_scaling"], pc["rope_factor"], pc["rope_low_freq_factor"],
                                pc["rope_high_freq_factor"], pc["rope_original_max_pos"])
        cos, sin = P.rope_tables(inv, T, hd)
        h = P.embed(w["model.embed_tokens.weight"], ids)
        for l in range(2):
            p = f"model.layers.{l}."
            x = P.rmsnorm(h, w[p + "input_layernorm.weight"], pc["rms_norm_eps"])
            q = P.apply_rope(P.linear(x, w[p + "self_attn.q_proj.weight"]).reshape(T, nq, hd), cos, sin)
            k = P.apply_rope(P.linear(x, w[p + "self_attn.k_proj.weight"]).reshape(T, nkv, hd), cos, sin)
            v = P.linear(x, w[p + "self_attn.v_proj.weight"]).reshape(T, nkv, hd)
            if l == 0:  # the plain implementation has no window: restrict the keys query by query
                a = np.stack([_window_row(q[t], k[max(0, t - W + 1):t + 1], v[max(0, t - W + 1):t + 1], nq, nkv, hd) for t in range(T)])
            else:
                a = P.causal_gqa_attention(q, k, v)
            h = h + P.linear(a, w[p + "self_attn.o_proj.weight"])
            x = P.rmsnorm(h, w[p + "post_attention_layernorm.weight"], pc["rms_norm_eps"])
            h = h + P.swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        head = w["model.embed_tokens.weight"] if pc["tie_word_embeddings"] else w["lm_head.weight"]
        ref = P.linear(P.rmsnorm(h, w["model.norm.weight"], pc["rms_norm_eps"]), head)
        eng = llmengine.Engine(d, dtype, block_size=page, num_blocks=n_pages, max_concurrent=2)  # a little more than one request's pages per group
        eng.configure_cache()
        assert eng.cm.num_groups == 2 and sorted(eng.cm.window(g) for g in range(2)) == [0, W]
        gw = [g for g in range(2) if eng.cm.window(g) == W][0]
        got, pos = [], 0
        for n in cuts:
            got.append(eng.run_step([(1, ids[pos:pos + n], range(n))]).clone())
            pos += n
            held = sum(pg >= 0 for pg in eng.cm.block_table(1, gw))
            assert held <= (W + page - 1) // page + 1  # the window group never holds more than the window needs
        assert sum(pg >= 0 for pg in eng.cm.block_table(1, 1 - gw)) == (T + page - 1) // page
        np.testing.assert_allclose(torch.cat(got).float().cpu().numpy(), ref, atol=tol, rtol=0)
        # a second request of the same length goes through the pages that came back
        eng.run_step([], end=[1])
        again = eng.run_step([(2, ids, range(T))], end=[2])
        np.testing.assert_allclose(again.float().cpu().numpy(), ref, atol=tol, rtol=0)
        eng.cm.check()
        assert eng.cm.free_pages(0) == n_pages and eng.cm.free_pages(1) == n_pages


def _window_row(q, k, v, nq, nkv, hd):
    out = np.zeros((nq, hd), dtype=np.float32)
    for hh in range(nq):
        s = (k[:, hh // (nq // nkv)] @ q[hh]) / np.sqrt(np.float32(hd))
        pr = np.exp(s - s.max())
        out[hh] = (pr / pr.sum()) @ v[:, hh // (nq // nkv)]
    return out.reshape(-1)


@pytest.mark.parametrize("name,dtype,seed", [("d", "fp32", 1), ("a", "fp32", 2), ("e", "fp32", 3), ("d", "bf16", 4), ("e", "bf16", 5),
                                             ("f", "bf16", 6)])
def test_scheduler_under_random_load_and_page_pressure(tmp_path, name, dtype, seed):
    """Forty requests of random lengths, budgets and temperatures arrive while others run, through a
    pool that holds about three of them: many end with "capacity". Every request's tokens are the
    plain implementation's for the same prompt (32-bit; a token may differ only at a provable near
    tie), "length" means exactly max_new_tokens, and no page is lost."""
    from tiny import TINY
    rng = np.random.default_rng(seed)
    cfg, page = dict(TINY, f=(TINY_F, 16))[name]
    d = str(tmp_path / "m")
    make_model_dir(d, cfg, torch.float32 if dtype == "fp32" else torch.bfloat16)
    pc, pw = P.read_model(d)
    maxpos = cfg["max_position_embeddings"]
    n_pages = (3 * maxpos // 2) // page
    eng = llmengine.Engine(d, dtype, block_size=page, num_blocks=n_pages, max_concurrent=6)
    sch = llmengine.ContinuousBatchScheduler(eng, None, max_concurrent=6, max_prefill_tokens_per_step=int(rng.integers(8, 100)))
    reqs = {}
    for i in range(40):
        L = int(rng.integers(1, maxpos // 2))
        new = int(rng.integers(0, min(60, maxpos - L)))
        temp = float(rng.choice([0.0, 0.0, 1.0]))
        prompt = rng.integers(0, cfg["vocab_size"], L).tolist()
        reqs[sch.enqueue(prompt, new, temp, i)] = (prompt, new, temp, i)
        if rng.random() < 0.5:
            for _ in range(int(rng.integers(1, 6))):
                sch.step()
    sch.run_until_idle()
    assert len(sch.results) == 40
    reasons = set()
    for r in sch.results:
        prompt, new, temp, sd = reqs[r.seq_id]
        toks = list(r.token_ids)
        reasons.add(r.finish_reason)
        assert toks[:len(prompt)] == prompt and r.finish_reason in ("length", "capacity")
        gen = toks[len(prompt):]
        if r.finish_reason == "length":
            assert len(gen) == new
        else:  # pages ran out during the prompt or before the last token
            assert len(gen) < max(new, 1)
        if gen:
            check_stream(pc, pw, prompt, toks, TOL[dtype] if dtype == "bf16" else 5e-4, temperature=temp, seed=sd)
    assert reasons == {"length", "capacity"}
    eng.cm.check()
    assert eng.cm.free_pages(0) == n_pages and eng.cm.free_slots == 6
