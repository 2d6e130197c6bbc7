"""What another architecture would need of the shared code, shown with toy parts that are defined
HERE and registered without a change to the package (no GPU: the kernels are the CPU test double):
an embedding with a scale and a head with a soft cap as registered parts; how random weights are
drawn as a field of each tensor need; tensors a checkpoint may carry unread; one rotation table for
all layers that share a position spec; a mixer whose state can only be carried over at the edges of
chunks, so that the scheduler cuts prompts at multiples of the chunk."""
from dataclasses import dataclass, replace

import numpy as np
import pytest
import torch

import llmengine
import plain_llama as P
from cpu_ops import CpuOps
from llmengine.config import LlamaConfig
from llmengine.config.registry import Architecture, register_architecture
from llmengine.models.llama import describe_llama
from llmengine.parts import (Embedding, Head, Mixer, StateNeed, TensorNeed, part_class, register_part)
from llmengine.weights import (Checkpoint, WeightError, load_tensors, model_tensor_needs, random_tensors,
                               write_safetensors)
from tiny import TINY_A, random_ids


# ------------------------------------------------------------------ embedding and head as parts
@dataclass(frozen=True)
class ScaledLookupSpec:
    kind: str
    weight: str
    vocab_size: int
    dim: int
    scale: float


@dataclass(frozen=True)
class CappedHeadSpec:
    kind: str
    weight: str
    bias: str
    vocab_size: int
    dim: int
    cap: float


def _register_scaled_and_capped():
    class ScaledLookup(Embedding):
        @staticmethod
        def tensor_needs(spec):
            return [TensorNeed(spec.weight, (spec.vocab_size, spec.dim))]

        def load(self, tensors):
            self.table = tensors[self.spec.weight]

        def forward(self, ctx):
            h = ctx.ws.get("model.residual", (ctx.n_tokens, self.spec.dim), torch.float32)
            self.env.ops.embed(self.table, ctx.token_ids, h)
            return h.mul_(self.spec.scale)

    class CappedHead(Head):
        @staticmethod
        def tensor_needs(spec):
            return [TensorNeed(spec.weight, (spec.vocab_size, spec.dim)),
                    TensorNeed(spec.bias, (spec.vocab_size,), "float32", init="zeros")]

        def load(self, tensors):
            self.weight, self.bias = tensors[self.spec.weight], tensors[self.spec.bias]

        def forward(self, x, ctx):
            logits = ctx.ws.get("model.logits", (max(x.shape[0], 1), self.spec.vocab_size), torch.float32)[:x.shape[0]]
            if x.shape[0]:
                self.env.ops.gemm(x, self.weight, logits)
                logits.copy_(self.spec.cap * torch.tanh((logits + self.bias) / self.spec.cap))
            return logits

    register_part("embedding", "scaled_lookup", ScaledLookup, replace=True)
    register_part("head", "capped", CappedHead, replace=True)

    def describe(cfg):
        spec = describe_llama(cfg)
        return replace(spec, architecture="ToyScaledCapped",
                       embedding=ScaledLookupSpec("scaled_lookup", spec.embedding.weight, cfg.vocab_size, cfg.hidden_size,
                                                  float(np.sqrt(cfg.hidden_size))),
                       head=CappedHeadSpec("capped", "lm_head.weight", "lm_head.bias", cfg.vocab_size, cfg.hidden_size, 3.0))

    register_architecture(Architecture("ToyScaledCapped", LlamaConfig.from_dict, describe,
                                       lambda c: dict(c.to_dict(), architectures=["ToyScaledCapped"])), replace=True)


def test_embedding_and_head_are_registered_parts(tmp_path):
    _register_scaled_and_capped()
    cfg = dict(TINY_A, architectures=["ToyScaledCapped"])
    d = str(tmp_path / "m")
    llmengine.write_random_model(d, cfg, seed=2, dtype=torch.float32, std=0.05)
    pc, w = P.read_model(d)
    assert w["lm_head.bias"].shape == (256,) and not w["lm_head.bias"].any()  # init="zeros"
    w["lm_head.bias"] = np.linspace(-1, 1, 256).astype(np.float32)  # make the bias count
    t = {k: torch.from_numpy(v) for k, v in w.items()}
    write_safetensors(d + "/model.safetensors", t)
    ids = random_ids(19, 256, 3)
    # the plain model with the two variants: scale the table, cap the logits
    w2 = dict(w)
    w2["model.embed_tokens.weight"] = w["model.embed_tokens.weight"] * np.float32(np.sqrt(64))
    h = P.final_hidden(pc, w2, ids)
    ref = 3.0 * np.tanh((P.logits_at(pc, w2, h, None) + w["lm_head.bias"]) / 3.0)
    eng = llmengine.Engine(d, "fp32", device="cpu", ops=CpuOps(), block_size=4, num_blocks=16)
    np.testing.assert_allclose(eng.forward_logits(ids), ref, atol=2e-4, rtol=0)
    first = eng.run_step([(1, ids[:7], [6])]).clone()
    np.testing.assert_allclose(first.numpy(), ref[6:7], atol=2e-4, rtol=0)
    rest = eng.run_step([(1, ids[7:], range(12))], end=[1])
    np.testing.assert_allclose(rest.numpy(), ref[7:], atol=2e-4, rtol=0)
    out, reason = eng.generate(ids[:5], 4)
    assert len(out) == 9 and reason == "length"


# ------------------------------------------------------------------ weights
def test_how_a_tensor_is_drawn_is_a_field_of_its_need():
    spec = describe_llama(LlamaConfig.from_dict(TINY_A))
    needs = model_tensor_needs(spec)
    assert needs["model.norm.weight"].init == "around_one" and needs["model.embed_tokens.weight"].init == "normal"
    t = random_tensors(spec, 3, torch.float32)
    assert abs(float(t["model.layers.1.input_layernorm.weight"].mean()) - 1.0) < 0.02
    assert abs(float(t["model.layers.0.mlp.up_proj.weight"].mean())) < 0.01
    _register_scaled_and_capped()
    toy = llmengine.config.get_architecture("ToyScaledCapped").describe(LlamaConfig.from_dict(TINY_A))
    tt = random_tensors(toy, 3, torch.float32)
    assert not tt["lm_head.bias"].any()  # a float32 vector that is no norm weight: zeros, because its need says so


def test_tensors_a_checkpoint_may_carry_unread(tmp_path):
    spec = describe_llama(LlamaConfig.from_dict(TINY_A))
    t = random_tensors(spec, 1, torch.float32)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)  # what some exporters save
    t["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    needs = model_tensor_needs(spec)
    assert "*.rotary_emb.inv_freq" in spec.ignore
    got = load_tensors(Checkpoint(str(tmp_path)), needs, spec.duplicates, torch.device("cpu"), torch.float32, ignore=spec.ignore)
    assert set(got) == set(needs)
    with pytest.raises(WeightError, match="unexpected tensors \\(2\\)"):
        load_tensors(Checkpoint(str(tmp_path)), needs, spec.duplicates, torch.device("cpu"), torch.float32)
    t["model.layers.0.self_attn.other_buffer"] = torch.ones(2)  # still refused: no pattern names it
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    with pytest.raises(WeightError, match="unexpected tensors \\(1\\): model.layers.0.self_attn.other_buffer"):
        load_tensors(Checkpoint(str(tmp_path)), needs, spec.duplicates, torch.device("cpu"), torch.float32, ignore=spec.ignore)


def test_layers_that_share_a_position_spec_share_one_table(tmp_path):
    cfg = dict(TINY_A, num_hidden_layers=32, max_position_embeddings=4096)
    d = str(tmp_path / "m")
    llmengine.write_random_model(d, cfg, seed=1, dtype=torch.float32)
    eng = llmengine.Engine(d, "fp32", device="cpu", ops=CpuOps(), block_size=4, num_blocks=8)
    model = eng._ensure_model()
    tables = {(b.mixer.position.cos.data_ptr(), b.mixer.position.sin.data_ptr()) for b in model.blocks}
    assert len(model.blocks) == 32 and len(tables) == 1
    assert model.blocks[0].mixer.position.cos.shape == (4096, 8)


# ------------------------------------------------------------------ a mixer that is cut at chunk edges only
@dataclass(frozen=True)
class ChunkMeanSpec:
    kind: str
    hidden: int
    chunk: int
    weight: str


SEEN = []  # (first position, number of tokens) of every multi-token portion the toy mixer was handed


def _register_chunked():
    """out_t = W * (mean of the finished chunks of `chunk` tokens before t's chunk, plus x_t). Its state
    is the sum over finished chunks; inside a step it can only fold WHOLE chunks into that state, so a
    portion that leaves part of the prompt for later must end at a chunk edge. Single decoded tokens
    carry a partial chunk in a second state vector."""
    class ChunkMean(Mixer):
        capturable = False  # reads the batch on the host

        @staticmethod
        def tensor_needs(spec):
            return [TensorNeed(spec.weight, (spec.hidden, spec.hidden))]

        def cache_needs(self):
            m = self.spec.chunk
            return (StateNeed("done", (self.spec.hidden,), torch.float32, portion_multiple=m),
                    StateNeed("open", (self.spec.hidden,), torch.float32, portion_multiple=m))

        def load(self, tensors):
            self.w = tensors[self.spec.weight]

        def forward(self, x, ctx, cache):
            m, done, open_ = self.spec.chunk, cache.states["done"], cache.states["open"]
            out = torch.empty(ctx.n_tokens, self.spec.hidden, dtype=torch.float32)
            qoff, start, slot = ctx.seq_qoff.tolist(), ctx.seq_start.tolist(), ctx.seq_slot.tolist()
            for s in range(ctx.n_seqs):
                xs = x[qoff[s]:qoff[s + 1]].float()
                if xs.shape[0] > 1:
                    SEEN.append((start[s], xs.shape[0]))
                for i in range(xs.shape[0]):
                    pos = start[s] + i
                    n_done = pos // m
                    base = done[slot[s]] / max(n_done * m, 1)
                    out[qoff[s] + i] = (base + xs[i]) @ self.w.float().t()
                    open_[slot[s]] += xs[i]
                    if (pos + 1) % m == 0:  # the chunk is whole: fold it into the finished sum
                        done[slot[s]] += open_[slot[s]]
                        open_[slot[s]].zero_()
            return out

    register_part("mixer", "chunk_mean", ChunkMean, replace=True)

    def describe(cfg):
        spec = describe_llama(cfg)
        layers = list(spec.layers)
        layers[1] = replace(layers[1], mixer=ChunkMeanSpec("chunk_mean", cfg.hidden_size, 4, "model.layers.1.toy.weight"))
        return replace(spec, architecture="ToyChunked", layers=tuple(layers))

    register_architecture(Architecture("ToyChunked", LlamaConfig.from_dict, describe,
                                       lambda c: dict(c.to_dict(), architectures=["ToyChunked"])), replace=True)


def test_the_scheduler_cuts_prompts_where_the_models_state_allows(tmp_path):
    _register_chunked()
    cfg = dict(TINY_A, architectures=["ToyChunked"])
    d = str(tmp_path / "m")
    llmengine.write_random_model(d, cfg, seed=4, dtype=torch.float32, std=0.05)
    eng = llmengine.Engine(d, "fp32", device="cpu", ops=CpuOps(), block_size=4, num_blocks=48)
    assert eng._ensure_model().portion_multiple == 4 and not eng.model.capturable
    prompts = [random_ids(n, 256, 30 + n) for n in (23, 9, 14)]
    alone = [eng.generate(p, 5) for p in prompts]
    SEEN.clear()
    with pytest.raises(ValueError, match="portion multiple"):
        llmengine.ContinuousBatchScheduler(eng, None, max_concurrent=3, max_prefill_tokens_per_step=3)
    sch = llmengine.ContinuousBatchScheduler(eng, None, max_concurrent=3, max_prefill_tokens_per_step=10)
    for p in prompts:
        sch.enqueue(p, 5)
    sch.run_until_idle()
    # every portion started at a chunk edge, and some prompt was really cut
    assert SEEN and all(first % 4 == 0 for first, _ in SEEN)
    assert any(first > 0 for first, _ in SEEN)
    # cut that way, the chunked state gives each request what it gives it alone and whole
    for r, (toks, reason) in zip(sch.results, alone):
        assert list(r.token_ids) == toks and r.finish_reason == reason
    eng.cm.check()
