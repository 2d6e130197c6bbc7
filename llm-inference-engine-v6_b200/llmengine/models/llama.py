"""The Llama dense GQA decoder ("LlamaForCausalLM") as a description in parts.

Tensor names, shapes and the layer structure are those the reference reads (src/model.cpp:179-287):
model.embed_tokens.weight [V,H]; per layer input_layernorm / post_attention_layernorm [H],
self_attn.{q,k,v,o}_proj.weight, mlp.{gate,up,down}_proj.weight; model.norm.weight [H];
lm_head.weight [V,H], which is the embedding itself when tie_word_embeddings is set
(src/weights.cpp:244-267, src/model.cpp:184-195).
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, LayerRun, ModelSpec,
                          NormSpec, PositionSpec)


def describe_llama(cfg: LlamaConfig) -> ModelSpec:
    s = cfg.rope_scaling
    position = PositionSpec(kind="rope", head_dim=cfg.head_dim, theta=cfg.rope_theta,
                            max_positions=cfg.max_position_embeddings,
                            scaling_factor=s.factor if s else 1.0,
                            low_freq_factor=s.low_freq_factor if s else 1.0,
                            high_freq_factor=s.high_freq_factor if s else 1.0,
                            original_max_positions=s.original_max_position_embeddings if s else 0)
    layers = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        layers.append(BlockSpec(
            kind="pre_norm",
            norm1=NormSpec("rmsnorm", cfg.hidden_size, cfg.rms_norm_eps, p + "input_layernorm.weight"),
            mixer=AttentionSpec(kind="attention", hidden=cfg.hidden_size, num_heads=cfg.num_attention_heads,
                                num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, position=position,
                                q_weight=p + "self_attn.q_proj.weight", k_weight=p + "self_attn.k_proj.weight",
                                v_weight=p + "self_attn.v_proj.weight", o_weight=p + "self_attn.o_proj.weight"),
            norm2=NormSpec("rmsnorm", cfg.hidden_size, cfg.rms_norm_eps, p + "post_attention_layernorm.weight"),
            feed_forward=GatedMLPSpec(kind="gated_mlp", hidden=cfg.hidden_size, intermediate=cfg.intermediate_size,
                                      gate_weight=p + "mlp.gate_proj.weight", up_weight=p + "mlp.up_proj.weight",
                                      down_weight=p + "mlp.down_proj.weight"),
        ))
    embed_name = "model.embed_tokens.weight"
    tied = cfg.tie_word_embeddings
    return ModelSpec(
        architecture=cfg.architecture,
        embedding=EmbeddingSpec(embed_name, cfg.vocab_size, cfg.hidden_size),
        layers=tuple(layers),
        order=tuple(LayerRun(l) for l in range(cfg.num_hidden_layers)),
        final_norm=NormSpec("rmsnorm", cfg.hidden_size, cfg.rms_norm_eps, "model.norm.weight"),
        head=HeadSpec(embed_name if tied else "lm_head.weight", cfg.vocab_size, cfg.hidden_size),
        max_positions=cfg.max_position_embeddings,
        eos_token_ids=cfg.eos_token_ids,
        duplicates={"lm_head.weight": embed_name} if tied else {},
        # buffers that exporters of this architecture save beside the weights and nobody reads
        ignore=("*.rotary_emb.inv_freq",),
    )


LLAMA = Architecture(name="LlamaForCausalLM", parse_config=LlamaConfig.from_dict, describe=describe_llama,
                     config_to_json=lambda cfg: cfg.to_dict())
register_architecture(LLAMA, replace=True)
