"""LlamaForCausalLM as a description in parts.

Embedding; L x (RMSNorm, grouped-query attention with rotary encoding, add,
RMSNorm, SwiGLU, add); RMSNorm; head, tied to the embedding when
``tie_word_embeddings`` is set (crates/vllm-models/src/llama/architecture.rs:11-165;
tensor names :25-28,75-77,102-118 and crates/vllm-models/src/llama/attention.rs:47-66).
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def llama_model_spec(c: LlamaConfig) -> ModelSpec:
    scaling = None
    if c.rope_scaling is not None:
        s = c.rope_scaling
        scaling = dict(factor=s.factor, low_freq_factor=s.low_freq_factor, high_freq_factor=s.high_freq_factor,
                       original_max_position_embeddings=s.original_max_position_embeddings)
    position = PartSpec("rope", dict(head_dim=c.head_dim, theta=c.rope_theta, scaling=scaling,
                                     max_position=c.max_position_embeddings))
    mixer = PartSpec("paged_attention", dict(
        hidden_size=c.hidden_size, num_heads=c.num_attention_heads, num_kv_heads=c.num_key_value_heads,
        head_dim=c.head_dim, window=0, scale=None, position=position))
    ffn = PartSpec("swiglu", dict(hidden_size=c.hidden_size, intermediate_size=c.intermediate_size))
    layers = tuple(
        LayerSpec(
            prefix=f"model.layers.{i}.",
            mixer=mixer,
            mixer_norm=PartSpec("rmsnorm", dict(size=c.hidden_size, eps=c.rms_norm_eps, name="input_layernorm.weight")),
            ffn=ffn,
            ffn_norm=PartSpec("rmsnorm", dict(size=c.hidden_size, eps=c.rms_norm_eps,
                                              name="post_attention_layernorm.weight")),
            arrangement="prenorm")
        for i in range(c.num_hidden_layers))
    embed_name = "model.embed_tokens.weight"
    return ModelSpec(
        hidden_size=c.hidden_size, vocab_size=c.vocab_size, max_position=c.max_position_embeddings,
        embedding=PartSpec("token_embedding", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size,
                                                   name=embed_name)),
        layers=layers,
        final_norm=PartSpec("rmsnorm", dict(size=c.hidden_size, eps=c.rms_norm_eps, name="model.norm.weight")),
        head=PartSpec("lm_head", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size,
                                      name=embed_name if c.tie_word_embeddings else "lm_head.weight")),
    )


LLAMA = register_architecture(Architecture(
    name="LlamaForCausalLM",
    config_from_dict=LlamaConfig.from_dict,
    model_spec=llama_model_spec,
    description="dense grouped-query decoder with rotary encoding and SwiGLU",
    family="Llama",
    allow_unexpected=lambda c: ("lm_head.weight",) if c.tie_word_embeddings else (),
), replace=True)
