"""The dense Llama decoder as a `ModelSpec`.

Layer make-up and order follow the reference's forward pass
(src/model/arch/llama.rs:158-246): RMSNorm -> grouped-query attention with
rotary positions -> residual; RMSNorm -> SwiGLU feed-forward -> residual; a
final RMSNorm and an output matrix that may be the embedding (src/model.rs:175-177).
Tensor names are the checkpoint-folder convention; they map one to one onto
the reference's GGUF names (src/model/arch/llama.rs:97-128).
"""
from __future__ import annotations

from ..registry import ARCHITECTURES
from ..spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .llama import LlamaConfig


def describe_llama(c: LlamaConfig) -> ModelSpec:
    position = PartSpec("rotary", dict(
        head_dim=c.head_dim, rotary_dim=c.head_dim, theta=c.rope_theta, layout=c.rope_layout,
        scaling=c.rope_scaling, max_positions=c.max_position_embeddings))
    layers = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            block="prenorm",
            mixer_norm=PartSpec("rmsnorm", dict(width=c.hidden_size, eps=c.rms_norm_eps),
                                prefix=p + "input_layernorm."),
            mixer=PartSpec("attention", dict(
                hidden_size=c.hidden_size, num_heads=c.num_attention_heads,
                num_kv_heads=c.num_key_value_heads, head_dim=c.head_dim,
                scale=c.head_dim ** -0.5, window=0, position=position),
                prefix=p + "self_attn."),
            ffn_norm=PartSpec("rmsnorm", dict(width=c.hidden_size, eps=c.rms_norm_eps),
                              prefix=p + "post_attention_layernorm."),
            ffn=PartSpec("gated_mlp", dict(hidden_size=c.hidden_size,
                                           intermediate_size=c.intermediate_size,
                                           activation="silu"),
                         prefix=p + "mlp."),
        ))
    embedding = PartSpec("embedding", dict(vocab_size=c.vocab_size, width=c.hidden_size),
                         prefix="model.embed_tokens.")
    lm_head = PartSpec("lm_head", dict(vocab_size=c.vocab_size, width=c.hidden_size),
                       prefix="lm_head.")
    if c.tie_word_embeddings:
        lm_head.aliases["weight"] = embedding.tensor_name("weight")
    return ModelSpec(
        hidden_size=c.hidden_size,
        vocab_size=c.vocab_size,
        max_positions=c.max_position_embeddings,
        embedding=embedding,
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(c.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", dict(width=c.hidden_size, eps=c.rms_norm_eps),
                            prefix="model.norm."),
        lm_head=lm_head,
        stop_token_ids=tuple(c.eos_token_id),
    )


def _register() -> None:
    from . import Architecture
    for name in ("LlamaForCausalLM", "llama"):
        ARCHITECTURES.register(name, Architecture(name, LlamaConfig.from_dict, describe_llama),
                               replace=True)


_register()
