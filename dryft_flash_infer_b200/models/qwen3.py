"""The Qwen3 dense decoder as a ``ModelSpec``: which parts, in which order, under which names.

Tensor names are those of the checkpoint whose modules the reference walks
(engine/engine.py:163-176, :236-239): ``model.embed_tokens``, per layer
``input_layernorm``, ``self_attn.{q,k,v,o}_proj``, ``self_attn.{q,k}_norm``,
``post_attention_layernorm``, ``mlp.{gate,up,down}_proj``, then ``model.norm`` and, when
the embeddings are not tied, ``lm_head``.
"""

from __future__ import annotations

from ..config import Qwen3Config, register_architecture
from ..parts import LayerSpec, ModelSpec, PartSpec, straight_schedule


def build_qwen3(config: Qwen3Config) -> ModelSpec:
    norm = PartSpec("rms_norm", {"eps": config.rms_norm_eps})
    mixer = PartSpec("attention", {
        "n_heads": config.num_attention_heads,
        "n_kv_heads": config.num_key_value_heads,
        "head_dim": config.head_dim,
        "qk_norm": True,
        "qk_norm_eps": config.rms_norm_eps,
        "position": PartSpec("rotary", {"head_dim": config.head_dim, "theta": config.rope_theta}),
        "window": 0,
    })
    feed_forward = PartSpec("swiglu", {"intermediate_size": config.intermediate_size,
                                       "activation": config.hidden_act})
    layers = []
    for i in range(config.num_hidden_layers):
        p = f"model.layers.{i}."
        names = {
            "mixer_norm.weight": p + "input_layernorm.weight",
            "ffn_norm.weight": p + "post_attention_layernorm.weight",
            "mixer.q_proj": p + "self_attn.q_proj.weight",
            "mixer.k_proj": p + "self_attn.k_proj.weight",
            "mixer.v_proj": p + "self_attn.v_proj.weight",
            "mixer.o_proj": p + "self_attn.o_proj.weight",
            "mixer.q_norm": p + "self_attn.q_norm.weight",
            "mixer.k_norm": p + "self_attn.k_norm.weight",
            "feed_forward.gate_proj": p + "mlp.gate_proj.weight",
            "feed_forward.up_proj": p + "mlp.up_proj.weight",
            "feed_forward.down_proj": p + "mlp.down_proj.weight",
        }
        layers.append(LayerSpec("pre_norm", mixer, feed_forward, {"mixer_norm": norm, "ffn_norm": norm}, names))
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab_size,
        hidden_size=config.hidden_size,
        max_positions=config.max_position_embeddings,
        layers=tuple(layers),
        schedule=straight_schedule(config.num_hidden_layers),
        final_norm=norm,
        embedding_name="model.embed_tokens.weight",
        final_norm_names={"weight": "model.norm.weight"},
        head_name=None if config.tie_word_embeddings else "lm_head.weight",
        # a tied model's file may still carry a copy of the head: it is the embedding, so it is skipped
        ignorable_tensors=("lm_head.weight",) if config.tie_word_embeddings else (),
    )


register_architecture(Qwen3Config.architecture, Qwen3Config, build_qwen3)
