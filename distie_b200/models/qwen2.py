"""Recipe of the Qwen2 dense decoder: typed configuration -> parts and run order.

Architecture of the reference's ``Qwen2CausalLM`` (worker/src/inference/qwen2/
model.py:293-314): token embedding; ``num_hidden_layers`` pre-norm blocks of
grouped-query attention (q/k/v with bias, output without, rotate-half RoPE) and a
SwiGLU feed-forward, RMSNorm before each; a final RMSNorm; a head that is the
embedding table when ``tie_word_embeddings``.  Tensor names are the checkpoint's
(model.py:386-400).  Every layer has its own cache slot and all share one need, so
the cache manager makes one group.
"""

from __future__ import annotations

from ..config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..config.qwen2_config import Qwen2Config
from ..config.registry import register_architecture


def qwen2_recipe(cfg: Qwen2Config) -> ModelSpec:
    position = PartSpec("rotary", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(
            LayerSpec(
                block="pre_norm",
                mixer=PartSpec(
                    "gqa_attention",
                    {
                        "num_heads": cfg.num_attention_heads,
                        "num_kv_heads": cfg.num_key_value_heads,
                        "head_dim": cfg.head_dim,
                        "qkv_bias": True,   # model.py:149-151
                        "out_bias": False,  # model.py:152
                        "window": None,     # sliding-window layers are rejected (model.py:58-60)
                        "position": position,
                    },
                    p + "self_attn.",
                ),
                feed_forward=PartSpec("swiglu", {"intermediate_size": cfg.intermediate_size}, p + "mlp."),
                norms={
                    "input": PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps}, p + "input_layernorm."),
                    "post_mixer": PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps}, p + "post_attention_layernorm."),
                },
            )
        )
    return ModelSpec(
        architecture="Qwen2ForCausalLM",
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        layers=tuple(layers),
        order=tuple(LayerCall(i, i, True) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps}, "model.norm."),
        embedding_name="model.embed_tokens.weight",
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        tolerated=("lm_head.weight",) if cfg.tie_word_embeddings else (),
        max_positions=cfg.max_position_embeddings,
        eos_token_id=cfg.eos_token_id,
    )


register_architecture("Qwen2ForCausalLM", Qwen2Config, qwen2_recipe)
