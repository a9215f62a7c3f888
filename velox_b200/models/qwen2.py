"""``Qwen2ForCausalLM`` (Qwen2.5 dense) as a model spec.

What the architecture is, in the reference's own modules: token embedding, N pre-norm decoder
layers, final RMSNorm, a bias-free lm_head that shares the embedding when
``tie_word_embeddings`` is set (src/transformer.py:14-68).  A layer is
``h += attn(rms(h)); h += mlp(rms(h))`` (src/decoder_layer.py:34-54); attention has q/k/v
biases and none on the output projection (src/decoder_layer.py:28, src/self_attention.py:32-33),
rotate-half RoPE on q and k (src/rope.py:45-63) and grouped KV heads; the MLP is
``down(silu(gate(x)) * up(x))`` without biases (src/mlp.py:9-15).

The q/k/v and gate/up checkpoint tensors are concatenated along dim 0, in that order, as
src/weight_loader.py:71-98 does; the order defines the column layout the attention and SwiGLU
parts assume.

This module only maps configuration keys to part parameters and checkpoint names to part
weights.  It has no forward pass.
"""
from __future__ import annotations

from typing import Dict, Optional

from ..config.model_config import ModelConfig, Qwen2Config
from ..config.registry import register_architecture
from ..parts.spec import (
    LayerSpec,
    ModelSpec,
    PartSpec,
    ScheduleEntry,
    TensorSource,
    WeightSpec,
)

ARCHITECTURE = "Qwen2ForCausalLM"

# End-of-sequence ids of the Qwen2.5 vocabulary, for a folder whose config.json and
# generation_config.json name none: what the reference falls back to (engine/engine.py:23).
DEFAULT_EOS_TOKEN_IDS = (151643, 151645)


def _matrix(*sources: TensorSource) -> WeightSpec:
    return WeightSpec(sources=tuple(sources), role="matrix")


def _vector(*sources: TensorSource) -> WeightSpec:
    return WeightSpec(sources=tuple(sources), role="vector")


def _rms(name: str, size: int, eps: float) -> PartSpec:
    return PartSpec(
        kind="rms",
        params={"size": size, "eps": eps},
        weights={"weight": _vector(TensorSource(name, (size,), init="one_plus_normal"))},
    )


def build_qwen2_spec(config: ModelConfig) -> ModelSpec:
    if not isinstance(config, Qwen2Config):
        raise TypeError(f"expected a Qwen2Config, got {type(config).__name__}")
    c = config
    E, H, G, D, I, V = (
        c.hidden_size,
        c.num_attention_heads,
        c.num_key_value_heads,
        c.head_dim,
        c.intermediate_size,
        c.vocab_size,
    )

    position = PartSpec(
        kind="rotary_half",
        params={
            "head_dim": D,
            "rotary_dim": D,
            "theta": c.rope_theta,
            "scaling_factor": c.rope_scaling_factor,
            "max_position": c.max_position_embeddings,
        },
    )

    layers = []
    for index in range(c.num_hidden_layers):
        p = f"model.layers.{index}."
        window: Optional[int] = c.layer_window(index)
        attention_weights: Dict[str, WeightSpec] = {
            "qkv.weight": _matrix(
                TensorSource(p + "self_attn.q_proj.weight", (H * D, E)),
                TensorSource(p + "self_attn.k_proj.weight", (G * D, E)),
                TensorSource(p + "self_attn.v_proj.weight", (G * D, E)),
            ),
            "qkv.bias": _vector(
                TensorSource(p + "self_attn.q_proj.bias", (H * D,)),
                TensorSource(p + "self_attn.k_proj.bias", (G * D,)),
                TensorSource(p + "self_attn.v_proj.bias", (G * D,)),
            ),
            "out.weight": _matrix(TensorSource(p + "self_attn.o_proj.weight", (E, H * D))),
        }
        mixer = PartSpec(
            kind="attention",
            params={
                "hidden_size": E,
                "num_heads": H,
                "num_kv_heads": G,
                "head_dim": D,
                "qkv_bias": True,
                "window": window,
                # src/self_attention.py:35
                "softmax_scale": 1.0 / (D ** 0.5),
            },
            weights=attention_weights,
        )
        feed_forward = PartSpec(
            kind="swiglu",
            params={"hidden_size": E, "intermediate_size": I},
            weights={
                "gate_up.weight": _matrix(
                    TensorSource(p + "mlp.gate_proj.weight", (I, E)),
                    TensorSource(p + "mlp.up_proj.weight", (I, E)),
                ),
                "down.weight": _matrix(TensorSource(p + "mlp.down_proj.weight", (E, I))),
            },
        )
        layers.append(
            LayerSpec(
                block="pre_norm",
                mixer=mixer,
                feed_forward=feed_forward,
                norms={
                    "mixer": _rms(p + "input_layernorm.weight", E, c.rms_norm_eps),
                    "feed_forward": _rms(p + "post_attention_layernorm.weight", E, c.rms_norm_eps),
                },
                position=position,
            )
        )

    embed_source = TensorSource("model.embed_tokens.weight", (V, E))
    head_source = embed_source if c.tie_word_embeddings else TensorSource("lm_head.weight", (V, E))
    spec = ModelSpec(
        architecture=c.architecture,
        hidden_size=E,
        vocab_size=V,
        max_position=c.max_position_embeddings,
        embedding=PartSpec(
            kind="token_embedding",
            params={"vocab_size": V, "hidden_size": E},
            weights={"weight": _matrix(embed_source)},
        ),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i) for i in range(c.num_hidden_layers)),
        final_norm=_rms("model.norm.weight", E, c.rms_norm_eps),
        lm_head=PartSpec(
            kind="linear_head",
            params={"hidden_size": E, "vocab_size": V},
            weights={"weight": _matrix(head_source)},
        ),
        eos_token_ids=tuple(c.eos_token_ids) or DEFAULT_EOS_TOKEN_IDS,
        # A tied checkpoint may still store a copy of the head; it is not read.
        ignored_tensors=("lm_head.weight",) if c.tie_word_embeddings else (),
    )
    spec.validate()
    return spec


register_architecture(ARCHITECTURE, Qwen2Config.from_dict, build_qwen2_spec)
