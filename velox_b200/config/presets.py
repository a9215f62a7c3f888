"""Named example configurations of the Qwen2.5 dense family, as ``config.json`` dictionaries.

They exist for runs with random weights (``--model-size`` of the benchmark command line): no
checkpoint is needed to time the layer sizes of a published model.  Nothing in the engine
reads them; a model folder's own ``config.json`` is what a model is built from.  The sizes are
those of the published Qwen2.5 checkpoints (0.5B ... 14B) and of two tiny test shapes.
"""
from __future__ import annotations

from typing import Any, Dict


def _qwen2(layers, hidden, heads, kv_heads, inter, vocab, tied, eps, max_pos=32768, theta=1000000.0,
           head_dim=None) -> Dict[str, Any]:
    cfg = {
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": layers,
        "hidden_size": hidden, "num_attention_heads": heads, "num_key_value_heads": kv_heads,
        "intermediate_size": inter, "vocab_size": vocab, "rope_theta": theta, "rms_norm_eps": eps,
        "tie_word_embeddings": tied, "use_sliding_window": False, "max_position_embeddings": max_pos,
        "hidden_act": "silu",
    }
    if head_dim is not None:
        cfg["head_dim"] = head_dim
    return cfg


MODEL_SIZES: Dict[str, Dict[str, Any]] = {
    "tiny-a": _qwen2(2, 64, 4, 2, 128, 256, True, 1e-6, max_pos=128, theta=10000.0, head_dim=16),
    "tiny-b": _qwen2(3, 256, 8, 1, 704, 512, False, 1e-5, max_pos=256, head_dim=32),
    "0.5b": _qwen2(24, 896, 14, 2, 4864, 151936, True, 1e-6),
    "1.5b": _qwen2(28, 1536, 12, 2, 8960, 151936, True, 1e-6),
    "3b": _qwen2(36, 2048, 16, 2, 11008, 151936, True, 1e-6),
    "7b": _qwen2(28, 3584, 28, 4, 18944, 152064, False, 1e-6),
    "14b": _qwen2(48, 5120, 40, 8, 13824, 152064, False, 1e-5),
}


def model_size(name: str) -> Dict[str, Any]:
    """A copy of the named configuration; KeyError lists the names."""
    try:
        return dict(MODEL_SIZES[name])
    except KeyError:
        raise KeyError(f"unknown model size {name!r}; known: {', '.join(sorted(MODEL_SIZES))}") from None
