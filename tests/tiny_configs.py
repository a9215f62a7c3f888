"""Tiny configurations for tests: config.json dicts that differ in every size and option.

tiny-A and tiny-B are the two tiny sizes the benchmark description names; tiny-W adds a sliding
window on its upper layers, a head size that is not a power of two and a vocabulary and width
that are not powers of two either.
"""
from __future__ import annotations

from typing import Any, Dict

TINY_A: Dict[str, Any] = {
    "architectures": ["Qwen2ForCausalLM"],
    "model_type": "qwen2",
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "intermediate_size": 128,
    "vocab_size": 256,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True,
    "use_sliding_window": False,
    "max_position_embeddings": 128,
    "hidden_act": "silu",
}

TINY_B: Dict[str, Any] = {
    "architectures": ["Qwen2ForCausalLM"],
    "model_type": "qwen2",
    "num_hidden_layers": 3,
    "hidden_size": 256,
    "num_attention_heads": 8,
    "num_key_value_heads": 1,
    "intermediate_size": 704,
    "vocab_size": 512,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "use_sliding_window": False,
    "max_position_embeddings": 256,
    "hidden_act": "silu",
}

# Width 240 = 5 heads x 48, 5 query heads on 5 KV heads (no grouping), vocabulary 331,
# intermediate 200, window 24 on layers 1.. (layer 0 sees every key), linear RoPE scaling.
TINY_W: Dict[str, Any] = {
    "architectures": ["Qwen2ForCausalLM"],
    "model_type": "qwen2",
    "num_hidden_layers": 4,
    "hidden_size": 240,
    "num_attention_heads": 5,
    "num_key_value_heads": 5,
    "head_dim": 48,
    "intermediate_size": 200,
    "vocab_size": 331,
    "rope_theta": 50000.0,
    "rope_scaling": {"type": "linear", "factor": 2.0},
    "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False,
    "use_sliding_window": True,
    "sliding_window": 24,
    "max_window_layers": 1,
    "max_position_embeddings": 512,
    "hidden_act": "silu",
}

# Head size 80 with hidden size that is not heads x head_dim (head_dim given explicitly),
# group of 3 query heads per KV head.
TINY_C: Dict[str, Any] = {
    "architectures": ["Qwen2ForCausalLM"],
    "model_type": "qwen2",
    "num_hidden_layers": 2,
    "hidden_size": 136,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 80,
    "intermediate_size": 312,
    "vocab_size": 1000,
    "rope_theta": 300000.0,
    "rms_norm_eps": 1e-4,
    "tie_word_embeddings": True,
    "use_sliding_window": False,
    "max_position_embeddings": 640,
    "hidden_act": "silu",
}

# Heads of 128 dims, three query heads per KV head: the shapes that take the decode fast paths
# (rotation and cache write in the QKV projection's epilogue, norm made inside the projections,
# tensor-map K/V tiles, a thread-block cluster per sequence and KV head).  Width 768 = 6 x 128.
TINY_D: Dict[str, Any] = {
    "architectures": ["Qwen2ForCausalLM"],
    "model_type": "qwen2",
    "num_hidden_layers": 2,
    "hidden_size": 768,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "intermediate_size": 1048,
    "vocab_size": 777,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False,
    "use_sliding_window": False,
    "max_position_embeddings": 1536,
    "hidden_act": "silu",
}

ALL = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_w": TINY_W, "tiny_c": TINY_C, "tiny_d": TINY_D}
