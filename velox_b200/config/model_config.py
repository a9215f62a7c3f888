"""Typed model configuration, read from an architecture's own ``config.json`` keys.

Every size and constant of a model comes from here; no kernel, part or engine module carries a
model size of its own.  The field list follows the reference's ``ModelConfig``
(src/config.py:6-42) and adds the keys the reference leaves implicit: ``head_dim`` (the
reference derives it as ``hidden_size // num_attention_heads``, src/transformer.py:19),
``hidden_act`` (fixed to SiLU in src/mlp.py:15) and the sliding-window keys that Qwen2
checkpoints carry and the reference never reads.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the offending key named."""


def _require(cfg: Mapping[str, Any], key: str) -> Any:
    if key not in cfg or cfg[key] is None:
        raise ConfigError(f"config.json is missing required key {key!r}")
    return cfg[key]


def _positive_int(cfg: Mapping[str, Any], key: str, default: Optional[int] = None) -> int:
    value = cfg.get(key)
    if value is None:
        value = default if default is not None else _require(cfg, key)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json key {key!r} must be a positive integer, got {value!r}")
    return value


@dataclass(frozen=True)
class ModelConfig:
    """Fields shared by every architecture; an architecture subclasses this with its own keys."""

    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    max_position_embeddings: int
    tie_word_embeddings: bool
    eos_token_ids: Tuple[int, ...] = ()

    def to_json_dict(self) -> Dict[str, Any]:  # pragma: no cover - overridden
        raise NotImplementedError


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    """``Qwen2ForCausalLM``: dense decoder, q/k/v bias, SwiGLU, pre-RMSNorm, rotate-half RoPE.

    Defaults of absent keys follow src/config.py:29-42: ``num_key_value_heads`` falls back to
    ``num_attention_heads``, ``rms_norm_eps`` to ``layer_norm_eps`` then 1e-6,
    ``max_position_embeddings`` to ``seq_length`` then 4096, ``rope_theta`` to 10000 and
    ``tie_word_embeddings`` to False.
    """

    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    # Linear position scaling only (positions are divided by this), as in src/rope.py:11-18.
    rope_scaling_factor: float = 1.0
    hidden_act: str = "silu"
    # Window of keys a query may see (itself included) in the layers that use one; None = all keys.
    sliding_window: Optional[int] = None
    # Layers with index >= max_window_layers use the window when it is enabled.
    max_window_layers: int = 0
    torch_dtype: str = "bfloat16"

    # ------------------------------------------------------------------ derived
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer: int) -> Optional[int]:
        """Key window of one layer: the first ``max_window_layers`` layers see every key."""
        if self.sliding_window is None or layer < self.max_window_layers:
            return None
        return self.sliding_window

    # ------------------------------------------------------------------ parsing
    @staticmethod
    def from_dict(cfg: Mapping[str, Any]) -> "Qwen2Config":
        archs = cfg.get("architectures") or ["Qwen2ForCausalLM"]
        hidden = _positive_int(cfg, "hidden_size")
        heads = _positive_int(cfg, "num_attention_heads")
        kv_heads = _positive_int(cfg, "num_key_value_heads", heads)
        if cfg.get("head_dim") is not None:
            head_dim = _positive_int(cfg, "head_dim")
        else:
            if hidden % heads != 0:
                raise ConfigError(
                    f"hidden_size={hidden} is not divisible by num_attention_heads={heads} "
                    "and config.json gives no head_dim"
                )
            head_dim = hidden // heads
        if heads % kv_heads != 0:
            raise ConfigError(
                f"num_attention_heads={heads} must be a multiple of num_key_value_heads={kv_heads}"
            )
        if head_dim % 2 != 0:
            raise ConfigError(f"head_dim={head_dim} must be even for rotate-half RoPE")

        act = cfg.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act={act!r} is not supported (Qwen2 uses 'silu')")

        scaling = cfg.get("rope_scaling")
        factor = 1.0
        if scaling:
            kind = scaling.get("type") or scaling.get("rope_type")
            if kind in (None, "default"):
                factor = 1.0
            elif kind == "linear":
                factor = float(scaling.get("factor", 1.0))
                if not factor > 0.0:
                    raise ConfigError(f"rope_scaling.factor must be positive, got {factor}")
            else:
                raise ConfigError(
                    f"rope_scaling type {kind!r} is not supported (only 'linear' is); "
                    "refusing to run with wrong rotation angles"
                )

        window: Optional[int] = None
        layers = _positive_int(cfg, "num_hidden_layers")
        max_window_layers = layers
        if cfg.get("use_sliding_window", False):
            window = _positive_int(cfg, "sliding_window")
            max_window_layers = int(cfg.get("max_window_layers", layers))
            if max_window_layers < 0:
                raise ConfigError("max_window_layers must be non-negative")

        eps = cfg.get("rms_norm_eps", cfg.get("layer_norm_eps", 1e-6))
        max_pos = cfg.get("max_position_embeddings", cfg.get("seq_length", 4096))
        eos = cfg.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        else:
            eos_ids = tuple(int(t) for t in eos)

        return Qwen2Config(
            architecture=str(archs[0]),
            vocab_size=_positive_int(cfg, "vocab_size"),
            hidden_size=hidden,
            num_hidden_layers=layers,
            max_position_embeddings=int(max_pos),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            eos_token_ids=eos_ids,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=_positive_int(cfg, "intermediate_size"),
            rms_norm_eps=float(eps),
            rope_theta=float(cfg.get("rope_theta", 10000.0)),
            rope_scaling_factor=factor,
            hidden_act=act,
            sliding_window=window,
            max_window_layers=max_window_layers,
            torch_dtype=str(cfg.get("torch_dtype", cfg.get("dtype", "bfloat16"))),
        )

    def to_json_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        out: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen2",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": (
                None
                if self.rope_scaling_factor == 1.0
                else {"type": "linear", "factor": self.rope_scaling_factor}
            ),
            "hidden_act": self.hidden_act,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": self.sliding_window is not None,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "torch_dtype": self.torch_dtype,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in {model_dir}")
    with open(path, "r", encoding="utf-8") as handle:
        cfg = json.load(handle)
    if not isinstance(cfg, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return cfg
