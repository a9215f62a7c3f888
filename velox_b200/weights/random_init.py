"""Random-weights mode: write a model folder from a configuration and a seed.

The folder holds ``config.json`` and ``model.safetensors`` under the architecture's own tensor
names, so it loads through the same by-name loader as a real checkpoint (and through any other
engine that reads the format).  The reference has no such mode; it always reads a downloaded
checkpoint (src/weight_loader.py:139-155).

Every tensor is drawn from its own generator, keyed by (seed, tensor name), so a tensor's
values do not depend on which other tensors exist or on the order they are made in.  Matrices
and biases are N(0, std); norm weights are 1 + N(0, std) so that a missing norm multiply shows.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Mapping, Optional, Union

import torch

from ..config.model_config import ModelConfig
from ..config.registry import architecture_of, get_architecture
from ..parts.spec import ModelSpec, TensorSource

_STORE_DTYPES = {
    "bfloat16": torch.bfloat16,
    "bf16": torch.bfloat16,
    "float32": torch.float32,
    "fp32": torch.float32,
}


def tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensor(source: TensorSource, seed: int, std: float, dtype: torch.dtype) -> torch.Tensor:
    generator = torch.Generator(device="cpu")
    generator.manual_seed(tensor_seed(seed, source.name))
    values = torch.empty(source.shape, dtype=torch.float32)
    values.normal_(0.0, std, generator=generator)
    if source.init == "one_plus_normal":
        values += 1.0
    elif source.init != "normal":
        raise ValueError(f"unknown init {source.init!r} for {source.name}")
    return values.to(dtype)


def random_state_dict(
    spec: ModelSpec, seed: int, std: float = 0.02, dtype: torch.dtype = torch.bfloat16
) -> Dict[str, torch.Tensor]:
    return {
        name: random_tensor(source, seed, std, dtype)
        for name, source in sorted(spec.checkpoint_tensors().items())
    }


def write_random_model(
    model_dir: str,
    config: Union[ModelConfig, Mapping[str, Any]],
    seed: int,
    dtype: str = "bfloat16",
    std: float = 0.02,
    spec: Optional[ModelSpec] = None,
) -> ModelSpec:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` under ``model_dir``.

    ``config`` is a typed configuration or the dict of a config.json (its ``architectures``
    entry picks the model, as everywhere).  ``dtype`` is the storage dtype of the file.
    """
    from safetensors.torch import save_file

    if dtype not in _STORE_DTYPES:
        raise ValueError(f"unknown storage dtype {dtype!r}; expected one of {sorted(_STORE_DTYPES)}")
    if isinstance(config, ModelConfig):
        typed = config
        arch = get_architecture(typed.architecture)
    else:
        arch = architecture_of(config)
        typed = arch.parse_config(config)
    if spec is None:
        spec = arch.build_spec(typed)

    os.makedirs(model_dir, exist_ok=True)
    config_json = dict(typed.to_json_dict())
    config_json["torch_dtype"] = "bfloat16" if _STORE_DTYPES[dtype] is torch.bfloat16 else "float32"
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(config_json, handle, indent=1, sort_keys=True)
    tensors = random_state_dict(spec, seed, std=std, dtype=_STORE_DTYPES[dtype])
    save_file(tensors, os.path.join(model_dir, "model.safetensors"), metadata={"format": "pt"})
    return spec
