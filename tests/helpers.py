"""Shared helpers of the tests: model folders in temporary places, prompts, tensors by name."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Sequence

import torch


def write_model(folder: str, cfg: Dict[str, Any], seed: int, dtype: str = "float32") -> None:
    from velox_b200.weights import write_random_model

    write_random_model(folder, cfg, seed=seed, dtype=dtype)


def read_tensors(folder: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return load_file(os.path.join(folder, "model.safetensors"))


def read_config(folder: str) -> Dict[str, Any]:
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as handle:
        return json.load(handle)


def random_prompt(vocab: int, length: int, seed: int) -> List[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=gen).tolist()


def random_prompts(vocab: int, lengths: Sequence[int], seed: int) -> List[List[int]]:
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in lengths]
