"""Weights from safetensors, by checkpoint tensor name.

What is read and how it is put together is not decided here: the model spec names, for every
weight of every part, the checkpoint tensors it is made of (several are concatenated along
dim 0, which is how q/k/v and gate/up become one matrix, as src/weight_loader.py:71-98 of the
reference does for its one architecture).

Storage on the device follows the weight's role: a "matrix" is kept in the compute dtype
(bfloat16 when serving; float32 in the 32-bit path), a "vector" (norm weights, biases) is
always float32 -- a bfloat16 value widens exactly and a tensor stored in 32-bit keeps its
bits -- and a "table" of integers is int32.

Errors: one ``WeightError`` lists every missing tensor, every unexpected tensor and every
tensor of the wrong shape (the reference raises on the first of each kind,
src/weight_loader.py:88-89,123-126,131-132, and only prints unexpected tensors).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from ..parts.spec import ModelSpec, WeightSpec

_SINGLE_FILE = "model.safetensors"
_INDEX_FILE = "model.safetensors.index.json"

_INTEGER_DTYPES = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8, torch.bool)


class WeightError(RuntimeError):
    """The checkpoint does not hold what the model spec reads."""

    def __init__(
        self,
        model_dir: str,
        missing: List[str],
        unexpected: List[str],
        wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
    ) -> None:
        self.missing = missing
        self.unexpected = unexpected
        self.wrong_shape = wrong_shape
        lines = [f"checkpoint in {model_dir} does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}):")
            for name, found, wanted in wrong_shape:
                lines.append(f"    {name}: checkpoint {tuple(found)}, model {tuple(wanted)}")
        super().__init__("\n".join(lines))


class Checkpoint:
    """The safetensors files of a model folder, read lazily one tensor at a time."""

    def __init__(self, model_dir: str) -> None:
        from safetensors import safe_open

        self.model_dir = model_dir
        self._files: Dict[str, str] = {}
        self._handles: Dict[str, object] = {}
        for path in _list_shards(model_dir):
            handle = safe_open(path, framework="pt", device="cpu")
            self._handles[path] = handle
            for name in handle.keys():
                self._files[name] = path
        if not self._files:
            raise RuntimeError(f"checkpoint in {model_dir} contains no tensors")

    def names(self) -> List[str]:
        return sorted(self._files)

    def __contains__(self, name: str) -> bool:
        return name in self._files

    def shape(self, name: str) -> Tuple[int, ...]:
        handle = self._handles[self._files[name]]
        return tuple(handle.get_slice(name).get_shape())

    def get(self, name: str) -> torch.Tensor:
        return self._handles[self._files[name]].get_tensor(name)


def _list_shards(model_dir: str) -> List[str]:
    if not os.path.isdir(model_dir):
        raise FileNotFoundError(f"model folder {model_dir} does not exist")
    index_path = os.path.join(model_dir, _INDEX_FILE)
    if os.path.exists(index_path):
        with open(index_path, "r", encoding="utf-8") as handle:
            index = json.load(handle)
        names = sorted(set(index["weight_map"].values()))
        return [os.path.join(model_dir, name) for name in names]
    single = os.path.join(model_dir, _SINGLE_FILE)
    if os.path.exists(single):
        return [single]
    raise FileNotFoundError(f"no safetensors weights found in {model_dir}")


def check_checkpoint(checkpoint: Checkpoint, spec: ModelSpec) -> None:
    """Raise one ``WeightError`` naming everything that does not match the spec."""
    wanted = spec.checkpoint_tensors()
    missing = [name for name in sorted(wanted) if name not in checkpoint]
    ignored = set(spec.ignored_tensors)
    unexpected = [
        name for name in checkpoint.names() if name not in wanted and name not in ignored
    ]
    wrong = []
    for name in sorted(wanted):
        if name in checkpoint:
            found = checkpoint.shape(name)
            if tuple(found) != tuple(wanted[name].shape):
                wrong.append((name, tuple(found), tuple(wanted[name].shape)))
    if missing or unexpected or wrong:
        raise WeightError(checkpoint.model_dir, missing, unexpected, wrong)


def storage_dtype(role: str, compute_dtype: torch.dtype) -> torch.dtype:
    if role == "matrix":
        return compute_dtype
    if role == "vector":
        return torch.float32
    if role == "table":
        return torch.int32
    raise ValueError(f"unknown weight role {role!r}")


class WeightStore:
    """Builds the device tensor of each ``WeightSpec``; the same sources give the same tensor.

    Sharing by source names is what makes a tied lm_head and the embedding one buffer.
    """

    def __init__(
        self,
        checkpoint: Checkpoint,
        spec: ModelSpec,
        compute_dtype: torch.dtype,
        device: torch.device | str,
    ) -> None:
        check_checkpoint(checkpoint, spec)
        self.checkpoint = checkpoint
        self.compute_dtype = compute_dtype
        self.device = torch.device(device)
        self._cache: Dict[Tuple[Tuple[str, ...], torch.dtype], torch.Tensor] = {}
        self.num_bytes = 0

    def load(self, weight: WeightSpec) -> torch.Tensor:
        dtype = storage_dtype(weight.role, self.compute_dtype)
        key = (tuple(src.name for src in weight.sources), dtype)
        cached = self._cache.get(key)
        if cached is not None:
            return cached
        pieces = []
        for src in weight.sources:
            tensor = self.checkpoint.get(src.name)
            if weight.role == "table" and tensor.dtype not in _INTEGER_DTYPES:
                raise TypeError(f"{src.name} feeds an integer table but is stored as {tensor.dtype}")
            pieces.append(tensor.to(device=self.device, dtype=dtype))
        fused = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=0)
        fused = fused.contiguous()
        self._cache[key] = fused
        self.num_bytes += fused.numel() * fused.element_size()
        return fused

    def load_all(self, weights: Dict[str, WeightSpec]) -> Dict[str, torch.Tensor]:
        return {name: self.load(weight) for name, weight in weights.items()}
