"""Data that describes a model: which parts it is made of and in what order they run.

An architecture module turns its typed configuration into a ``ModelSpec``.  Nothing in a spec is
code: parts are named by registry key with their sizes and constants as parameters, weights are
named by checkpoint tensor name, and the order in which layers run is a list.  The engine, the
cache manager, the weight loader and the random-weights writer all work from the spec alone, so
a new architecture adds a spec builder and, where needed, new part classes, and nothing else.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class TensorSource:
    """One tensor of the checkpoint, by its name there."""

    name: str
    shape: Tuple[int, ...]
    # How the random-weights mode fills it: "normal" = N(0, std); "one_plus_normal" = 1 + N(0, std).
    init: str = "normal"


@dataclass(frozen=True)
class WeightSpec:
    """A weight of a part: one checkpoint tensor, or several concatenated along dim 0.

    ``role`` decides the storage on the device: a "matrix" is kept in the compute dtype
    (bfloat16 when serving), a "vector" (norm weights, biases) always in float32, a "table" of
    integers in int32.
    """

    sources: Tuple[TensorSource, ...]
    role: str = "matrix"

    @property
    def shape(self) -> Tuple[int, ...]:
        first = self.sources[0].shape
        rows = sum(src.shape[0] for src in self.sources)
        return (rows,) + tuple(first[1:])


@dataclass(frozen=True)
class PartSpec:
    """A part by registry key, its parameters, and where its weights come from."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    weights: Dict[str, WeightSpec] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer, a feed-forward and their norms."""

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]
    # Position encoding the mixer applies; None for a mixer that needs none.
    position: Optional[PartSpec] = None
    block_params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelSpec.layers`` and may appear in several entries (the same weights run
    twice).  Every entry has a cache of its own unless ``cache_of`` names an earlier entry of the
    schedule, in which case the mixer reads that entry's cache and writes none.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    lm_head: PartSpec
    eos_token_ids: Tuple[int, ...] = ()
    # Checkpoint tensors that may be present and are not read (no error for them).
    ignored_tensors: Tuple[str, ...] = ()

    def part_specs(self) -> List[PartSpec]:
        out: List[PartSpec] = [self.embedding]
        for layer in self.layers:
            out.append(layer.mixer)
            out.append(layer.feed_forward)
            out.extend(layer.norms.values())
            if layer.position is not None:
                out.append(layer.position)
        out.extend([self.final_norm, self.lm_head])
        return out

    def checkpoint_tensors(self) -> Dict[str, TensorSource]:
        """Every checkpoint tensor the model reads, by name (a tied tensor appears once)."""
        tensors: Dict[str, TensorSource] = {}
        for part in self.part_specs():
            for weight in part.weights.values():
                for src in weight.sources:
                    known = tensors.get(src.name)
                    if known is not None and known.shape != src.shape:
                        raise ValueError(
                            f"tensor {src.name} is declared with shapes {known.shape} and {src.shape}"
                        )
                    tensors[src.name] = src
        return tensors

    def validate(self) -> None:
        if not self.schedule:
            raise ValueError("a model needs at least one schedule entry")
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule entry {index} names layer {entry.layer}, which does not exist")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < index:
                    raise ValueError(
                        f"schedule entry {index} reads the cache of entry {entry.cache_of}, "
                        "which must be an earlier entry"
                    )
                if self.schedule[entry.cache_of].cache_of is not None:
                    raise ValueError(
                        f"schedule entry {index} reads the cache of entry {entry.cache_of}, "
                        "which has no cache of its own"
                    )
