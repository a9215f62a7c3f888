"""Interfaces of the parts a model is put together from.

Every part is built from a ``PartSpec``: its parameters (sizes and constants) and its weights,
already on the device under the part's own local names.  No part knows which model it is in or
which layer it is; it sees tensors and the step context.

Interfaces (T = tokens of the step, E = model width, dt = compute dtype):

``Norm.forward(resid, delta, out, num_rows, rows=None, write_resid=True)``
    resid float32 [T, E] is the residual stream; delta dt [T, E] or None is what the previous
    part produced and has not been added yet.  Adds, optionally writes the sum back, writes the
    normalised rows to ``out`` (dt).  Fusing the add into the norm is why the interface has
    both.

``Norm.pending(resid, out, num_rows)`` may return a ``PendingNorm`` instead of running (a norm
    that is a row scale times a weight can be made inside the projection that follows); None
    means it has to run.

A part's product that is waiting to be added to the residual stream ("delta") is a tensor
dt [T, E], or None when the part has added it into ``ctx.residual`` (the float32 residual
stream, set by the block around the calls) itself.

``Mixer.forward(x, ctx, cache) -> delta``
    x dt [T, E] is the normalised input.  ``cache`` is the mixer's own ``LayerCache`` (its
    pages of the cache group it declared and/or its slot-indexed state) or, for a layer that
    reads another layer's cache, that layer's cache with ``cache.read_only`` set.
    ``Mixer.cache_spec()`` declares what it needs: a ``PagedCacheSpec`` (keys and values in
    pages; a window or all keys), a ``StateSpec`` (fixed size per request), both or neither.

``FeedForward.forward(x, ctx) -> delta``

``PositionEncoding``: owned by the mixer that applies it; the rotary kinds offer
    ``rotate_and_store`` (rotate q in place, rotate k and write k, v to the cache in one kernel).

``Block.forward(hidden, ctx, cache)``: the arrangement of norms, mixer and feed-forward around
    the residual stream; ``hidden`` carries (resid, pending delta).

``Embedding.forward(ids, resid, ctx)``, ``LMHead.forward(x, num_rows, ctx) -> float32 [R, V]``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class PagedCacheSpec:
    """Keys and values of every token, in pages; ``window`` None keeps all keys."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size, one row per state slot, zeroed when a slot is taken."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class CacheNeeds:
    paged: Optional[PagedCacheSpec] = None
    state: Optional[StateSpec] = None


class PendingNorm:
    """A norm that has not run yet: the float32 rows it reads (no pending delta), its weight and
    eps, and the buffer its result belongs in.  A part that declares ``accepts_pending_norm``
    may get this in place of its normalised input and hand it to ``ops.linear.linear`` or
    ``swiglu_linear``, which make the norm inside the projection when the step is small;
    ``materialize()`` runs the norm kernel (once) for anybody who needs the tensor."""

    def __init__(self, norm, resid: torch.Tensor, out: torch.Tensor, num_rows: int) -> None:
        self.norm = norm
        self.resid = resid
        self.out = out
        self.num_rows = num_rows
        self.weight = norm.weight
        self.eps = norm.eps
        self._done = False

    @property
    def dtype(self) -> torch.dtype:
        return self.out.dtype

    def materialize(self) -> torch.Tensor:
        if not self._done:
            self.norm.forward(self.resid, None, self.out, self.num_rows)
            self._done = True
        return self.out


class Part:
    """Base of every part: parameters, weights by local name, compute dtype."""

    def __init__(
        self,
        params: Dict[str, Any],
        weights: Dict[str, torch.Tensor],
        dtype: torch.dtype,
        device: torch.device,
    ) -> None:
        self.params = dict(params)
        self.weights = weights
        self.dtype = dtype
        self.device = device

    def expect(self, name: str, shape: Tuple[int, ...]) -> torch.Tensor:
        tensor = self.weights.get(name)
        if tensor is None:
            raise KeyError(f"{type(self).__name__} needs a weight named {name!r}")
        if tuple(tensor.shape) != tuple(shape):
            raise ValueError(
                f"{type(self).__name__}: weight {name!r} has shape {tuple(tensor.shape)}, "
                f"expected {tuple(shape)}"
            )
        return tensor


class Mixer(Part):
    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds()

    def attention_signature(self):
        """(num_kv_heads, heads per KV head, window, head_dim) if the step should lay out
        attention work for it; layers with equal signatures in one cache group share a layout."""
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


class Norm(Part):
    def forward(self, resid, delta, out, num_rows, rows=None, write_resid=True) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError

    def pending(self, resid, out, num_rows) -> Optional["PendingNorm"]:
        """A description of this norm of ``resid`` (nothing pending to add) for a projection to
        make on the fly, or None if the norm has to run as a kernel of its own."""
        return None


class PositionEncoding(Part):
    pass


@dataclass
class HiddenState:
    """The residual stream (float32) and what has been produced but not added to it yet."""

    resid: torch.Tensor
    delta: Optional[torch.Tensor] = None
