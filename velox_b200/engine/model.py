"""A causal language model put together from a ``ModelSpec``.

The class has no architecture in it: it builds the parts the spec names, runs the schedule the
spec lists, and leaves every formula to the parts.  The forward is the reference's
(src/transformer.py:43-52,64-68): embedding, the layers in order, final norm on the rows whose
logits are wanted, lm_head on those rows only.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import CacheGroup
from ..cache.storage import LayerCache
from ..parts.base import CacheNeeds, HiddenState
from ..parts.registry import part_class
from ..parts.spec import ModelSpec, PartSpec
from ..weights.loader import WeightStore


def _build(kind: str, spec: PartSpec, store: WeightStore, dtype, device, **extra):
    cls = part_class(kind, spec.kind)
    return cls(spec.params, store.load_all(spec.weights), dtype, device, **extra)


class CausalLM:
    def __init__(
        self,
        spec: ModelSpec,
        store: WeightStore,
        dtype: torch.dtype,
        device: torch.device,
        max_position: Optional[int] = None,
    ) -> None:
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.hidden_size = spec.hidden_size
        self.vocab_size = spec.vocab_size

        self.embedding = _build("embedding", spec.embedding, store, dtype, device)
        self.final_norm = _build("norm", spec.final_norm, store, dtype, device)
        self.lm_head = _build("lm_head", spec.lm_head, store, dtype, device)

        positions: Dict[int, object] = {}
        self.blocks = []
        for layer in spec.layers:
            position = None
            if layer.position is not None:
                key = id(layer.position)
                position = positions.get(key)
                if position is None:
                    params = dict(layer.position.params)
                    if max_position is not None and "max_position" in params:
                        # The table is as long as the longest sequence the caller will run.
                        params["max_position"] = int(max_position)
                    position = part_class("position", layer.position.kind)(params, {}, dtype, device)
                    positions[key] = position
            mixer_cls = part_class("mixer", layer.mixer.kind)
            mixer_extra = {"position": position} if position is not None else {}
            mixer = mixer_cls(
                layer.mixer.params, store.load_all(layer.mixer.weights), dtype, device, **mixer_extra
            )
            feed_forward = _build("feed_forward", layer.feed_forward, store, dtype, device)
            norms = {name: _build("norm", norm, store, dtype, device) for name, norm in layer.norms.items()}
            block_cls = part_class("block", layer.block)
            self.blocks.append(block_cls(mixer, feed_forward, norms, layer.block_params))

        # Cache groups: one per distinct need (all keys / a window) among the entries that own
        # a cache.  entry_group[i] is the group whose tables address entry i's pages.
        self.cache_groups: List[CacheGroup] = []
        self.entry_needs: List[CacheNeeds] = []
        self.entry_group: List[Optional[int]] = []
        by_window: Dict[Optional[int], int] = {}
        for entry in spec.schedule:
            needs = self.blocks[entry.layer].mixer.cache_needs()
            self.entry_needs.append(needs)
            if needs.paged is None:
                self.entry_group.append(None)
                continue
            window = needs.paged.window
            if window not in by_window:
                by_window[window] = len(self.cache_groups)
                name = "all_keys" if window is None else f"window_{window}"
                self.cache_groups.append(CacheGroup(name=name, window=window))
            self.entry_group.append(by_window[window])
        if not self.cache_groups:
            # A model without paged state still gets one (empty) group so tables exist.
            self.cache_groups.append(CacheGroup(name="all_keys", window=None))
        for index, entry in enumerate(spec.schedule):
            if entry.cache_of is not None:
                mine, theirs = self.entry_needs[index], self.entry_needs[entry.cache_of]
                if mine.paged != theirs.paged:
                    raise ValueError(
                        f"schedule entry {index} reads the cache of entry {entry.cache_of} "
                        f"but needs {mine.paged}, not {theirs.paged}"
                    )

    # ------------------------------------------------------------------ what the step lays out
    def attention_signatures(self):
        """Distinct (cache group, (kv_heads, group, window, head_dim)) pairs among the schedule's mixers."""
        seen = []
        for index, entry in enumerate(self.spec.schedule):
            signature = self.blocks[entry.layer].mixer.attention_signature()
            if signature is None:
                continue
            key = (self.entry_group[index], signature)
            if key not in seen:
                seen.append(key)
        return seen

    def parts_take_padded_steps(self) -> bool:
        """Whether every mixer and feed-forward has said that it takes steps whose arrays are
        padded with tokens of no sequence (``takes_padded_steps``): only then are steps of any
        shape captured and replayed."""
        return all(getattr(part, "takes_padded_steps", False)
                   for block in self.blocks for part in (block.mixer, block.feed_forward))

    def head_dims(self) -> List[int]:
        dims = []
        for needs in self.entry_needs:
            if needs.paged is not None and needs.paged.head_dim not in dims:
                dims.append(needs.paged.head_dim)
        return dims

    # ------------------------------------------------------------------ forward
    def forward(self, ctx, caches: List[LayerCache], input_ids, logit_rows, num_logit_rows: int):
        """Run the step's tokens through every schedule entry; logits (float32) at ``logit_rows``."""
        ws = ctx.workspace
        resid = ws.get("model.resid", (ws.max_tokens, self.hidden_size), torch.float32)
        self.embedding.forward(input_ids, resid, ctx)
        hidden = HiddenState(resid=resid, delta=None)
        for index, entry in enumerate(self.spec.schedule):
            self.blocks[entry.layer].forward(hidden, ctx, caches[index])
        if num_logit_rows == 0:
            return None
        final = ws.get("model.final", (ws.max_logit_rows, self.hidden_size), self.dtype)
        self.final_norm.forward(hidden.resid, hidden.delta, final, num_logit_rows,
                                rows=logit_rows, write_resid=False)
        return self.lm_head.forward(final, num_logit_rows, ctx)
