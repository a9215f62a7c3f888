"""The step function: one batch of (request, its next tokens) through the model, from the cache.

``ModelRunner.step`` takes portions of prompts beside single decoded tokens, cut anywhere, runs
only the tokens it is given as one flat batch, and returns float32 logits at the wanted places.
It is the only way tokens reach the model: generation (``engine.Engine``) and trace replay
(``bin/trace_run``) both call it, with the cache manager deciding where the keys and values
go.  The reference runs two homogeneous forwards per step, a prefill batch and a decode batch
on two streams (engine/engine.py:303-329, engine/model_runner.py:171-270); here a decoded
token is a portion of length one and the whole step is one forward.

Per step the host builds, as int32 arrays (engine/model_runner.py:175-210 of the reference
builds the same quantities): token ids, absolute positions, per cache group the flat cache
slot of every token and the block table of every sequence, per sequence the first row, the
portion length and the cache length after the step, the rows whose logits are wanted, and the
attention work items.  Everything goes to the device in one copy from pinned memory.

The caller grows the block tables before the step (``CacheManager.append_slots``) and records
progress after it (``CacheManager.advance``).
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import gc
import os

import numpy as np
import torch

from ..cache.manager import CacheManager, SequenceCache
from ..cache.storage import LayerCache, allocate_layer_cache
from ..ops import attention_plan as ap
from ..ops import kernels
from .model import CausalLM


@dataclass
class StepChunk:
    """A request's next tokens in this step and the places among them whose logits are wanted."""

    seq: SequenceCache
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class GroupContext:
    block_tables: torch.Tensor  # int32 [S, width]
    slot_mapping: torch.Tensor  # int32 [T]; -1 = do not write


@dataclass
class DevicePlan:
    launches: List[Tuple[int, torch.Tensor, int]] = field(default_factory=list)
    merge_items: Optional[torch.Tensor] = None
    num_merges: int = 0
    merge_rows: int = 16  # the most rows a merge item can have (height of the split tiles)
    cluster: int = 1  # CTAs that share each item of the narrow bf16 kind
    # 2: the tensor-memory kind's items have long key ranges and outnumber the SMs (its launcher
    # then puts two CTAs on an SM); 1: the launcher decides by the grid alone.
    tc_ctas_per_sm: int = 1
    # Zeroed counters for the fused merge of the bfloat16 kernels; None: a merge kernel runs.
    split_counters: Optional[torch.Tensor] = None
    partial_o: Optional[torch.Tensor] = None
    partial_lse: Optional[torch.Tensor] = None
    # Set by the first layer that has run this layout: its tensors need no second look.
    checked: bool = False


class Workspace:
    """Named device buffers that live across steps; parts ask for them by name and size."""

    def __init__(self, max_tokens: int, max_logit_rows: int, device: torch.device) -> None:
        self.max_tokens = max_tokens
        self.max_logit_rows = max_logit_rows
        self.device = device
        self._buffers: Dict[str, torch.Tensor] = {}
        # Counts allocations: a captured graph is valid while this stands still.
        self.generation = 0

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        buf = self._buffers.get(name)
        if buf is None or buf.dtype != dtype or tuple(buf.shape) != tuple(shape):
            buf = torch.zeros(shape, dtype=dtype, device=self.device)
            self._buffers[name] = buf
            self.generation += 1
        return buf

    def num_bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


@dataclass
class StepContext:
    num_tokens: int
    num_seqs: int
    positions: torch.Tensor
    q_start: torch.Tensor
    q_len: torch.Tensor
    kv_len: torch.Tensor
    seq_slots: torch.Tensor
    groups: List[GroupContext]
    status: torch.Tensor
    workspace: Workspace
    plans: Dict[Tuple[Optional[int], Tuple], DevicePlan]
    # The float32 residual stream while a block runs its parts (they may add into it), else None.
    residual: Optional[torch.Tensor] = None
    # A float32 buffer the block offers the mixer for a copy of the residual rows as they are
    # after the mixer's product (a feed-forward that adds into the stream from many CTAs reads its
    # input there), and whether the mixer has written it.
    residual_mirror: Optional[torch.Tensor] = None
    residual_mirror_written: bool = False
    # int32 on the device, or None: the tokens the sampler drew in the step before, one per row.
    # A token id of -1 - r in this step's ids stands for row r of it (looked up by the embedding).
    fed_tokens: Optional[torch.Tensor] = None
    # Host copies, for parts that lay out work of their own.
    q_lens_host: List[int] = field(default_factory=list)
    kv_lens_host: List[int] = field(default_factory=list)

    def attention_plan(self, group: Optional[int], signature: Tuple) -> DevicePlan:
        return self.plans[(group, signature)]


class _Packer:
    """Lays int32 arrays end to end (16-byte aligned) so one copy moves them all."""

    def __init__(self) -> None:
        self.pieces: List[Tuple[int, np.ndarray]] = []
        self.size = 0

    def add(self, array: np.ndarray) -> Tuple[int, Tuple[int, ...]]:
        flat = np.ascontiguousarray(array, dtype=np.int32).reshape(-1)
        offset = self.size
        self.pieces.append((offset, flat))
        self.size += (flat.size + 3) // 4 * 4
        return offset, tuple(array.shape)


class _PaddedStage:
    """Host side of one decode bucket: two pinned copies of the captured step's arrays (used in
    turn, so that one can be written while the other's copy to the device may still run), views
    into them by name, and a record of what each copy holds."""

    def __init__(self, layout, bucket: int, num_groups: int, no_slot: int) -> None:
        where, plan_where, size = layout
        self.layout = layout
        self.bucket = bucket
        self.no_slot = no_slot
        self.num_groups = num_groups
        self.buffers = [torch.zeros(size, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.events: List[Optional[torch.cuda.Event]] = [None, None]
        self.flip = 0
        self.plan_options: Dict[Tuple, Tuple] = {}
        self.views: List[Dict] = []
        self.held: List[Dict] = []
        for buffer in self.buffers:
            array = buffer.numpy()
            views: Dict = {}
            for name, (offset, shape) in where.items():
                count = int(np.prod(shape)) if shape else 1
                views[name] = array[offset : offset + count].reshape(shape)
            for key, (entry_where, merge_where) in plan_where.items():
                (offset, shape), = entry_where.values()
                views[("items", key)] = array[offset : offset + shape[0] * 8].reshape(shape[0], 8)
                if merge_where is not None:
                    offset, shape = merge_where
                    views[("merges", key)] = array[offset : offset + shape[0] * 8].reshape(shape[0], 8)
            self.views.append(views)
            self.held.append({"count": -1, "rows": [[None] * bucket for _ in range(num_groups)]})

    def take(self):
        """The copy to write now: (its index, its views, what it holds)."""
        index = self.flip
        self.flip ^= 1
        if self.events[index] is not None:
            self.events[index].synchronize()
        return index, self.views[index], self.held[index]

    def copied(self, index: int) -> None:
        if self.events[index] is None:
            self.events[index] = torch.cuda.Event()
        self.events[index].record()

    def write_padding(self, index: int, n: int) -> None:
        """Everything that depends only on how many real sequences the step has."""
        bucket = self.bucket
        views, held = self.views[index], self.held[index]
        views["ids"][n:] = 0
        views["positions"][n:] = 0
        views["q_start"][:] = np.arange(bucket, dtype=np.int32)
        views["q_len"][:] = 1
        views["kv_len"][n:] = 1
        views["seq_slots"][n:] = self.no_slot
        views["logit_rows"][:] = np.arange(bucket, dtype=np.int32)
        for g in range(self.num_groups):
            views[f"slots{g}"][n:] = -1
            views[f"tables{g}"][n:] = 0
            held["rows"][g][n:] = [None] * (bucket - n)


# VELOX_B200_NO_TC_ATTENTION=1 keeps prompt portions on the mma.sync family (for bisecting).
_USE_TC_ATTENTION = os.environ.get("VELOX_B200_NO_TC_ATTENTION") != "1"

_STATUS_NAMES = {
    1: "a token id outside the vocabulary",
    2: "a position outside the position table",
    4: "a cache slot outside the pool",
    8: "a page id outside the pool",
    16: "a bounded wait ran out",
    32: "a partial attention row outside the scratch",
}


class ModelRunner:
    def __init__(
        self,
        model: CausalLM,
        cache: CacheManager,
        max_num_seqs: int,
        max_num_batched_tokens: int,
        max_logit_rows: Optional[int] = None,
        plan_overrides: Optional[dict] = None,
        enable_graphs: bool = True,
    ) -> None:
        kernels._require_cuda()
        self.model = model
        self.cache = cache
        self.device = model.device
        self.dtype = model.dtype
        self.page_size = cache.page_size
        self.max_num_seqs = max_num_seqs
        self.max_tokens = max(max_num_batched_tokens, max_num_seqs)
        self.plan_overrides = dict(plan_overrides or {})
        # Not a planner option: up to how many keys the layout without splits through memory is
        # used for padded single-token steps (tests move it down to their sizes).
        self.short_reach = int(self.plan_overrides.pop("short_reach", self.SHORT_REACH))
        if [g.window for g in cache.groups] != [g.window for g in model.cache_groups]:
            raise ValueError("the cache manager's groups are not the model's cache groups")

        self.workspace = Workspace(self.max_tokens, max_logit_rows or max_num_seqs, self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        # Set by whoever owns the sampler, before any graph is captured: its device tokens, which
        # a step's ids may name instead of a token (StepContext.fed_tokens).
        self.fed_tokens: Optional[torch.Tensor] = None
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count

        # One cache per schedule entry that owns one; entries that read another's share it.
        self.layer_caches: List[LayerCache] = []
        for index, entry in enumerate(model.spec.schedule):
            if entry.cache_of is not None:
                owner = self.layer_caches[entry.cache_of]
                self.layer_caches.append(
                    LayerCache(group=owner.group, k=owner.k, v=owner.v, state=owner.state, read_only=True)
                )
            else:
                self.layer_caches.append(
                    allocate_layer_cache(
                        model.entry_needs[index], model.entry_group[index], cache.num_pages,
                        cache.page_size, max_num_seqs, self.dtype, self.device,
                    )
                )
        self._signatures = model.attention_signatures()
        # One counter per (merge item, KV head); the kernels leave them at zero.
        self._split_counters = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)

        self._host: List[Optional[torch.Tensor]] = [None, None]
        self._copied: List[Optional[torch.cuda.Event]] = [None, None]
        self._device_meta: Optional[torch.Tensor] = None
        self._flip = 0
        self.num_steps = 0
        self.last_meta_bytes = 0
        # Launches of this package's kernels made by replaying captured steps.
        self.kernels_replayed = 0
        # The float32 path stays eager: it is the checking path, and without the fixed key-range
        # splits of a captured step its results do not depend on how the work was cut.
        self.enable_graphs = enable_graphs and self.dtype != torch.float32
        # Captured single-token steps by (bucket of sequences, reach in keys).
        self._graphs: Dict[Tuple[int, int], tuple] = {}
        longest = cache.max_model_len
        self._reaches: List[int] = [longest] if longest <= self.short_reach else [self.short_reach, longest]
        # Captured steps of other shapes, by rounded shape; the shapes used last are kept.
        self._mixed_graphs: "OrderedDict[tuple, tuple]" = OrderedDict()
        self._mixed_graphs_kept = 64
        self._mixed_seen: Dict[tuple, int] = {}
        # How the steps that are not single-token steps ran: replayed, launch by launch, captured.
        self.mixed_step_counts = {"replayed": 0, "eager": 0, "captured": 0}
        self._mixed_graphs_on = (self.enable_graphs and os.environ.get("VELOX_B200_NO_MIXED_GRAPHS") != "1"
                                 and model.parts_take_padded_steps())
        self._last_shape: Tuple[tuple, int] = ((), 0)
        # One memory pool for whatever a capture allocates (a library's workspace): the graphs
        # run one at a time on one stream, so they can share it instead of each keeping its own.
        self._graph_pool = torch.cuda.graph_pool_handle() if self.enable_graphs else None
        self._padded_stages: Dict[Tuple[int, int], "_PaddedStage"] = {}
        self._graphs_broken = False
        self._meta_generation = 0

        cache.on_slot_acquired = self._zero_state

    # ------------------------------------------------------------------ state slots
    def _zero_state(self, seq: SequenceCache) -> None:
        """A request that takes a state slot starts from zero state."""
        for layer_cache in self.layer_caches:
            if layer_cache.state is not None and not layer_cache.read_only:
                layer_cache.state[seq.slot].zero_()

    def kv_cache_bytes(self) -> int:
        return sum(c.num_bytes() for c in self.layer_caches if not c.read_only)

    # ------------------------------------------------------------------ staging
    def _staging(self, size: int) -> Tuple[torch.Tensor, torch.Tensor]:
        index = self._flip
        self._flip ^= 1
        if self._copied[index] is not None:
            self._copied[index].synchronize()
        host = self._host[index]
        if host is None or host.numel() < size:
            capacity = max(size, 1 << 14)
            capacity = 1 << (capacity - 1).bit_length()
            host = torch.empty(capacity, dtype=torch.int32, pin_memory=True)
            self._host[index] = host
        if self._device_meta is None or self._device_meta.numel() < size:
            capacity = 1 << (max(size, 1 << 14) - 1).bit_length()
            self._device_meta = torch.empty(capacity, dtype=torch.int32, device=self.device)
            self._meta_generation += 1
        if self._copied[index] is None:
            self._copied[index] = torch.cuda.Event()
        return host, self._device_meta

    # ------------------------------------------------------------------ the step
    @torch.no_grad()
    def step(self, chunks: Sequence[StepChunk], capture: bool = True) -> Optional[torch.Tensor]:
        """Run one batch.  Returns float32 logits [number of wanted places, vocab] in the order
        of the chunks and of their ``want`` lists, or None if nothing is wanted.

        ``capture=False`` keeps steps with prompt portions out of the captured-graph route (the
        graphs of single-token steps exist since warm-up and are used either way): a caller that
        queues steps ahead of the device has its launches hidden already, and a capture would
        only make the device wait for the host."""
        if not chunks:
            return None
        if self._graph_eligible(chunks):
            logits = self._graph_step(chunks)
            if logits is not None:
                self.num_steps += 1
                return logits
        if self._mixed_graphs_on and capture:
            logits = self._mixed_step(chunks)
            self.num_steps += 1
            return logits
        ctx, ids, logit_rows, num_logit_rows = self.prepare(chunks)
        logits = self.model.forward(ctx, self.layer_caches, ids, logit_rows, num_logit_rows)
        self.num_steps += 1
        return logits

    # ------------------------------------------------------------------ mixed steps as CUDA graphs
    def _mixed_step(self, chunks: Sequence[StepChunk]) -> Optional[torch.Tensor]:
        """A step of any shape, laid out with its arrays padded to round sizes (``prepare`` with
        ``round_shape``) so that steps of the same rounded shape run the same launches on the
        same buffers.  The first step of a shape runs launch by launch; from the second on the
        shape has a captured graph and a step costs the host its layout, one copy and one
        launch, where the launches of a 512-token step cost it about twice what they cost the
        device.  Graphs are kept for the shapes used last."""
        ctx, ids, logit_rows, num_logit_rows = self.prepare(chunks, round_shape=True)
        key, wanted = self._last_shape
        entry = self._mixed_graphs.get(key)
        generation = (self.workspace.generation, self._meta_generation)
        if entry is not None and entry[2] == generation:
            self._mixed_graphs.move_to_end(key)
            entry[0].replay()
            self.kernels_replayed += entry[3]
            self.mixed_step_counts["replayed"] += 1
            return None if wanted == 0 else entry[1][:wanted]
        logits = self.model.forward(ctx, self.layer_caches, ids, logit_rows, num_logit_rows)
        self.mixed_step_counts["eager"] += 1
        seen = self._mixed_seen.get(key, 0) + 1
        self._mixed_seen[key] = seen
        if len(self._mixed_seen) > 4096:
            self._mixed_seen.clear()
        if seen >= 2 and not self._graphs_broken:
            # The shape has come back: capture what has just run (the capture itself runs nothing).
            try:
                graph = torch.cuda.CUDAGraph()
                launches_before = kernels.launch_count
                collecting = gc.isenabled()
                gc.disable()
                try:
                    with torch.cuda.graph(graph, pool=self._graph_pool):
                        captured = self.model.forward(ctx, self.layer_caches, ids, logit_rows, num_logit_rows)
                finally:
                    if collecting:
                        gc.enable()
                if generation == (self.workspace.generation, self._meta_generation):
                    self._mixed_graphs[key] = (graph, captured, generation, kernels.launch_count - launches_before)
                    self.mixed_step_counts["captured"] += 1
                    while len(self._mixed_graphs) > self._mixed_graphs_kept:
                        self._mixed_graphs.popitem(last=False)
            except Exception as exc:  # a part that cannot be captured: run launch by launch from now on
                import logging

                logging.getLogger(__name__).warning("CUDA graph capture of a mixed step failed (%s); running eagerly", exc)
                self._mixed_graphs_on = False
                torch.cuda.synchronize(self.device)
        return None if logits is None else logits[:wanted]

    @staticmethod
    def _round_tokens(count: int) -> int:
        """Token counts that share a captured step: multiples of 16 up to 128, of 32 up to 1,024,
        of 64 beyond (the padding rows cost what real rows cost)."""
        step = 16 if count <= 128 else 32 if count <= 1024 else 64
        return -(-count // step) * step

    @staticmethod
    def _round_count(count: int, granule: int = 8) -> int:
        """Powers of two up to the granule, multiples of it beyond."""
        if count <= 0:
            return 0
        if count <= granule:
            return 1 << (count - 1).bit_length()
        return -(-count // granule) * granule

    def prepare(self, chunks: Sequence[StepChunk], pad_to: Optional[int] = None, round_shape: bool = False,
                reach: Optional[int] = None):
        """Build the step's device-side description: (context, token ids, logit rows, their count).

        ``pad_to`` (single-token steps only) pads the batch to that many sequences with rows
        that do nothing: they write to no cache slot, attend through no work item, and their
        logits are never looked at.  A padded step has the same shape whatever the real batch
        is, every array lands at the same place of the device buffer, and the logits of all
        ``pad_to`` rows are computed.

        ``round_shape`` (any step) rounds every extent up: tokens, sequences, wanted rows, the
        work items of each kernel family and the merge items, and gives the block tables their
        full width.  Padding tokens belong to no sequence, write to no cache slot and are
        covered by no work item; padding items have sequence -1 and do nothing.  Steps with
        equal rounded extents get equal layouts; ``self._last_shape`` is (the extents as a
        key, the number of rows really wanted).
        """
        P = self.page_size
        real_seqs = len(chunks)
        q_lens = [len(chunk.tokens) for chunk in chunks]
        if q_lens and min(q_lens) < 1:
            raise ValueError("every chunk of a step needs at least one token")
        padded = pad_to is not None
        if padded and (any(n != 1 for n in q_lens) or real_seqs > pad_to):
            raise ValueError("only steps of single tokens can be padded")
        num_seqs = pad_to if padded else real_seqs
        num_tokens = num_seqs if padded else sum(q_lens)
        if num_tokens > self.max_tokens:
            raise ValueError(f"step of {num_tokens} tokens exceeds the runner's {self.max_tokens}")
        if num_seqs > self.max_num_seqs:
            raise ValueError(f"step of {num_seqs} requests exceeds the runner's {self.max_num_seqs}")

        ids = np.zeros(num_tokens, np.int32)
        positions = np.zeros(num_tokens, np.int32)
        q_start = np.arange(num_seqs, dtype=np.int32) if padded else np.empty(num_seqs, np.int32)
        q_len_arr = np.ones(num_seqs, np.int32)
        kv_len_arr = np.ones(num_seqs, np.int32)
        kv_lens: List[int] = []
        seq_slots = np.full(num_seqs, self.max_num_seqs, np.int32)
        logit_rows: List[int] = []
        num_groups = len(self.cache.groups)
        slot_maps = [np.full(num_tokens, -1, np.int32) for _ in range(num_groups)]
        width = 1
        row = 0
        for s, chunk in enumerate(chunks):
            seq, n = chunk.seq, q_lens[s]
            start = seq.num_computed
            if (start + n + P - 1) // P > seq.num_logical_blocks:
                raise ValueError(
                    f"{seq.seq_id}: block tables hold {seq.num_logical_blocks} pages, "
                    f"{start + n} tokens need more (append_slots was not called)"
                )
            ids[row : row + n] = chunk.tokens
            pos = np.arange(start, start + n, dtype=np.int32)
            positions[row : row + n] = pos
            q_start[s] = row
            q_len_arr[s] = n
            kv_len_arr[s] = start + n
            kv_lens.append(start + n)
            if seq.slot is not None:
                seq_slots[s] = seq.slot
            for g in range(num_groups):
                table = np.asarray(seq.tables[g], dtype=np.int32)
                slot_maps[g][row : row + n] = table[pos // P] * P + pos % P
            width = max(width, seq.num_logical_blocks)
            if not padded:
                for w in chunk.want:
                    if not 0 <= w < n:
                        raise ValueError(f"{seq.seq_id}: wanted place {w} is outside its {n} tokens")
                    logit_rows.append(row + w)
            row += n
        if padded:
            width = self.cache.max_blocks_per_seq
            logit_rows = list(range(num_seqs))
        wanted_rows = len(logit_rows)
        if round_shape and not padded:
            real_tokens = num_tokens
            num_tokens = min(self.max_tokens, self._round_tokens(real_tokens))
            num_seqs = min(self.max_num_seqs, 1 << (real_seqs - 1).bit_length())
            extra = num_tokens - real_tokens
            ids = np.concatenate([ids, np.zeros(extra, np.int32)])
            positions = np.concatenate([positions, np.zeros(extra, np.int32)])
            slot_maps = [np.concatenate([m, np.full(extra, -1, np.int32)]) for m in slot_maps]
            more = num_seqs - real_seqs
            q_start = np.concatenate([q_start, np.full(more, real_tokens, np.int32)])
            q_len_arr = np.concatenate([q_len_arr[:real_seqs], np.zeros(more, np.int32)])
            kv_len_arr = np.concatenate([kv_len_arr[:real_seqs], np.zeros(more, np.int32)])
            seq_slots = np.concatenate([seq_slots[:real_seqs], np.full(more, self.max_num_seqs, np.int32)])
            width = self.cache.max_blocks_per_seq
            logit_rows = logit_rows + [0] * (self._round_count(wanted_rows) - wanted_rows)
        width = (width + 7) // 8 * 8
        tables = [np.zeros((num_seqs, width), np.int32) for _ in range(num_groups)]
        for s, chunk in enumerate(chunks):
            for g in range(num_groups):
                t = chunk.seq.tables[g]
                tables[g][s, : len(t)] = t
        num_logit_rows = len(logit_rows)
        if num_logit_rows > self.workspace.max_logit_rows:
            self.workspace.max_logit_rows = num_logit_rows

        # Attention work, one layout per distinct (cache group, head grouping, window).
        host_plans = {}
        for group, signature in self._signatures:
            opt = self._plan_options(signature)
            if padded:
                splits, cluster = self._padded_splits(num_seqs, opt, reach)
                plan = ap.plan_attention(q_lens, kv_lens, opt, fixed_splits=splits, fixed_cluster=cluster)
                plan = ap.pad_plan(plan, num_seqs, splits, opt)
            else:
                plan = ap.plan_attention(q_lens, kv_lens, opt)
                if round_shape:
                    plan = ap.round_plan(plan, self._round_count)
            host_plans[(group, signature)] = plan
        if round_shape and not padded:
            self._last_shape = (
                (num_tokens, num_seqs, len(logit_rows), width, tuple(
                    (key, plan.cluster, tuple((kind, len(items)) for kind, items in sorted(plan.items.items())),
                     len(plan.merge_items), plan.partial_rows > 0)
                    for key, plan in host_plans.items())),
                wanted_rows,
            )

        packer = _Packer()
        where = {
            "ids": packer.add(ids),
            "positions": packer.add(positions),
            "q_start": packer.add(q_start),
            "q_len": packer.add(q_len_arr),
            "kv_len": packer.add(kv_len_arr),
            "seq_slots": packer.add(seq_slots),
            "logit_rows": packer.add(np.asarray(logit_rows, np.int32)),
        }
        for g in range(num_groups):
            where[f"slots{g}"] = packer.add(slot_maps[g])
            where[f"tables{g}"] = packer.add(tables[g])
        plan_where = {}
        for key, plan in host_plans.items():
            entry = {kind: packer.add(items) for kind, items in sorted(plan.items.items())}
            merge = packer.add(plan.merge_items) if len(plan.merge_items) else None
            plan_where[key] = (entry, merge)

        host, dev = self._staging(packer.size)
        host_np = host.numpy()
        for offset, flat in packer.pieces:
            host_np[offset : offset + flat.size] = flat
        dev[: packer.size].copy_(host[: packer.size], non_blocking=True)
        self._copied[self._flip ^ 1].record()
        self.last_meta_bytes = packer.size * 4
        self._last_layout = (where, plan_where, packer.size)

        def view(name: str) -> torch.Tensor:
            offset, shape = where[name]
            count = int(np.prod(shape)) if shape else 1
            return dev[offset : offset + count].view(shape)

        plans: Dict[Tuple[Optional[int], Tuple], DevicePlan] = {}
        for key, plan in host_plans.items():
            entry, merge = plan_where[key]
            device_plan = DevicePlan(cluster=plan.cluster)
            long_items = plan.items.get(ap.KIND_BF16_TC)
            if long_items is not None and len(long_items):
                real = long_items[long_items[:, 0] >= 0]
                if len(real) * key[1][0] > self.num_sms and len(real):
                    tiles = -(-(real[:, 4] - real[:, 3]).astype(np.int64) // ap.KEY_TILE)
                    if float(tiles.mean()) >= self.TC_LONG_TILES:
                        device_plan.tc_ctas_per_sm = 2
            for kind, (offset, shape) in entry.items():
                count = shape[0]
                device_plan.launches.append((kind, dev[offset : offset + count * 8].view(count, 8), count))
            if merge is not None:
                offset, shape = merge
                device_plan.merge_items = dev[offset : offset + shape[0] * 8].view(shape[0], 8)
                device_plan.num_merges = shape[0]
                device_plan.merge_rows = max(ap.TILE_ROWS[kind] for kind in entry)
                needed = shape[0] * key[1][0]
                if self.dtype != torch.float32 and needed <= self._split_counters.numel():
                    device_plan.split_counters = self._split_counters
            if plan.partial_rows:
                head_dim = key[1][3]
                device_plan.partial_o = self._scratch("attention.partial_o", plan.partial_rows * head_dim)
                device_plan.partial_lse = self._scratch("attention.partial_lse", plan.partial_rows)
            plans[key] = device_plan

        ctx = StepContext(
            num_tokens=num_tokens,
            num_seqs=num_seqs,
            positions=view("positions"),
            q_start=view("q_start"),
            q_len=view("q_len"),
            kv_len=view("kv_len"),
            seq_slots=view("seq_slots"),
            groups=[
                GroupContext(block_tables=view(f"tables{g}"), slot_mapping=view(f"slots{g}"))
                for g in range(num_groups)
            ],
            status=self.status,
            workspace=self.workspace,
            plans=plans,
            fed_tokens=self.fed_tokens,
            q_lens_host=[int(n) for n in q_len_arr],
            kv_lens_host=[int(n) for n in kv_len_arr],
        )
        return ctx, view("ids"), view("logit_rows"), num_logit_rows

    # ------------------------------------------------------------------ decode steps as CUDA graphs
    def _plan_options(self, signature) -> "ap.PlanOptions":
        """How attention work is cut for layers of this (KV heads, heads per KV head, window,
        head size): what an SM holds of the kernels depends on the head size."""
        num_kv_heads, heads_per_kv, window, head_dim = signature
        use_f32 = self.dtype == torch.float32
        options = dict(num_kv_heads=num_kv_heads, group=heads_per_kv, window=window, use_f32=use_f32,
                       target_ctas=2 * self.num_sms)
        if not use_f32:
            options["narrow_target_ctas"] = kernels.narrow_attention_slots(head_dim) * self.num_sms
            options["narrow_max_cluster"] = kernels.max_attention_cluster(head_dim)
            options["narrow_cluster_limits"] = kernels.attention_cluster_limits(head_dim)
            options["wide_on_tensor_memory"] = kernels.attention_has_tc(head_dim) and _USE_TC_ATTENTION
        if "target_ctas" in self.plan_overrides and "narrow_target_ctas" not in self.plan_overrides:
            options["narrow_target_ctas"] = self.plan_overrides["target_ctas"]
        options.update(self.plan_overrides)
        return ap.PlanOptions(**options)

    # Key tiles per work item from which the tensor-memory attention runs two CTAs on an SM when
    # it has more items than SMs (measured: 192 items of 500 tiles 616 us against 774 with one
    # CTA per SM, 192 items of 48 tiles 84 against 78).
    TC_LONG_TILES = 96

    # A padded single-token step is laid out for sequences of up to so many keys (its "reach"):
    # the shortest class has no splits through memory, whose merge costs a layer of a small model
    # about six microseconds, the other is cut for ``max_model_len``.
    SHORT_REACH = 8192

    def _reach_of(self, longest: int) -> int:
        """The smallest reach that holds a sequence of ``longest`` keys."""
        for reach in self._reaches:
            if longest <= reach:
                return reach
        return self._reaches[-1]

    def _padded_splits(self, num_seqs: int, opt: "ap.PlanOptions", reach: Optional[int] = None) -> Tuple[int, int]:
        """(splits through memory, cluster size) of a padded single-token step: enough CTAs to
        fill the GPU at this batch size, the same for every sequence of up to ``reach`` keys
        (``max_model_len`` if not given) whatever its length."""
        tiles = -(-opt.group // 16)
        per_split = max(1, num_seqs * opt.num_kv_heads * tiles)
        narrow = not opt.use_f32 and opt.group <= opt.narrow_max_rows
        target = opt.narrow_target_ctas if narrow and opt.narrow_target_ctas is not None else opt.target_ctas
        # Rounded down: all CTAs should be resident at once; a few more than that would run as
        # a second wave after the first has finished.
        wanted = max(1, target // per_split)
        if not narrow:
            return max(1, min(32, wanted)), 1
        cluster = ap.choose_cluster(opt, per_split, wanted)
        if cluster == 1:
            return max(1, min(32, wanted)), 1
        # The layout is the same for every length, so the longest sequence it is made for decides
        # whether splitting through memory as well is worth its slower merge.
        longest = self.cache.max_model_len if reach is None else min(reach, self.cache.max_model_len)
        return max(1, min(32, wanted // cluster, ap.splits_through_memory(longest, cluster, opt))), cluster

    def _graph_eligible(self, chunks: Sequence[StepChunk]) -> bool:
        if not self.enable_graphs or self._graphs_broken:
            return False
        if len(chunks) > self.max_num_seqs:
            return False
        return all(len(c.tokens) == 1 and tuple(c.want) == (0,) for c in chunks)

    def _bucket(self, num_seqs: int) -> int:
        size = 1
        while size < num_seqs:
            size *= 2
        return min(size, self.max_num_seqs)

    def _graph_step(self, chunks: Sequence[StepChunk]) -> Optional[torch.Tensor]:
        """A step of single tokens, padded to a bucket size and replayed as one CUDA graph
        (the reference captures its decode forward per bucket too, engine/model_runner.py:330-393)."""
        bucket = self._bucket(len(chunks))
        reach = self._reach_of(max(c.seq.num_computed for c in chunks) + 1)
        entry = self._graphs.get((bucket, reach))
        if entry is not None and entry[2] != (self.workspace.generation, self._meta_generation):
            entry = None
        if entry is None:
            try:
                entry = self._capture(bucket, reach)
            except Exception as exc:  # a part that cannot be captured: run eagerly from now on
                import logging

                logging.getLogger(__name__).warning("CUDA graph capture failed (%s); running eagerly", exc)
                self._graphs_broken = True
                torch.cuda.synchronize(self.device)
                return None
            self._graphs[(bucket, reach)] = entry
        if not self._fill_padded(entry, bucket, chunks, reach):
            self.prepare(chunks, pad_to=bucket, reach=reach)
        if entry[2] != (self.workspace.generation, self._meta_generation):
            # A buffer grew while the step was laid out: the graph points at old memory.
            self._graphs.pop((bucket, reach), None)
            return None
        graph, logits = entry[0], entry[1]
        graph.replay()
        self.kernels_replayed += entry[4]
        return logits[: len(chunks)]

    def capture_decode_graphs(self) -> int:
        """Capture the graph of every decode bucket that has none yet (1, 2, 4, ... up to the most
        requests, each for every reach), smallest first; returns how many it captured.  Nothing happens where steps
        are not replayed as graphs.  A later step that makes a work buffer grow still recaptures
        its bucket; after a warm-up that has run a full prefill portion none does."""
        if not self.enable_graphs or self._graphs_broken:
            return 0
        captured = 0
        bucket = 1
        while True:
            bucket = min(bucket, self.max_num_seqs)
            for reach in self._reaches:
                entry = self._graphs.get((bucket, reach))
                if entry is not None and entry[2] == (self.workspace.generation, self._meta_generation):
                    continue
                try:
                    self._graphs[(bucket, reach)] = self._capture(bucket, reach)
                except Exception as exc:  # the same fallback as at the first use of a bucket
                    import logging

                    logging.getLogger(__name__).warning("CUDA graph capture failed (%s); running eagerly", exc)
                    self._graphs_broken = True
                    torch.cuda.synchronize(self.device)
                    return captured
                captured += 1
            if bucket >= self.max_num_seqs:
                return captured
            bucket *= 2

    def _fill_padded(self, entry, bucket: int, chunks: Sequence[StepChunk], reach: Optional[int] = None) -> bool:
        """Write a padded single-token step straight into the places the captured step reads
        (the layout of a bucket never changes), with arrays instead of per-token loops.  What
        reaches the device is what ``prepare(chunks, pad_to=bucket)`` writes.  Every bucket has
        two pinned host copies of its arrays, used in turn, and remembers what each holds: a
        block-table row is written again only when its sequence's tables have changed, the
        padding only when the number of real sequences has.  False: use ``prepare``."""
        where, plan_where, size = entry[3]
        if any(sig[1] > 16 for _, sig in self._signatures):
            return False
        reach = self._reaches[-1] if reach is None else reach
        stage = self._padded_stages.get((bucket, reach))
        if stage is None or stage.layout is not entry[3]:
            stage = _PaddedStage(entry[3], bucket, len(self.cache.groups), self.max_num_seqs)
            self._padded_stages[(bucket, reach)] = stage
        P = self.page_size
        n = len(chunks)
        positions = np.fromiter((c.seq.num_computed for c in chunks), np.int64, n)
        blocks = (positions // P).tolist()
        for c, block in zip(chunks, blocks):
            if block >= c.seq.num_logical_blocks:
                raise ValueError(f"{c.seq.seq_id}: append_slots was not called before the step")
        index, views, held = stage.take()
        fresh = held["count"] != n
        if fresh:
            stage.write_padding(index, n)
            held["count"] = n
        views["ids"][:n] = [c.tokens[0] for c in chunks]
        views["positions"][:n] = positions
        kv_lens = positions + 1
        views["kv_len"][:n] = kv_lens
        views["seq_slots"][:n] = [self.max_num_seqs if c.seq.slot is None else c.seq.slot for c in chunks]
        offsets = positions % P
        rows = held["rows"]
        for g in range(len(self.cache.groups)):
            views[f"slots{g}"][:n] = np.fromiter(
                (c.seq.tables[g][b] for c, b in zip(chunks, blocks)), np.int64, n) * P + offsets
            tables = views[f"tables{g}"]
            row_keys = rows[g]
            for s, c in enumerate(chunks):
                key = (c.seq.serial, c.seq.tables_version)
                if row_keys[s] != key:
                    t = c.seq.tables[g]
                    tables[s, : len(t)] = t
                    tables[s, len(t):] = 0
                    row_keys[s] = key
        for key, (entry_where, merge_where) in plan_where.items():
            opt, splits = stage.plan_options.get(key, (None, None))
            if opt is None:
                opt = self._plan_options(key[1])
                splits, _ = self._padded_splits(bucket, opt, reach)
                stage.plan_options[key] = (opt, splits)
            items_view, merges_view = views[("items", key)], views.get(("merges", key))
            if splits <= 1 and not fresh:
                # Only the key ranges move from step to step.
                lo = np.maximum(0, kv_lens - opt.window) if opt.window else 0
                items_view[:n, 3] = lo
                items_view[:n, 4] = kv_lens
                continue
            _, items, merges, _ = ap.plan_single_tokens(kv_lens, bucket, splits, opt)
            items_view[:] = items
            if merges is not None and merges_view is not None:
                merges_view[:] = merges
        host, dev = stage.buffers[index], self._device_for(size)
        dev[:size].copy_(host, non_blocking=True)
        stage.copied(index)
        self.last_meta_bytes = size * 4
        return True

    def _device_for(self, size: int) -> torch.Tensor:
        if self._device_meta is None or self._device_meta.numel() < size:
            capacity = 1 << (max(size, 1 << 14) - 1).bit_length()
            self._device_meta = torch.empty(capacity, dtype=torch.int32, device=self.device)
            self._meta_generation += 1
        return self._device_meta

    def _capture(self, bucket: int, reach: Optional[int] = None):
        reach = self._reaches[-1] if reach is None else reach
        # Twice eagerly on an all-padding batch: buffers get their final size and addresses.
        for _ in range(2):
            ctx, ids, rows, count = self.prepare([], pad_to=bucket, reach=reach)
            self.model.forward(ctx, self.layer_caches, ids, rows, count)
        torch.cuda.synchronize(self.device)
        generation = (self.workspace.generation, self._meta_generation)
        ctx, ids, rows, count = self.prepare([], pad_to=bucket, reach=reach)
        layout = self._last_layout
        graph = torch.cuda.CUDAGraph()
        launches_before = kernels.launch_count
        # No cycle collection while the stream is capturing: a collected tensor frees device
        # memory, and the allocator's bookkeeping for that is not allowed during a capture.
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph, pool=self._graph_pool):
                logits = self.model.forward(ctx, self.layer_caches, ids, rows, count)
        finally:
            if collecting:
                gc.enable()
        launches = kernels.launch_count - launches_before
        torch.cuda.synchronize(self.device)
        if generation != (self.workspace.generation, self._meta_generation):
            raise RuntimeError("buffers moved during capture")
        # (graph, logits, buffer generation, layout of the step's arrays, kernels per replay)
        return graph, logits, generation, layout, launches

    def _scratch(self, name: str, count: int) -> torch.Tensor:
        ws = self.workspace
        current = ws._buffers.get(name)
        if current is not None and current.numel() >= count:
            return current
        capacity = 1 << (max(count, 1 << 16) - 1).bit_length()
        return ws.get(name, (capacity,), torch.float32)

    # ------------------------------------------------------------------ checks
    def check_status(self) -> None:
        """Read the device status word (this synchronises) and raise if a kernel flagged a fault."""
        self.raise_for_status(int(self.status[0].item()))

    def raise_for_status(self, word: int) -> None:
        """Raise for a status word that was read back (by ``check_status`` or, in generation,
        behind the sampled tokens), after clearing the word on the device."""
        if word:
            self.status.zero_()
            what = [text for bit, text in _STATUS_NAMES.items() if word & bit]
            raise RuntimeError("a kernel of the step refused an access: " + "; ".join(what))
