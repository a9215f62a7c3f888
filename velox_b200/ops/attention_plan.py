"""Host-side layout of attention work for one step: which tile of rows meets which keys.

The attention kernels (csrc/attention.cu) run *work items*; this module makes them from the
batch's (portion length, cache length) pairs.  A row is a (query token, query head of a KV
group) pair, ``row = token_in_portion * group + head_in_group``.  Rows of one sequence are cut
into tiles of the kernel family's height; a tile's key range is what its first and last token
may see (causal bound above, window bound below); a long key range of a short tile is split
so that the step fills the GPU, and the splits are merged afterwards.

The reference sizes its split count from ``batch * kv_heads`` against the SM count with a cap
of 8 (src/decode_attention.py:237-252); the rule here is the same idea without the cap, in
units of 64-key tiles.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

KIND_F32, KIND_BF16_WIDE, KIND_BF16_NARROW, KIND_BF16_TC = 0, 1, 2, 3
TILE_ROWS = {KIND_F32: 16, KIND_BF16_WIDE: 64, KIND_BF16_NARROW: 16, KIND_BF16_TC: 128}
KEY_TILE = 64
ITEM_WIDTH = 8


@dataclass
class AttentionPlan:
    # kind -> int32 [n, 8] work items
    # {seq, row_begin, row_count, kv_begin, kv_end, partial_base, merge index, number of splits}
    items: Dict[int, np.ndarray] = field(default_factory=dict)
    # int32 [m, 8] {seq, row_begin, row_count, first_partial_base, num_splits, split_stride, 0, 0}
    merge_items: np.ndarray = field(default_factory=lambda: np.zeros((0, ITEM_WIDTH), np.int32))
    # Rows of float32 scratch ([rows, D] and [rows]) the splits write.
    partial_rows: int = 0
    # CTAs of a thread-block cluster that share each item of the narrow bf16 kind: every CTA
    # takes a run of the item's key tiles and they merge on the chip.  The splits above are
    # what is left for the scratch in memory; the two multiply.
    cluster: int = 1


@dataclass(frozen=True)
class PlanOptions:
    num_kv_heads: int
    group: int
    window: Optional[int]
    use_f32: bool
    # CTAs the step should reach before key ranges stop being split.
    target_ctas: int = 148 * 2
    # A split never gets fewer keys than this.
    min_split_keys: int = 256
    # The same for the tensor-memory family, whose CTAs walk 64 keys in 0.84 us while the merge
    # of a split through memory takes about ten: shorter splits cost more than they save
    # (a 512-token portion alone in the cache: 22.7 us a layer with splits of 256 keys, 13.5
    # without any).
    tc_min_split_keys: int = 1024
    # What cutting that family's key ranges is expected to cost a launch, in microseconds (the
    # partial rows written and read again, the merge by the last CTA of every tile).
    tc_merge_us: float = 30.0
    max_splits: int = 64
    # Portions with at most this many rows use the narrow (16-row) bf16 family.
    narrow_max_rows: int = 64
    # The same target for the narrow bf16 family, whose CTAs an SM holds fewer of
    # (None: target_ctas), and the largest cluster that may share one of its items.
    narrow_target_ctas: Optional[int] = None
    narrow_max_cluster: int = 1
    # Longer portions go to the tensor-memory family (128-row tiles) instead of the wide one.
    wide_on_tensor_memory: bool = False
    # ((cluster size, clusters of that size the device holds at a time), ...): a size is used
    # only if every (tile, KV head) of the step gets its cluster in one wave.  Empty: no limit.
    narrow_cluster_limits: Tuple[Tuple[int, int], ...] = ()
    # With a cluster, a key range is split through memory as well only if two such splits leave
    # every CTA at least this many keys (the merge through memory is the slow one, about as long
    # as sixteen key tiles of a CTA); once it is split, the merge is paid and every CTA may get
    # as few as ``narrow_global_fine_keys``.
    narrow_global_split_keys: int = 1024
    narrow_global_fine_keys: int = 512


def splits_through_memory(span, cluster: int, opt: PlanOptions):
    """How many clusters a key range of ``span`` keys (a number or an array) may be spread over
    when each cluster has ``cluster`` CTAs: one, unless two splits leave a CTA
    ``narrow_global_split_keys`` keys; then as many as leave it ``narrow_global_fine_keys``."""
    coarse = span // (cluster * max(opt.narrow_global_split_keys, 1))
    fine = span // (cluster * max(min(opt.narrow_global_fine_keys, opt.narrow_global_split_keys), 1))
    if isinstance(span, np.ndarray):
        return np.where(coarse >= 2, fine, 1)
    return fine if coarse >= 2 else 1


def tc_uniform_splits(num_tiles: int, mean_span: float, opt: PlanOptions) -> int:
    """How many key ranges every long tile of the tensor-memory family is cut into, by what the
    launch is then expected to take.  Its CTAs run two to an SM (``target_ctas`` places) and walk a
    64-key tile in about 1.46 us that way, 0.9 us alone on an SM; a launch takes as many rounds as
    its CTAs need places, each as long as one CTA's run of tiles, and splitting costs ``tc_merge_us``
    (partial rows written in float32, read again and merged by the last CTA of every tile, at the
    end of the launch).  Filling the places only by whole multiples ("as many splits as fit at
    once") leaves 160 tiles x heads of a 512-token portion on 296 places unsplit at 0.54 of the
    device; three splits run in two rounds of a third of the length, seven in four rounds of a
    seventh (measured at those sizes behind 30,000 keys: 586 us unsplit, 413 in three, 408 in
    seven).  A larger count is taken only where it is expected to save a tenth (measured: a
    2,048-token portion behind 2,048 keys is 5 % slower in three splits than in none, behind
    30,000 keys 38 % faster)."""
    ctas = num_tiles * opt.num_kv_heads
    tiles = max(mean_span, 1.0) / KEY_TILE
    places = max(opt.target_ctas, 1)
    alone = max(places // 2, 1)
    least = max(opt.tc_min_split_keys, opt.min_split_keys, 1)
    most = int(min(opt.max_splits, 16, max(mean_span // least, 1)))
    best, best_cost = 1, None
    for count in range(1, most + 1):
        total = ctas * count
        per_cta = tiles / count
        cost = per_cta * 0.9 if total <= alone else -(-total // places) * per_cta * 1.46
        if count > 1:
            cost += opt.tc_merge_us
        if best_cost is None or cost < 0.9 * best_cost:
            best, best_cost = count, cost
    return best


def choose_cluster(opt: PlanOptions, pairs: int, wanted: int) -> int:
    """Cluster size for the narrow kind when `pairs` (tile, KV head) pairs each want `wanted`
    CTAs: the largest allowed power of two that is not more than wanted and fits in one wave."""
    limits = dict(opt.narrow_cluster_limits)
    size = 1
    while size * 2 <= opt.narrow_max_cluster:
        size *= 2
    while size > 1:
        if size <= wanted and (size not in limits or pairs <= limits[size]):
            return size
        size //= 2
    return 1


def _key_range(q_len: int, kv_len: int, group: int, window: Optional[int], row_begin: int,
               row_count: int) -> Tuple[int, int]:
    ctx = kv_len - q_len
    first_tok = row_begin // group
    last_tok = (row_begin + row_count - 1) // group
    hi = ctx + last_tok + 1
    lo = max(0, ctx + first_tok - window + 1) if window else 0
    return lo, hi


def plan_attention(
    q_lens: Sequence[int],
    kv_lens: Sequence[int],
    opt: PlanOptions,
    fixed_splits: Optional[int] = None,
    fixed_cluster: int = 1,
) -> AttentionPlan:
    """Lay out one step.  ``fixed_splits`` forces that many splits for every tile (some may be
    empty) and ``fixed_cluster`` the cluster size of the narrow kind, which gives a layout whose
    shape depends on the batch size only.

    Without forced splits the layout of a long step is computed with arrays
    (``_plan_with_arrays``); the loops of ``plan_attention_plain`` say the same thing tile by
    tile, serve the short steps, and are what the tests compare the arrays with."""
    if fixed_splits is None:
        # The arrays cost about as much as forty tiles of the loops, whatever the step.
        rows = sum(q_lens) * opt.group
        if rows > _ARRAYS_FROM_TILES * TILE_ROWS[KIND_BF16_TC if opt.wide_on_tensor_memory and not opt.use_f32
                                                 else KIND_F32]:
            return _plan_with_arrays(q_lens, kv_lens, opt)
    return plan_attention_plain(q_lens, kv_lens, opt, fixed_splits, fixed_cluster)


_ARRAYS_FROM_TILES = 40


def _plan_with_arrays(q_lens: Sequence[int], kv_lens: Sequence[int], opt: PlanOptions) -> AttentionPlan:
    """``plan_attention_plain`` without forced splits, a sequence's tiles at a time."""
    group = opt.group
    q_len = np.asarray(q_lens, dtype=np.int64)
    kv_len = np.asarray(kv_lens, dtype=np.int64)[: len(q_len)]
    q_len = q_len[: len(kv_len)]
    rows = q_len * group
    if opt.use_f32:
        kind_of_seq = np.full(len(rows), KIND_F32, np.int64)
    else:
        long_kind = KIND_BF16_TC if opt.wide_on_tensor_memory else KIND_BF16_WIDE
        kind_of_seq = np.where(rows <= opt.narrow_max_rows, KIND_BF16_NARROW, long_kind)
    height_of_kind = np.zeros(max(TILE_ROWS) + 1, np.int64)
    for k, h in TILE_ROWS.items():
        height_of_kind[k] = h
    height_of_seq = height_of_kind[kind_of_seq]
    tiles_of_seq = np.where(rows > 0, -(-rows // height_of_seq), 0)
    total = int(tiles_of_seq.sum())
    if total == 0:
        return AttentionPlan()
    seq_of = np.repeat(np.arange(len(rows), dtype=np.int64), tiles_of_seq)
    first_tile_of_seq = np.cumsum(tiles_of_seq) - tiles_of_seq
    kind_of = kind_of_seq[seq_of]
    row_begin = (np.arange(total, dtype=np.int64) - first_tile_of_seq[seq_of]) * height_of_seq[seq_of]
    row_count = np.minimum(height_of_seq[seq_of], rows[seq_of] - row_begin)
    ctx = (kv_len - q_len)[seq_of]
    hi = ctx + (row_begin + row_count - 1) // group + 1
    if opt.window:
        lo = np.maximum(0, ctx + row_begin // group - opt.window + 1)
    else:
        lo = np.zeros(total, np.int64)
    span = hi - lo
    num_tiles = len(kind_of)
    base_ctas = num_tiles * opt.num_kv_heads
    narrow = kind_of == KIND_BF16_NARROW

    # CTAs a tile's key range should be spread over so that the step fills the GPU.
    target = np.full(num_tiles, opt.target_ctas, np.int64)
    if opt.narrow_target_ctas is not None:
        target[narrow] = opt.narrow_target_ctas
    least = np.where(kind_of == KIND_BF16_TC, max(opt.tc_min_split_keys, opt.min_split_keys, 1), max(opt.min_split_keys, 1))
    per_tile = np.minimum(target // max(base_ctas, 1), span // least)
    wanted = np.where(base_ctas >= target, 1, np.maximum(1, per_tile))
    on_tc = kind_of == KIND_BF16_TC
    if on_tc.any():
        # The tensor-memory family's launch is its own: one count for all its tiles, by the
        # expected time of the launch; a tile gets it as far as its own key range allows.
        uniform = tc_uniform_splits(int(on_tc.sum()), float(span[on_tc].mean()), opt)
        wanted = np.where(on_tc, np.maximum(1, np.minimum(uniform, span // least)), wanted)

    cluster = 1
    if opt.narrow_max_cluster > 1 and narrow.any():
        cluster = choose_cluster(opt, int(narrow.sum()) * opt.num_kv_heads, int(wanted[narrow].max()))
    if cluster > 1:
        through_memory = np.minimum(wanted // cluster, splits_through_memory(span, cluster, opt))
        wanted = np.where(narrow, through_memory, wanted)
    splits = np.maximum(1, np.minimum(wanted, opt.max_splits))

    # Items: one row per unsplit tile; the split tiles (few) are cut one by one, in tile order,
    # because the places of their partial rows follow that order.
    items = np.zeros((num_tiles, ITEM_WIDTH), np.int64)
    items[:, 0] = seq_of
    items[:, 1] = row_begin
    items[:, 2] = row_count
    items[:, 3] = lo
    items[:, 4] = hi
    items[:, 5] = -1
    order_key = np.arange(num_tiles, dtype=np.int64) * (opt.max_splits + 1)
    extra_rows, extra_keys, extra_kinds = [], [], []
    merges: List[List[int]] = []
    partial_rows = 0
    split_tiles = np.nonzero(splits > 1)[0]
    for t in split_tiles:
        n = int(splits[t])
        t_lo, t_hi, rows_t = int(lo[t]), int(hi[t]), int(row_count[t])
        first_tile = t_lo // KEY_TILE
        tiles_per_split = -(-(-(-t_hi // KEY_TILE) - first_tile) // n)
        stride = opt.num_kv_heads * rows_t
        merge_index = len(merges)
        merges.append([int(seq_of[t]), int(row_begin[t]), rows_t, partial_rows, n, stride, 0, 0])
        for s in range(n):
            begin = max(t_lo, (first_tile + s * tiles_per_split) * KEY_TILE)
            end = max(min(t_hi, (first_tile + (s + 1) * tiles_per_split) * KEY_TILE), begin)
            extra_rows.append([int(seq_of[t]), int(row_begin[t]), rows_t, begin, end, partial_rows, merge_index, n])
            extra_keys.append(int(order_key[t]) + s)
            extra_kinds.append(int(kind_of[t]))
            partial_rows += stride
    keep = splits <= 1
    all_items = items[keep]
    all_keys = order_key[keep]
    all_kinds = kind_of[keep]
    if extra_rows:
        all_items = np.concatenate([all_items, np.asarray(extra_rows, np.int64).reshape(-1, ITEM_WIDTH)])
        all_keys = np.concatenate([all_keys, np.asarray(extra_keys, np.int64)])
        all_kinds = np.concatenate([all_kinds, np.asarray(extra_kinds, np.int64)])

    plan = AttentionPlan(partial_rows=partial_rows, cluster=cluster)
    # Kinds appear in the order of their first tile, as the loops would meet them.
    first_seen = {}
    for k in kind_of.tolist():
        first_seen.setdefault(k, len(first_seen))
    for kind in sorted(first_seen, key=first_seen.get):
        mine = all_kinds == kind
        arr = all_items[mine][np.argsort(all_keys[mine], kind="stable")]
        if len(arr) > 1:
            # Longest key ranges first: the tail of the grid is then made of short items.
            arr = arr[np.argsort(-(arr[:, 4] - arr[:, 3]), kind="stable")]
        plan.items[int(kind)] = arr.astype(np.int32)
    if merges:
        plan.merge_items = np.asarray(merges, dtype=np.int32).reshape(-1, ITEM_WIDTH)
    return plan


def plan_attention_plain(
    q_lens: Sequence[int],
    kv_lens: Sequence[int],
    opt: PlanOptions,
    fixed_splits: Optional[int] = None,
    fixed_cluster: int = 1,
) -> AttentionPlan:
    """Lay out one step, tile by tile.  ``fixed_splits`` forces that many splits for every tile (some may be
    empty) and ``fixed_cluster`` the cluster size of the narrow kind, which gives a layout whose
    shape depends on the batch size only."""
    tiles: List[Tuple[int, int, int, int, int, int]] = []  # kind, seq, row_begin, row_count, lo, hi
    for seq, (q_len, kv_len) in enumerate(zip(q_lens, kv_lens)):
        rows = q_len * opt.group
        if rows <= 0:
            continue
        if opt.use_f32:
            kind = KIND_F32
        else:
            kind = KIND_BF16_NARROW if rows <= opt.narrow_max_rows else (
                KIND_BF16_TC if opt.wide_on_tensor_memory else KIND_BF16_WIDE)
        height = TILE_ROWS[kind]
        for row_begin in range(0, rows, height):
            row_count = min(height, rows - row_begin)
            lo, hi = _key_range(q_len, kv_len, opt.group, opt.window, row_begin, row_count)
            tiles.append((kind, seq, row_begin, row_count, lo, hi))

    base_ctas = len(tiles) * opt.num_kv_heads
    tc_spans = [hi - lo for kind, _, _, _, lo, hi in tiles if kind == KIND_BF16_TC]
    tc_uniform = tc_uniform_splits(len(tc_spans), sum(tc_spans) / len(tc_spans), opt) if tc_spans else 1

    def wanted_ctas(kind: int, span: int) -> int:
        """CTAs a tile's key range should be spread over so that the step fills the GPU."""
        if kind == KIND_BF16_TC:
            least = max(opt.tc_min_split_keys, opt.min_split_keys, 1)
            return max(1, min(tc_uniform, span // least))
        target = opt.target_ctas
        if kind == KIND_BF16_NARROW and opt.narrow_target_ctas is not None:
            target = opt.narrow_target_ctas
        if base_ctas >= target:
            return 1
        # Rounded down: the items should all be resident at once, not spill into a second wave.
        wanted = target // max(base_ctas, 1)
        least = max(opt.tc_min_split_keys, opt.min_split_keys) if kind == KIND_BF16_TC else opt.min_split_keys
        return max(1, min(wanted, span // max(least, 1)))

    # One cluster size for all items of the narrow kind (it is a property of the launch).
    cluster = 1
    if fixed_splits is not None:
        cluster = max(1, fixed_cluster)
    elif opt.narrow_max_cluster > 1:
        narrow = [wanted_ctas(k, hi - lo) for k, _, _, _, lo, hi in tiles if k == KIND_BF16_NARROW]
        if narrow:
            cluster = choose_cluster(opt, len(narrow) * opt.num_kv_heads, max(narrow))

    per_kind: Dict[int, List[List[int]]] = {}
    merges: List[List[int]] = []
    partial_rows = 0
    for kind, seq, row_begin, row_count, lo, hi in tiles:
        span = hi - lo
        if fixed_splits is not None:
            splits = fixed_splits
        else:
            wanted = wanted_ctas(kind, span)
            if kind == KIND_BF16_NARROW and cluster > 1:
                wanted = min(wanted // cluster, splits_through_memory(span, cluster, opt))
            splits = max(1, min(wanted, opt.max_splits))
        out = per_kind.setdefault(kind, [])
        if splits <= 1:
            out.append([seq, row_begin, row_count, lo, hi, -1, 0, 0])
            continue
        first_tile = lo // KEY_TILE
        num_key_tiles = -(-hi // KEY_TILE) - first_tile
        tiles_per_split = -(-num_key_tiles // splits)
        stride = opt.num_kv_heads * row_count
        merge_index = len(merges)
        merges.append([seq, row_begin, row_count, partial_rows, splits, stride, 0, 0])
        for s in range(splits):
            begin = max(lo, (first_tile + s * tiles_per_split) * KEY_TILE)
            end = min(hi, (first_tile + (s + 1) * tiles_per_split) * KEY_TILE)
            end = max(end, begin)
            out.append([seq, row_begin, row_count, begin, end, partial_rows, merge_index, splits])
            partial_rows += stride

    plan = AttentionPlan(partial_rows=partial_rows, cluster=cluster)
    for kind, rows_ in per_kind.items():
        arr = np.asarray(rows_, dtype=np.int32).reshape(-1, ITEM_WIDTH)
        if fixed_splits is None and len(arr) > 1:
            # Longest key ranges first: the tail of the grid is then made of short items.
            order = np.argsort(-(arr[:, 4] - arr[:, 3]), kind="stable")
            arr = arr[order]
        plan.items[kind] = arr
    if merges:
        plan.merge_items = np.asarray(merges, dtype=np.int32).reshape(-1, ITEM_WIDTH)
    return plan


def round_plan(plan: AttentionPlan, round_count) -> AttentionPlan:
    """The same work with every array padded to ``round_count(length)`` entries: padding work
    items and merge items have sequence -1 and do nothing.  Plans of steps that differ a little
    then have equal array sizes."""
    out = AttentionPlan(partial_rows=plan.partial_rows, cluster=plan.cluster)
    for kind, items in plan.items.items():
        padding = np.zeros((round_count(len(items)) - len(items), ITEM_WIDTH), np.int32)
        padding[:, 0] = -1
        padding[:, 5] = -1
        out.items[kind] = np.concatenate([items.astype(np.int32, copy=False), padding], axis=0)
    merges = plan.merge_items
    if len(merges):
        padding = np.zeros((round_count(len(merges)) - len(merges), ITEM_WIDTH), np.int32)
        padding[:, 0] = -1
        merges = np.concatenate([merges, padding], axis=0)
    out.merge_items = merges
    return out


def pad_plan(plan: AttentionPlan, num_seqs: int, splits: int, opt: PlanOptions) -> AttentionPlan:
    """Give a plan of single-token sequences (made with ``fixed_splits=splits``) the shape it
    would have with ``num_seqs`` sequences: missing work items are padding (seq = -1).  The
    result has the same array sizes for every real batch size up to ``num_seqs``."""
    rows = opt.group
    if opt.use_f32:
        kind = KIND_F32
    else:
        kind = KIND_BF16_NARROW if rows <= opt.narrow_max_rows else (
            KIND_BF16_TC if opt.wide_on_tensor_memory else KIND_BF16_WIDE)
    height = TILE_ROWS[kind]
    tiles = -(-rows // height)
    want_items = num_seqs * tiles * max(splits, 1)
    items = plan.items.get(kind, np.zeros((0, ITEM_WIDTH), np.int32))
    if set(plan.items) - {kind} or len(items) > want_items:
        raise ValueError("pad_plan: the plan is not one of single-token sequences")
    padding = np.zeros((want_items - len(items), ITEM_WIDTH), np.int32)
    padding[:, 0] = -1
    padding[:, 5] = -1
    out = AttentionPlan(items={kind: np.concatenate([items, padding], axis=0)}, cluster=plan.cluster)
    if splits > 1:
        want_merges = num_seqs * tiles
        merge_padding = np.zeros((want_merges - len(plan.merge_items), ITEM_WIDTH), np.int32)
        merge_padding[:, 0] = -1
        out.merge_items = np.concatenate([plan.merge_items, merge_padding], axis=0)
        out.partial_rows = want_items * opt.num_kv_heads * height
    return out


def plan_single_tokens(kv_lens: np.ndarray, num_seqs: int, splits: int, opt: PlanOptions):
    """The padded layout of a step of single tokens, computed with arrays instead of loops.

    Equal to ``pad_plan(plan_attention([1] * n, kv_lens, opt, fixed_splits=splits), ...)`` for
    groups of at most 16 query heads per KV head (one tile per sequence).  Returns
    (kind, items [num_seqs * splits, 8], merge_items [num_seqs, 8] or None, partial_rows).
    """
    if opt.group > 16:
        raise ValueError("plan_single_tokens handles one 16-row tile per sequence")
    kind = KIND_F32 if opt.use_f32 else KIND_BF16_NARROW
    n = len(kv_lens)
    splits = max(splits, 1)
    items = np.zeros((num_seqs * splits, ITEM_WIDTH), np.int32)
    items[:, 0] = -1
    items[:, 5] = -1
    kv = np.asarray(kv_lens, dtype=np.int64)
    lo = np.maximum(0, kv - opt.window) if opt.window else np.zeros_like(kv)
    if splits == 1:
        items[:n, 0] = np.arange(n)
        items[:n, 2] = opt.group
        items[:n, 3] = lo
        items[:n, 4] = kv
        return kind, items, None, 0
    stride = opt.num_kv_heads * opt.group
    first_tile = lo // KEY_TILE
    num_tiles = -(-kv // KEY_TILE) - first_tile
    per_split = -(-num_tiles // splits)
    s_idx = np.arange(splits, dtype=np.int64)[None, :]
    begin = np.maximum(lo[:, None], (first_tile[:, None] + s_idx * per_split[:, None]) * KEY_TILE)
    end = np.minimum(kv[:, None], (first_tile[:, None] + (s_idx + 1) * per_split[:, None]) * KEY_TILE)
    end = np.maximum(end, begin)
    seq = np.repeat(np.arange(n), splits)
    real = items[: n * splits]
    real[:, 0] = seq
    real[:, 2] = opt.group
    real[:, 3] = begin.reshape(-1)
    real[:, 4] = end.reshape(-1)
    real[:, 5] = np.arange(n * splits) * stride
    real[:, 6] = seq
    real[:, 7] = splits
    merges = np.zeros((num_seqs, ITEM_WIDTH), np.int32)
    merges[:, 0] = -1
    merges[:n, 0] = np.arange(n)
    merges[:n, 2] = opt.group
    merges[:n, 3] = np.arange(n) * splits * stride
    merges[:n, 4] = splits
    merges[:n, 5] = stride
    return kind, items, merges, num_seqs * splits * opt.num_kv_heads * TILE_ROWS[kind]
