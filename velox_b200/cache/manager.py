"""Cache manager: pages and block tables for every request, in every cache group.

A *cache group* is a set of layers with the same need: all keys, or a window of them.  Every
group has a pool of pages of its own (its own allocator and its own device tensors) and every
request has one block table per group.  All tables of a request have the same logical length,
because every group caches the same token positions; they differ in what has been given back:
a group with a window returns a page as soon as no later query can see any key in it, and the
table keeps ``NULL_PAGE`` in that place, so kernels index every table the same way
(``table[position // page_size]``).

Pages are given back when a request ends (``free``), when it is preempted for recompute
(``reset_for_recompute``) and when a window has passed them (``advance``).  The reference has
one group and no windows (src/block_manager.py:10-138); its capacity checks, table growth and
slot arithmetic are what this class does per group.

Beside the pages there is a pool of *state slots*: a request holds one slot from admission
to release, and anything of fixed size per request (a mixer's recurrent state, sampling state,
the row of the device block table) lives in arrays indexed by the slot.  The reference calls
this ``seq_index`` (engine/scheduler.py:58,113-129).
"""
from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence

from .allocator import NULL_PAGE, OutOfPagesError, PageAllocator


@dataclass(frozen=True)
class CacheGroup:
    """Layers that share a pool: ``window`` is None for all keys, else the number of keys seen."""

    name: str
    window: Optional[int] = None


@dataclass
class SequenceCache:
    """What one request holds in the cache: a block table per group and a state slot."""

    seq_id: str
    num_computed: int = 0
    tables: List[List[int]] = field(default_factory=list)
    # Per group, the first logical block that has not been given back yet.
    first_live: List[int] = field(default_factory=list)
    slot: Optional[int] = None
    # A number no other sequence of the process has, and a count of the changes to the tables
    # (pages appended, given back, dropped): who keeps a copy of the tables knows by the pair
    # whether the copy still holds.
    serial: int = field(default_factory=itertools.count().__next__)
    tables_version: int = 0

    @property
    def num_logical_blocks(self) -> int:
        return len(self.tables[0]) if self.tables else 0


class CacheManager:
    def __init__(
        self,
        groups: Sequence[CacheGroup],
        num_pages: int,
        page_size: int,
        max_model_len: Optional[int] = None,
        max_num_seqs: int = 1,
    ) -> None:
        if page_size <= 0 or (page_size & (page_size - 1)) != 0:
            raise ValueError(f"page_size must be a power of two, got {page_size}")
        if not groups:
            raise ValueError("a cache manager needs at least one cache group")
        self.groups: List[CacheGroup] = list(groups)
        self.page_size = page_size
        self.num_pages = num_pages
        self.allocators: List[PageAllocator] = [PageAllocator(num_pages) for _ in self.groups]

        # A pool of N pages hands out N - 1 of them (page 0 is reserved), so one request can
        # never hold more than (N - 1) * page_size tokens.  The reference counts the reserved
        # page in (src/block_manager.py:22-24) and with that admits a request that can never
        # fit and preempts itself for ever.
        capacity = max(num_pages - 1, 0) * page_size
        self.max_model_len = min(max_model_len, capacity) if max_model_len else capacity
        self.max_blocks_per_seq = -(-self.max_model_len // page_size)

        self.max_num_seqs = max_num_seqs
        self._free_slots: Deque[int] = deque(range(max_num_seqs))
        self._live: Dict[str, SequenceCache] = {}
        # Called with the sequence when it gets a slot / before it loses it.
        self.on_slot_acquired: Optional[Callable[[SequenceCache], None]] = None
        self.on_slot_released: Optional[Callable[[SequenceCache], None]] = None

    # ------------------------------------------------------------------ sequences
    def new_sequence(self, seq_id: str) -> SequenceCache:
        return SequenceCache(
            seq_id=seq_id,
            tables=[[] for _ in self.groups],
            first_live=[0 for _ in self.groups],
        )

    # ------------------------------------------------------------------ capacity
    @property
    def num_total_pages(self) -> int:
        """Usable pages of one pool (every pool has the same size)."""
        return self.num_pages - 1

    def num_free_pages(self) -> int:
        """Free pages of the fullest pool: what every group can still give."""
        return min(alloc.num_free for alloc in self.allocators)

    def pages_to_append(self, seq: SequenceCache, num_new_tokens: int) -> int:
        """New pages per group needed so that ``num_new_tokens`` more tokens have a place."""
        required = seq.num_computed + num_new_tokens
        needed = -(-required // self.page_size)
        return max(0, needed - seq.num_logical_blocks)

    def can_append(self, seq: SequenceCache, num_new_tokens: int) -> bool:
        if seq.num_computed + num_new_tokens > self.max_model_len:
            return False
        return self.pages_to_append(seq, num_new_tokens) <= self.num_free_pages()

    def append_slots(self, seq: SequenceCache, num_new_tokens: int) -> bool:
        """Grow every table of ``seq`` for ``num_new_tokens`` more tokens; all groups or none."""
        if seq.num_computed + num_new_tokens > self.max_model_len:
            return False
        extra = self.pages_to_append(seq, num_new_tokens)
        if extra == 0:
            return True
        if seq.num_logical_blocks + extra > self.max_blocks_per_seq:
            return False
        if extra > self.num_free_pages():
            return False
        for table, alloc in zip(seq.tables, self.allocators):
            table.extend(alloc.take(extra))
        seq.tables_version += 1
        self._live[seq.seq_id] = seq
        return True

    # ------------------------------------------------------------------ progress and release
    def advance(self, seq: SequenceCache, num_tokens: int) -> None:
        """Record that ``num_tokens`` more tokens are in the cache; return pages a window passed.

        The next query is at position ``num_computed`` and sees keys
        ``> num_computed - window``; a block whose last position is below that is dead for it
        and for every later query.
        """
        seq.num_computed += num_tokens
        for index, group in enumerate(self.groups):
            if group.window is None:
                continue
            first_needed = seq.num_computed - group.window + 1
            if first_needed <= 0:
                continue
            dead_blocks = min(first_needed // self.page_size, len(seq.tables[index]))
            table = seq.tables[index]
            for block in range(seq.first_live[index], dead_blocks):
                self.allocators[index].give_back(table[block])
                table[block] = NULL_PAGE
                seq.tables_version += 1
            seq.first_live[index] = max(seq.first_live[index], dead_blocks)

    def free(self, seq: SequenceCache) -> None:
        """Give back every page the sequence still holds and forget its tables."""
        for index, alloc in enumerate(self.allocators):
            table = seq.tables[index]
            for block in range(seq.first_live[index], len(table)):
                alloc.give_back(table[block])
            seq.tables[index] = []
            seq.first_live[index] = 0
        seq.tables_version += 1
        self._live.pop(seq.seq_id, None)

    def reset_for_recompute(self, seq: SequenceCache) -> None:
        """Preemption by recompute: drop the pages and start over from token 0."""
        self.free(seq)
        seq.num_computed = 0

    # ------------------------------------------------------------------ addressing
    def slot_for(self, seq: SequenceCache, group: int, position: int) -> int:
        """Flat index of a token position in the group's ``[pages * page_size]`` view."""
        page = seq.tables[group][position // self.page_size]
        return page * self.page_size + (position % self.page_size)

    # ------------------------------------------------------------------ state slots
    def acquire_slot(self, seq: SequenceCache) -> bool:
        if seq.slot is not None:
            return True
        if not self._free_slots:
            return False
        seq.slot = self._free_slots.popleft()
        if self.on_slot_acquired is not None:
            self.on_slot_acquired(seq)
        return True

    def release_slot(self, seq: SequenceCache) -> None:
        if seq.slot is None:
            return
        if self.on_slot_released is not None:
            self.on_slot_released(seq)
        self._free_slots.append(seq.slot)
        seq.slot = None

    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    # ------------------------------------------------------------------ reporting and checks
    def usage(self) -> float:
        total = self.num_total_pages
        used = max(alloc.num_used for alloc in self.allocators)
        return 0.0 if total == 0 else used / total

    def stats(self) -> Dict[str, float]:
        return {
            "total_blocks": float(self.num_total_pages),
            "free_blocks": float(self.num_free_pages()),
            "used_blocks": float(max(alloc.num_used for alloc in self.allocators)),
            "usage": self.usage(),
        }

    def assert_consistent(self) -> None:
        """Every pool is consistent and every held page is held by exactly one live table."""
        for index, alloc in enumerate(self.allocators):
            alloc.assert_consistent()
            seen: Dict[int, str] = {}
            for seq in self._live.values():
                table = seq.tables[index]
                for block in range(seq.first_live[index], len(table)):
                    page = table[block]
                    if page == NULL_PAGE:
                        raise AssertionError(f"{seq.seq_id}: live block {block} is the null page")
                    if page in seen:
                        raise AssertionError(
                            f"page {page} of group {self.groups[index].name} is held by "
                            f"{seen[page]} and {seq.seq_id}"
                        )
                    if alloc.holders(page) != 1:
                        raise AssertionError(f"page {page} has {alloc.holders(page)} holders")
                    seen[page] = seq.seq_id
                for block in range(0, seq.first_live[index]):
                    if table[block] != NULL_PAGE:
                        raise AssertionError(f"{seq.seq_id}: released block {block} still names a page")
            if len(seen) != alloc.num_used:
                raise AssertionError(
                    f"group {self.groups[index].name}: {alloc.num_used} pages in use, "
                    f"{len(seen)} found in live tables (a page was lost)"
                )
        slots = [seq.slot for seq in self._live.values() if seq.slot is not None]
        if len(set(slots)) != len(slots):
            raise AssertionError("two live sequences share a state slot")
