"""Who runs in the next step, and with how many tokens.

The policy is the reference scheduler's (engine/scheduler.py:136-291 of that project), because
its decisions are what a user of that engine observes:

  1. requests that ended in the last step give their pages and their slot back now, not before;
  2. every decoding request gets its one token first, while the step's token budget lasts;
  3. requests in the middle of their prompt get their next portion: what is left, cut to the
     budget, to ``max_prefill_chunk_size`` and to the pages that are free;
  4. new requests are admitted from the head of the queue, in arrival order and without ever
     passing over the head, while a state slot is free and the pools stay above a watermark.

Pages run out in three ways, with three answers.  A decode that cannot grow takes pages from
the request that started running last, then the one before, until it fits; if it reaches
itself it gives up and is the one preempted.  The prompt portion of the request that has been
running longest may do the same; younger ones sit the step out.  A victim that had already been
given its token in this step loses it again (the reference leaves such a request in the step's
batch with empty tables, engine/scheduler.py:241-244 there).  A newcomer never takes
anything.  Preempting is recomputing: the victim's pages go back, nothing of it counts as
computed, it keeps what it has generated and goes to the front of the queue, and when it is
admitted again prompt and generated tokens are prefilled as one prompt.

With several cache groups a token needs a place in every pool, so free pages are always those
of the fullest pool (``CacheManager.num_free_pages``).

Here the step is assembled by a ``_StepPlan`` (budget, the three lists) that the three phases
fill in turn; the scheduler itself only holds the queues and the counters.
"""
from __future__ import annotations

import logging
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Iterator, List, Optional

from ..cache.manager import CacheManager
from ..config.engine_config import SchedulerConfig
from .request import FinishReason, Request, RequestStatus

_log = logging.getLogger(__name__)


@dataclass
class SchedulerOutput:
    """One step's work: portions of prompts, single decoded tokens, and who was preempted."""

    prefill_batch: List[Request] = field(default_factory=list)
    decode_batch: List[Request] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    num_batched_tokens: int = 0

    @property
    def scheduled(self) -> List[Request]:
        """All requests of the step: prompt portions first, decoded tokens after them."""
        return [*self.prefill_batch, *self.decode_batch]

    def is_empty(self) -> bool:
        return len(self.prefill_batch) + len(self.decode_batch) == 0


class _StepPlan:
    """The step under construction: what is left of the token budget, and the output."""

    def __init__(self, budget: int) -> None:
        self.budget = budget
        self.out = SchedulerOutput()

    def give(self, request: Request, tokens: int, decoding: bool) -> None:
        request.current_chunk_size = tokens
        (self.out.decode_batch if decoding else self.out.prefill_batch).append(request)
        self.out.num_batched_tokens += tokens
        self.budget -= tokens

    def take_back(self, request: Request) -> None:
        """Undo ``give``: a request that was given work earlier in this step and has now lost
        its pages runs nothing, and its tokens return to the budget."""
        for batch in (self.out.decode_batch, self.out.prefill_batch):
            if request in batch:
                batch.remove(request)
                self.out.num_batched_tokens -= request.current_chunk_size
                self.budget += request.current_chunk_size
        request.current_chunk_size = 0


class Scheduler:
    def __init__(self, cache: CacheManager, config: Optional[SchedulerConfig] = None) -> None:
        self.cache = cache
        self.config = SchedulerConfig() if config is None else config
        # No request may be longer than what one request's block table can address.
        self.config.max_model_len = min(self.config.max_model_len, cache.max_model_len)
        self.requests: Dict[str, Request] = {}
        self.waiting: Deque[Request] = deque()  # arrival order; preempted requests at the front
        self.running: List[Request] = []        # in the order they started running
        self.num_finished = 0
        self.num_preemptions = 0
        # Newcomers leave this many pages of every pool alone.
        self._watermark_pages = max(1, int(self.config.watermark * cache.num_total_pages))
        # Told about every request that leaves for good (finished or aborted).
        self.on_request_released: Optional[Callable[[Request], None]] = None

    # ------------------------------------------------------------------ requests in and out
    def add_request(self, request: Request) -> None:
        longest = self.config.max_model_len
        prompt, wanted = request.num_prompt_tokens, request.sampling_params.max_tokens
        if request.request_id in self.requests:
            raise ValueError(f"there is already a request called {request.request_id!r}")
        if prompt >= longest:
            raise ValueError(
                f"a prompt of {prompt} tokens does not fit: max_model_len={longest} must leave room to generate")
        if prompt + wanted > longest:
            raise ValueError(
                f"{prompt} prompt tokens with max_tokens={wanted}: that exceeds max_model_len={longest}")
        request.cache = self.cache.new_sequence(request.request_id)
        self.requests[request.request_id] = request
        self.waiting.append(request)

    def get_request(self, request_id: str) -> Optional[Request]:
        return self.requests.get(request_id)

    def abort_request(self, request_id: str) -> bool:
        """Take a live request out at once; False if there is none of that name."""
        request = self.requests.get(request_id)
        if request is None or request.finished:
            return False
        request.finish(FinishReason.ABORT)
        for queue in (self.waiting, self.running):
            if request in queue:
                queue.remove(request)
        self._let_go(request)
        return True

    def has_work(self) -> bool:
        return len(self.waiting) > 0 or len(self.running) > 0

    @property
    def num_running(self) -> int:
        return len(self.running)

    @property
    def num_waiting(self) -> int:
        return len(self.waiting)

    def stats(self) -> Dict[str, float]:
        own = {"num_running": len(self.running), "num_waiting": len(self.waiting),
               "num_preemptions": self.num_preemptions, "num_finished": self.num_finished}
        return {**{name: float(value) for name, value in own.items()}, **self.cache.stats()}

    # ------------------------------------------------------------------ a step
    def schedule(self) -> SchedulerOutput:
        self._collect_finished()
        plan = _StepPlan(self.config.max_num_batched_tokens)
        self._continue_decodes(plan)
        self._continue_prompts(plan)
        self._admit(plan)
        return plan.out

    def _running_as(self, status: RequestStatus) -> Iterator[Request]:
        """The running requests in that status, oldest first; safe against preemptions that
        happen while the caller walks them."""
        for request in tuple(self.running):
            if request.status is status and request in self.running:
                yield request

    def _collect_finished(self) -> None:
        still_running = [r for r in self.running if not r.finished]
        for request in self.running:
            if request.finished:
                self.num_finished += 1
                self._let_go(request)
        self.running = still_running

    def _continue_decodes(self, plan: _StepPlan) -> None:
        for request in self._running_as(RequestStatus.RUNNING_DECODE):
            if plan.budget < 1:
                return
            if self._free_pages_for(request, 1, plan) and self.cache.append_slots(request.cache, 1):
                plan.give(request, 1, decoding=True)
            elif request in self.running:
                self._preempt(request, plan)

    def _continue_prompts(self, plan: _StepPlan) -> None:
        longest_running = True
        for request in self._running_as(RequestStatus.RUNNING_PREFILL):
            if plan.budget < 1:
                return
            may_take, longest_running = longest_running, False
            tokens = self._portion(request, plan.budget, self.cache.num_free_pages())
            # Only the request that has waited longest takes pages from others, newest first.
            while tokens == 0 and may_take and self.running[-1] is not request:
                self._preempt(self.running[-1], plan)
                tokens = self._portion(request, plan.budget, self.cache.num_free_pages())
            if tokens > 0 and self.cache.append_slots(request.cache, tokens):
                plan.give(request, tokens, decoding=False)

    def _admit(self, plan: _StepPlan) -> None:
        while plan.budget > 0 and self.waiting and len(self.running) < self.config.max_num_seqs:
            head = self.waiting[0]
            if not self.cache.acquire_slot(head.cache):
                return
            tokens = self._portion(head, plan.budget, self.cache.num_free_pages() - self._watermark_pages)
            if tokens == 0 or not self.cache.append_slots(head.cache, tokens):
                # Not now.  Nobody behind the head goes first, so admission ends for this step.
                self.cache.reset_for_recompute(head.cache)
                self.cache.release_slot(head.cache)
                return
            self.waiting.popleft()
            self.running.append(head)
            head.status = RequestStatus.RUNNING_PREFILL
            plan.give(head, tokens, decoding=False)

    # ------------------------------------------------------------------ sizes
    def _portion(self, request: Request, budget: int, spare_pages: int) -> int:
        """Tokens of its prompt the request gets now: what it still lacks, within the budget and
        the portion size, and within the pages it has plus ``spare_pages`` more per pool."""
        cache = self.cache
        done = request.num_computed_tokens
        pages = min(request.cache.num_logical_blocks + max(spare_pages, 0), cache.max_blocks_per_seq)
        fits = min(pages * cache.page_size, cache.max_model_len) - done
        wanted = min(request.num_uncomputed_tokens, budget, self.config.max_prefill_chunk_size)
        return max(0, min(wanted, fits))

    # ------------------------------------------------------------------ giving back
    def _let_go(self, request: Request) -> None:
        """The request leaves for good: pages, slot, its entry, and a word to whoever listens."""
        self.cache.free(request.cache)
        self.cache.release_slot(request.cache)
        self.requests.pop(request.request_id, None)
        if self.on_request_released is not None:
            self.on_request_released(request)

    def _preempt(self, victim: Request, plan: _StepPlan) -> None:
        """Recompute later: pages and slot go back, the request goes to the front of the queue."""
        plan.take_back(victim)
        self.cache.reset_for_recompute(victim.cache)
        self.cache.release_slot(victim.cache)
        if victim in self.running:
            self.running.remove(victim)
        victim.status = RequestStatus.PREEMPTED
        victim.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(victim)
        plan.out.preempted.append(victim)
        _log.debug("%s preempted (%d preemptions so far)", victim.request_id, self.num_preemptions)

    def _free_pages_for(self, request: Request, tokens: int, plan: _StepPlan) -> bool:
        """Make ``request`` able to grow by ``tokens``, taking from the newest running request
        first.  The newest is taken even when it is ``request`` itself (then False): reaching
        past it to an older one would let late arrivals starve early ones."""
        while not self.cache.can_append(request.cache, tokens):
            if not self.running:
                return False
            newest = self.running[-1]
            self._preempt(newest, plan)
            if newest is request:
                return False
        return True
