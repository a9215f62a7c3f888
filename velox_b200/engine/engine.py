"""The engine: scheduler, step function and sampler in one loop, and the Python entry point.

The public surface follows the reference (engine/engine.py:105-417; README "offline" snippet):

    engine = Engine.from_pretrained(EngineConfig(model="<folder>"))
    request = Request("r0", prompt_token_ids=[...], sampling_params=SamplingParams(max_tokens=64))
    engine.generate([request])
    request.output_token_ids

plus ``add_request`` / ``step`` / ``has_work`` / ``abort_request`` / ``snapshot`` for callers
that drive the loop themselves, and ``LLM`` as a thin wrapper that takes and returns token id
lists.  One step is: schedule -> one mixed forward -> sample the rows that completed -> one
read-back of the sampled tokens (the only host wait of the step) -> bookkeeping.

``step`` does these one after the other.  ``step_pipelined`` (what ``generate`` uses unless
``EngineConfig.pipeline_decode`` is off) queues step k + 1 before it reads the tokens of step
k: everything the scheduler needs of step k is known without them (which requests got a token,
which reached their length), and the ids step k + 1 feeds for those tokens are stand-ins that
the embedding kernel resolves from the sampler's device buffer.  The host's work for a step
then runs beside the device's work for the step before.  A token that turns out to be a stop
token ends its request one step late: the extra step's token for it is thrown away.
"""
from __future__ import annotations

import json
import logging
import os
import gc
import time
from dataclasses import dataclass, field
from typing import Dict, FrozenSet, Iterable, List, Optional, Sequence, Tuple

import torch

from ..cache.manager import CacheManager
from ..cache.storage import compute_num_pages
from ..config.engine_config import EngineConfig, SchedulerConfig
from ..config.registry import architecture_of, load_model_config
from ..config.model_config import read_config_json
from ..ops import kernels
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, TokenReadback
from ..weights.loader import Checkpoint, WeightStore
from .model import CausalLM
from .request import FinishReason, Request
from .runner import ModelRunner, StepChunk
from .scheduler import Scheduler

logger = logging.getLogger(__name__)


def load_model(model_dir: str, dtype: torch.dtype, device: torch.device, max_position: Optional[int] = None):
    """Model folder -> (typed config, spec, model).  The class is chosen by config.json."""
    raw = read_config_json(model_dir)
    arch = architecture_of(raw)
    config = arch.parse_config(raw)
    spec = arch.build_spec(config)
    store = WeightStore(Checkpoint(model_dir), spec, dtype, device)
    model = CausalLM(spec, store, dtype, device, max_position=max_position)
    return config, spec, model


def _eos_token_ids(model_dir: str, spec_ids: Sequence[int]) -> FrozenSet[int]:
    path = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(path):
        try:
            with open(path, "r", encoding="utf-8") as handle:
                eos = json.load(handle).get("eos_token_id")
            if isinstance(eos, int):
                return frozenset({eos})
            if eos:
                return frozenset(int(t) for t in eos)
        except (OSError, ValueError):
            pass
    # The architecture's own ids (its config.json's, or what its spec builder falls back to); a
    # model whose folder and spec name none ends on length and stop tokens only.
    return frozenset(spec_ids)


@dataclass
class _Flight:
    """A step that is queued (or running) on the device and whose tokens the host has not read."""

    scheduled: List[Tuple[Request, int]]   # (request, tokens it was given)
    sampled: List[Request]                 # row r of the sampler's tokens is sampled[r]'s
    ticket: object = None                  # of the read-back of the tokens (and the status word)
    events: Optional[Tuple[torch.cuda.Event, torch.cuda.Event]] = None
    sampling_host_ms: float = 0.0          # the host's time to queue sampling and read-back
    committed: bool = False
    tokens: Optional[List[int]] = None     # the sampled tokens, once they have been read
    places: List[int] = field(default_factory=list)  # where each row's token goes; -1: nowhere


class Engine:
    def __init__(
        self,
        model: CausalLM,
        config: EngineConfig,
        num_pages: int,
        eos_token_ids: Optional[Iterable[int]] = None,
    ) -> None:
        config.validate()
        self.config = config
        self.model = model
        self.device = model.device
        self.eos_token_ids: FrozenSet[int] = frozenset(() if eos_token_ids is None else eos_token_ids)
        self.cache = CacheManager(
            model.cache_groups,
            num_pages=num_pages,
            page_size=config.block_size,
            max_model_len=config.max_model_len,
            max_num_seqs=config.max_num_seqs,
        )
        self.scheduler = Scheduler(
            self.cache,
            SchedulerConfig(
                max_num_seqs=config.max_num_seqs,
                max_num_batched_tokens=config.max_num_batched_tokens,
                max_prefill_chunk_size=config.max_prefill_chunk_size,
                max_model_len=config.max_model_len,
            ),
        )
        self.max_model_len = self.scheduler.config.max_model_len
        self.runner = ModelRunner(
            model,
            self.cache,
            max_num_seqs=config.max_num_seqs,
            max_num_batched_tokens=config.max_num_batched_tokens,
            enable_graphs=config.enable_cuda_graphs,
        )
        self.sampler = Sampler(
            self.device, model.vocab_size, config.max_num_seqs, self.max_model_len, seed=config.seed
        )
        runner_hook = self.cache.on_slot_acquired

        def on_slot(seq):
            if runner_hook is not None:
                runner_hook(seq)
            request = self.scheduler.requests.get(seq.seq_id)
            if request is not None:
                self.sampler.start_sequence(seq.slot, request.all_token_ids, request.sampling_params)

        self.cache.on_slot_acquired = on_slot
        # A step's ids may name a token of the step before by its row in the sampler's buffer.
        self.runner.fed_tokens = self.sampler.tokens
        # How sampled tokens (and the status word behind them) reach the host.
        self.readback = TokenReadback(config.max_num_seqs + 1)
        self._flight: Optional[_Flight] = None

        self.stats: Dict[str, List[float]] = {
            "scheduler_ms": [],
            "prepare_ms": [],
            "gpu_ms": [],
            "cpu_sync_wait_ms": [],
            "sampling_ms": [],
            "step_ms": [],
        }
        self.num_steps = 0
        self._timing = True
        # What exists now (modules, weights, the tables above) lives as long as the engine.
        # Moved to the permanent generation, it is not walked again by every full collection:
        # such a walk is a pause of some 10 ms in the middle of decoding.
        gc.collect()
        gc.freeze()

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_pretrained(cls, config: Optional[EngineConfig] = None, **overrides) -> "Engine":
        config = config or EngineConfig(**overrides)
        config.validate()
        kernels._require_cuda()
        device = torch.device(config.device)
        dtype = config.torch_dtype()
        model_config = load_model_config(config.model)
        config.max_model_len = min(config.max_model_len, model_config.max_position_embeddings)
        _, spec, model = load_model(config.model, dtype, device, max_position=config.max_model_len)
        num_pages = config.num_gpu_blocks or compute_num_pages(
            model.entry_needs,
            config.block_size,
            dtype,
            device,
            gpu_memory_utilization=config.gpu_memory_utilization,
            reserve_bytes=config.kv_cache_reserve_mb * 1024 * 1024,
        )
        # No request can use more than max_model_len tokens per sequence slot.
        most = config.max_num_seqs * (-(-config.max_model_len // config.block_size)) + 1
        if config.num_gpu_blocks is None:
            num_pages = min(num_pages, most)
        engine = cls(model, config, num_pages, _eos_token_ids(config.model, spec.eos_token_ids))
        engine.warmup()
        return engine

    def warmup(self) -> None:
        """Requests through the whole loop before the first real step, so that library handles,
        kernel images and the work buffers at their final sizes exist (the reference warms up
        and captures its decode graphs at construction too, engine/engine.py:174-211): prompts
        as long as a prefill portion, as many as fill a step (the route of long steps), two
        decoded tokens each, and then the graph of every decode bucket."""
        limit = self.max_model_len - 2
        if limit < 1:
            return
        portion = min(self.config.max_prefill_chunk_size, self.config.max_num_batched_tokens, limit)
        # As many requests as fill a step's token budget: where one request cannot be that long
        # (a short max_model_len), the step with the most tokens is still one that has been run.
        count = max(1, min(self.config.max_num_seqs, self.config.max_num_batched_tokens // max(1, portion)))
        requests = [
            Request(f"__warmup_{i}__", [0] * max(1, portion), SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
            for i in range(count)
        ]
        for request in requests:
            self.add_request(request)
        guard = 0
        while self.has_work() and guard < 16 + 2 * count:
            self.step()
            guard += 1
        for request in requests:
            self.scheduler.abort_request(request.request_id)
        self.scheduler.schedule()  # aborted requests' pages and slots go back now
        torch.cuda.synchronize(self.device)
        self.runner.capture_decode_graphs()
        torch.cuda.synchronize(self.device)
        for values in self.stats.values():
            values.clear()
        self.num_steps = 0
        self.scheduler.num_finished = 0
        self.scheduler.num_preemptions = 0
        for how in getattr(self.runner, "mixed_step_counts", {}):
            self.runner.mixed_step_counts[how] = 0

    # ------------------------------------------------------------------ requests
    def add_request(self, request: Request) -> None:
        self.scheduler.add_request(request)

    def abort_request(self, request_id: str) -> bool:
        return self.scheduler.abort_request(request_id)

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._flight is not None

    # ------------------------------------------------------------------ one step, in three parts
    def _launch(self, ahead: bool = False) -> Optional[_Flight]:
        """Schedule a step and queue it on the device: forward, sampling, and the copy of the
        sampled tokens to pinned memory.  Nothing here waits for the device.  ``ahead``: the
        step is queued behind one that is still running."""
        step_start = time.perf_counter()
        scheduled = self.scheduler.schedule()
        t_sched = time.perf_counter()
        self.stats["scheduler_ms"].append((t_sched - step_start) * 1000)
        if scheduled.is_empty():
            return None

        chunks: List[StepChunk] = []
        sampled: List[Request] = []
        given: List[Tuple[Request, int]] = []
        for request in scheduled.scheduled:
            n = request.current_chunk_size
            if request.cache.slot is None or n < 1:
                raise RuntimeError(f"{request.request_id} was scheduled without a state slot or without tokens")
            completes = request.num_computed_tokens + n >= len(request.all_token_ids)
            chunks.append(
                StepChunk(request.cache, request.tokens_for_chunk(n), want=(n - 1,) if completes else ())
            )
            given.append((request, n))
            if completes:
                sampled.append(request)

        flight = _Flight(scheduled=given, sampled=sampled)
        if self._timing:
            flight.events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            flight.events[0].record()
        logits = self.runner.step(chunks, capture=False) if ahead else self.runner.step(chunks)
        t_prepare = time.perf_counter()
        self.stats["prepare_ms"].append((t_prepare - t_sched) * 1000)
        if sampled:
            tokens_gpu = self.sampler.sample(
                logits,
                [r.sampling_params for r in sampled],
                [r.request_id for r in sampled],
                [r.num_output_tokens for r in sampled],
                slots=[r.seq_index for r in sampled],
                history_lengths=[r.num_tokens for r in sampled],
                status=getattr(self.runner, "status", None),
            )
            flight.ticket = self.readback.begin(tokens_gpu)
        if flight.events is not None:
            flight.events[1].record()
        flight.sampling_host_ms = (time.perf_counter() - t_prepare) * 1000
        return flight

    def _commit(self, flight: _Flight) -> None:
        """What follows from a queued step without its tokens: the caches hold what it was
        given, every sampled request is one token longer (a stand-in that names the sampler's
        row takes the token's place), and a request that has reached its length is over."""
        flight.committed = True
        for request, n in flight.scheduled:
            if request.finished:  # aborted, or ended by the tokens of the step before
                continue
            self.cache.advance(request.cache, n)
            request.refresh_status()
        for row, request in enumerate(flight.sampled):
            if request.finished:
                flight.places.append(-1)
                continue
            flight.places.append(request.append_pending(-1 - row))
            request.refresh_status()
            if request.num_output_tokens >= request.max_tokens:
                request.finish(FinishReason.LENGTH, announce=False)

    def _await(self, flight: _Flight) -> None:
        """Wait for the step's tokens (the one place per step where the host waits for the
        device) and look at the status word that came with them."""
        if not flight.sampled or flight.tokens is not None:
            return
        sync_start = time.perf_counter()
        tokens = self.readback.end(flight.ticket)
        word = tokens.pop() if len(tokens) > len(flight.sampled) else 0
        now = time.perf_counter()
        self.stats["cpu_sync_wait_ms"].append((now - sync_start) * 1000)
        # queueing the sampler plus the wait for its tokens (one after the other when a step is run
        # start to end; with steps queued ahead the wait is what is left of the step before)
        self.stats["sampling_ms"].append(flight.sampling_host_ms + (now - sync_start) * 1000)
        if flight.events is not None:
            self.stats["gpu_ms"].append(flight.events[0].elapsed_time(flight.events[1]))
        if word:
            # Kernels that refuse an access or give up a wait only set a bit in the device
            # status word, which rides behind the tokens; tokens drawn after that mean nothing.
            self.runner.raise_for_status(word)
        flight.tokens = tokens

    def _deliver(self, flight: _Flight) -> None:
        """Hand the tokens of a booked step to their requests."""
        for request, token, place in zip(flight.sampled, flight.tokens or (), flight.places):
            if place < 0:
                continue
            if request.finish_reason is FinishReason.ABORT:
                request.drop_pending(place)
                continue
            request.resolve_pending(place, int(token))
            reason = request.should_stop(int(token), self.eos_token_ids)
            if request.finished:
                request.announce_finish(reason)
            elif reason is not None:
                # A stop token.  If the request is part of a step that is already queued, that
                # step's token for it is dropped when it comes (the request is over by then).
                request.finish(reason)

    def _abandon(self, *flights: Optional[_Flight]) -> None:
        """Steps whose tokens cannot be trusted: their requests are taken out (stand-ins for
        tokens that will not come are dropped), so that the engine can go on with the rest."""
        for flight in flights:
            if flight is None:
                continue
            for request, place in zip(flight.sampled, flight.places):
                if place >= 0:
                    request.drop_pending(place)
            for request, _ in flight.scheduled:
                if request.finished and not request.finish_announced:
                    request.announce_finish(FinishReason.ABORT)
                self.scheduler.abort_request(request.request_id)

    def drain(self) -> None:
        """Finish the step that is on its way, if any: afterwards every token that has been
        drawn is in its request and no work is queued."""
        flight, self._flight = self._flight, None
        if flight is not None:
            self._finish_flight(flight)

    def _finish_flight(self, flight: _Flight, queued_behind: Optional[_Flight] = None) -> None:
        """Tokens of ``flight`` to their requests.  A step that has not been booked yet is only
        booked once its status word has come back clean (a refused step can then be run again);
        if it has been booked, and maybe another step queued behind it, the requests of both are
        given up before the error goes to the caller."""
        try:
            self._await(flight)
        except Exception:
            if flight.committed:
                self._abandon(flight, queued_behind)
            raise
        if not flight.committed:
            self._commit(flight)
        self._deliver(flight)

    @torch.no_grad()
    def step(self) -> None:
        """One step, start to end: when it returns, its tokens are in their requests."""
        step_start = time.perf_counter()
        self.drain()
        flight = self._launch()
        if flight is None:
            return
        self._finish_flight(flight)
        self.num_steps += 1
        self.stats["step_ms"].append((time.perf_counter() - step_start) * 1000)

    @torch.no_grad()
    def step_pipelined(self) -> None:
        """Queue the next step, then hand out the tokens of the one before it.  ``has_work``
        stays true while a step is on its way; ``drain`` ends the pipeline."""
        step_start = time.perf_counter()
        previous, self._flight = self._flight, None
        if previous is not None:
            self._commit(previous)
            # A request with penalties keeps its tokens in the sampler's history, which is
            # written from the host's list when the request (re)takes a slot: such requests
            # get their tokens before anything is scheduled.
            if any(r.sampling_params.has_penalties for r in previous.sampled):
                self._finish_flight(previous)
                previous = None
        try:
            flight = self._launch(ahead=True)
        except BaseException:
            # The step before is still on its way and booked: drain() hands its tokens out.
            self._flight = previous
            raise
        if previous is not None:
            self._finish_flight(previous, queued_behind=flight)
        self._flight = flight
        if flight is not None:
            self.num_steps += 1
            self.stats["step_ms"].append((time.perf_counter() - step_start) * 1000)

    @torch.no_grad()
    def generate(self, requests: Sequence[Request], max_steps: Optional[int] = None) -> List[Request]:
        for request in requests:
            self.add_request(request)
        one_step = self.step_pipelined if self.config.pipeline_decode else self.step
        steps = 0
        while self.has_work():
            one_step()
            steps += 1
            if max_steps is not None and steps >= max_steps:
                break
        self.drain()
        return list(requests)

    def snapshot(self) -> Dict[str, float]:
        stats = self.scheduler.stats()
        stats["num_steps"] = float(self.num_steps)
        stats["kv_cache_bytes"] = float(self.runner.kv_cache_bytes())
        for how, count in getattr(self.runner, "mixed_step_counts", {}).items():
            stats[f"mixed_steps_{how}"] = float(count)
        return stats


class LLM:
    """Token ids in, token ids out: the shortest way to generate with a model folder.

        llm = LLM("<folder>", dtype="bfloat16", max_num_seqs=8)
        outputs = llm.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0.0, max_tokens=16))
    """

    def __init__(self, model: str, **engine_options) -> None:
        self.engine = Engine.from_pretrained(EngineConfig(model=model, **engine_options))
        self._counter = 0

    def generate(
        self,
        prompt_token_ids: Sequence[Sequence[int]],
        sampling_params: Optional[SamplingParams | Sequence[SamplingParams]] = None,
    ) -> List[List[int]]:
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            params = [sampling_params or SamplingParams()] * len(prompt_token_ids)
        else:
            params = list(sampling_params)
            if len(params) != len(prompt_token_ids):
                raise ValueError("one SamplingParams per prompt, or one for all")
        requests = []
        for prompt, p in zip(prompt_token_ids, params):
            requests.append(Request(f"llm-{self._counter}", list(prompt), p))
            self._counter += 1
        self.engine.generate(requests)
        return [r.output_token_ids for r in requests]
