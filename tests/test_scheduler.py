"""The scheduler's decisions, with a fake step: budgets, portions, order, and what happens when
pages run out."""
import pytest

from velox_b200.cache import CacheGroup, CacheManager
from velox_b200.config import SchedulerConfig
from velox_b200.engine.request import FinishReason, Request, RequestStatus
from velox_b200.engine.scheduler import Scheduler
from velox_b200.sampling.params import SamplingParams


def make(num_pages=64, page_size=4, max_num_seqs=4, budget=32, chunk=16, max_model_len=256, groups=None):
    cache = CacheManager(groups or [CacheGroup("all")], num_pages=num_pages, page_size=page_size,
                         max_model_len=max_model_len, max_num_seqs=max_num_seqs)
    config = SchedulerConfig(max_num_seqs=max_num_seqs, max_num_batched_tokens=budget,
                             max_prefill_chunk_size=chunk, max_model_len=max_model_len)
    return Scheduler(cache, config), cache


def request(name, prompt_len, max_tokens=8):
    return Request(name, list(range(1, prompt_len + 1)), SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True))


def fake_step(scheduler, cache, output, token=7):
    """What the engine does after a forward, without a model."""
    for r in output.scheduled:
        # Whoever runs in a step holds a slot and pages for all of its tokens, and is not queued
        # (a request preempted and admitted again in the same step is running again).
        assert r.cache.slot is not None and r not in scheduler.waiting
        assert r.current_chunk_size > 0
        assert r.cache.num_logical_blocks * cache.page_size >= r.num_computed_tokens + r.current_chunk_size
        completes = r.num_computed_tokens + r.current_chunk_size >= len(r.all_token_ids)
        cache.advance(r.cache, r.current_chunk_size)
        r.refresh_status()
        if completes:
            r.append_token(token)
            r.refresh_status()
            reason = r.should_stop(token, frozenset())
            if reason is not None:
                r.finish(reason)


def run_all(scheduler, cache, limit=500):
    history = []
    while scheduler.has_work() and len(history) < limit:
        out = scheduler.schedule()
        history.append(out)
        fake_step(scheduler, cache, out)
        cache.assert_consistent()
    return history


def test_prompts_are_cut_into_portions_under_the_budget():
    scheduler, cache = make(budget=20, chunk=16)
    a, b = request("a", 40), request("b", 10)
    scheduler.add_request(a)
    scheduler.add_request(b)
    out = scheduler.schedule()
    assert [(r.request_id, r.current_chunk_size) for r in out.prefill_batch] == [("a", 16), ("b", 4)]
    assert out.num_batched_tokens == 20 and not out.decode_batch
    fake_step(scheduler, cache, out)
    out = scheduler.schedule()
    assert [(r.request_id, r.current_chunk_size) for r in out.prefill_batch] == [("a", 16), ("b", 4)]
    fake_step(scheduler, cache, out)
    out = scheduler.schedule()
    # a has 8 left, b 2: both finish their prompts and will sample
    assert [(r.request_id, r.current_chunk_size) for r in out.prefill_batch] == [("a", 8), ("b", 2)]
    fake_step(scheduler, cache, out)
    assert a.status is RequestStatus.RUNNING_DECODE and len(a.output_token_ids) == 1


def test_decodes_go_first_and_cost_one_token_each():
    scheduler, cache = make(budget=10, chunk=8)
    a = request("a", 3)
    scheduler.add_request(a)
    fake_step(scheduler, cache, scheduler.schedule())
    b = request("b", 30)
    scheduler.add_request(b)
    out = scheduler.schedule()
    assert out.decode_batch == [a] and a.current_chunk_size == 1
    assert out.prefill_batch == [b] and b.current_chunk_size == 8
    assert out.scheduled == [b, a]
    fake_step(scheduler, cache, out)
    out = scheduler.schedule()
    assert out.decode_batch == [a] and b.current_chunk_size == 8  # 10 - 1 = 9, capped by the chunk size


def test_admission_is_in_order_and_limited_by_slots():
    scheduler, cache = make(max_num_seqs=2, budget=64)
    reqs = [request(f"r{i}", 5, max_tokens=2) for i in range(4)]
    for r in reqs:
        scheduler.add_request(r)
    out = scheduler.schedule()
    assert out.prefill_batch == reqs[:2] and scheduler.num_waiting == 2
    assert [r.seq_index for r in reqs[:2]] == [0, 1] and reqs[2].seq_index is None
    history = run_all(scheduler, cache)
    assert all(r.finished and r.finish_reason is FinishReason.LENGTH for r in reqs)
    assert scheduler.num_finished == 4
    assert cache.num_free_pages() == cache.num_total_pages and cache.num_free_slots == 2
    # finished requests are reaped at the start of the next schedule(), not in their last step
    first_finish = next(i for i, h in enumerate(history) if any(r.finished for r in h.scheduled))
    assert reqs[2] not in history[first_finish].scheduled


def test_head_of_line_is_never_skipped():
    # 9 usable pages of 4 tokens; watermark 1 page.  The head needs 8 pages and gets them;
    # then a 40-token request waits at the head and the short one behind it waits too.
    scheduler, cache = make(num_pages=10, budget=64, chunk=64, max_model_len=40)
    big, big2, small = request("big", 30, 2), request("big2", 30, 2), request("small", 3, 2)
    for r in (big, big2, small):
        scheduler.add_request(r)
    out = scheduler.schedule()
    assert out.prefill_batch == [big]
    assert list(scheduler.waiting) == [big2, small]


def test_watermark_keeps_pages_free_at_admission():
    scheduler, cache = make(num_pages=11, budget=64, chunk=64, max_model_len=44)  # 10 usable, watermark 1
    a = request("a", 39, 1)
    scheduler.add_request(a)
    out = scheduler.schedule()
    # 9 pages = 36 tokens may be taken at admission; the rest follows as a running prefill
    assert a.current_chunk_size == 36
    fake_step(scheduler, cache, out)
    out = scheduler.schedule()
    assert out.prefill_batch == [a] and a.current_chunk_size == 3


def test_portion_shrinks_to_the_free_pages():
    scheduler, cache = make(num_pages=13, budget=64, chunk=32, max_model_len=48)  # 12 usable
    a, b = request("a", 30, 1), request("b", 30, 1)
    scheduler.add_request(a)
    scheduler.add_request(b)
    out = scheduler.schedule()
    # a takes 30 tokens = 8 pages; 4 are free, minus the watermark: b gets 3 pages = 12 tokens
    assert [(r.request_id, r.current_chunk_size) for r in out.prefill_batch] == [("a", 30), ("b", 12)]


def test_decode_preempts_the_newest_and_it_requeues_at_the_front():
    scheduler, cache = make(num_pages=7, page_size=4, budget=64, chunk=64, max_model_len=24)  # 6 usable pages
    a, b = request("a", 8, 10), request("b", 7, 10)
    scheduler.add_request(a)
    scheduler.add_request(b)
    c = request("c", 2, 2)
    out = scheduler.schedule()
    assert out.prefill_batch == [a, b]  # a: 2 pages, b: 2 pages (8th slot free in its second page)
    fake_step(scheduler, cache, out)
    scheduler.add_request(c)
    preempted_seen = []
    for _ in range(60):
        if not scheduler.has_work():
            break
        out = scheduler.schedule()
        preempted_seen.extend(r.request_id for r in out.preempted)
        if out.preempted:
            victim = out.preempted[0]
            # recompute: nothing cached, generated tokens kept, back at the head of the queue
            # (it may be admitted again in the same schedule() when the pages allow it)
            assert victim.num_computed_tokens == 0
            if victim in out.prefill_batch:
                assert victim.status is RequestStatus.RUNNING_PREFILL
            else:
                assert victim.status is RequestStatus.PREEMPTED and victim.block_table == []
                assert scheduler.waiting[0] is victim
        fake_step(scheduler, cache, out)
        cache.assert_consistent()
    assert preempted_seen and preempted_seen[0] in ("b", "c")
    assert "a" not in preempted_seen[:1]
    assert all(r.finished for r in (a, b, c))
    assert len(a.output_token_ids) == 10 and len(b.output_token_ids) == 10
    assert scheduler.num_preemptions == len(preempted_seen)
    assert cache.num_free_pages() == cache.num_total_pages


def test_preempted_request_is_prefilled_again_with_its_generated_tokens():
    scheduler, cache = make(num_pages=6, page_size=4, budget=64, chunk=64, max_model_len=20)  # 5 usable
    a, b = request("a", 6, 8), request("b", 6, 8)
    scheduler.add_request(a)
    scheduler.add_request(b)
    seen_b_prefill_lengths = []
    for _ in range(80):
        if not scheduler.has_work():
            break
        out = scheduler.schedule()
        for r in out.prefill_batch:
            if r is b:
                seen_b_prefill_lengths.append((r.num_computed_tokens, r.current_chunk_size, len(r.all_token_ids)))
        fake_step(scheduler, cache, out)
    assert a.finished and b.finished and b.num_preemptions >= 1
    # after a preemption b starts again from token 0 and covers prompt + generated tokens
    restarts = [entry for entry in seen_b_prefill_lengths if entry[0] == 0]
    assert len(restarts) >= 2 and restarts[-1][2] > 6
    assert len(b.output_token_ids) == 8


def test_a_lone_request_that_cannot_grow_preempts_itself_and_retries():
    scheduler, cache = make(num_pages=4, page_size=4, budget=64, chunk=64, max_model_len=12)  # 3 usable = 12 tokens
    a = request("a", 6, 6)
    scheduler.add_request(a)
    history = run_all(scheduler, cache, limit=100)
    assert a.finished and len(a.output_token_ids) == 6
    assert len(history) < 100


def test_oldest_running_prefill_may_preempt_younger_ones():
    scheduler, cache = make(num_pages=9, page_size=4, budget=16, chunk=8, max_model_len=32)  # 8 usable
    a, b = request("a", 30, 1), request("b", 20, 1)
    scheduler.add_request(a)
    scheduler.add_request(b)
    preemptions = []
    for _ in range(100):
        if not scheduler.has_work():
            break
        out = scheduler.schedule()
        preemptions.extend(r.request_id for r in out.preempted)
        fake_step(scheduler, cache, out)
        cache.assert_consistent()
    assert a.finished and b.finished
    assert preemptions and set(preemptions) == {"b"}


def test_a_prefill_that_takes_pages_from_a_request_already_in_the_step():
    # a: an old long prompt; b: a younger request that is decoding.  When a's next portion needs
    # pages, b (the newest) is preempted although this step had already given it its token.
    scheduler, cache = make(num_pages=9, page_size=4, budget=16, chunk=8, max_model_len=32)
    a, b = request("a", 28, 2), request("b", 3, 20)
    scheduler.add_request(a)
    scheduler.add_request(b)
    both = []
    for _ in range(200):
        if not scheduler.has_work():
            break
        out = scheduler.schedule()
        both.extend(r.request_id for r in out.scheduled if r in scheduler.waiting or not r.cache.tables[0])
        assert out.num_batched_tokens == sum(r.current_chunk_size for r in out.scheduled)
        for r in scheduler.waiting:
            assert r.num_computed_tokens == 0 and r.cache.slot is None and r.current_chunk_size == 0
            assert r.status in (RequestStatus.WAITING, RequestStatus.PREEMPTED)
        fake_step(scheduler, cache, out)
        cache.assert_consistent()
    assert not both
    assert a.finished and b.finished and b.num_preemptions >= 1
    assert len(a.output_token_ids) == 2 and len(b.output_token_ids) == 20
    scheduler.schedule()
    assert cache.num_free_pages() == cache.num_total_pages and cache.num_free_slots == 4


def test_capacity_does_not_count_the_reserved_page():
    # 5 pages of 4: four can be handed out, so 16 tokens is the most one request can ever hold.
    scheduler, cache = make(num_pages=5, page_size=4, budget=64, chunk=64, max_model_len=64)
    assert cache.max_model_len == 16 and scheduler.config.max_model_len == 16
    with pytest.raises(ValueError, match="exceeds"):
        scheduler.add_request(request("never", 15, 2))
    fits = request("fits", 14, 2)
    scheduler.add_request(fits)
    history = run_all(scheduler, cache, limit=50)
    assert fits.finished and len(fits.output_token_ids) == 2 and len(history) < 50
    assert fits.num_preemptions == 0


def test_limits_and_abort():
    scheduler, cache = make(max_model_len=32, num_pages=64)
    with pytest.raises(ValueError, match="does not fit"):
        scheduler.add_request(request("long", 32, 1))
    with pytest.raises(ValueError, match="exceeds"):
        scheduler.add_request(request("long2", 20, 13))
    with pytest.raises(ValueError):
        Request("empty", [], SamplingParams())
    a, b = request("a", 5, 4), request("b", 5, 4)
    scheduler.add_request(a)
    scheduler.add_request(b)
    with pytest.raises(ValueError, match="already"):
        scheduler.add_request(request("a", 3, 1))
    fake_step(scheduler, cache, scheduler.schedule())
    assert scheduler.abort_request("a") and a.finish_reason is FinishReason.ABORT
    assert not scheduler.abort_request("a") and not scheduler.abort_request("zzz")
    run_all(scheduler, cache)
    assert b.finished and cache.num_free_pages() == cache.num_total_pages and cache.num_free_slots == 4


def test_pages_are_counted_in_every_group():
    groups = [CacheGroup("all"), CacheGroup("w", window=8)]
    scheduler, cache = make(num_pages=12, page_size=4, budget=64, chunk=64, max_model_len=44, groups=groups)
    reqs = [request(f"r{i}", 14, 6) for i in range(3)]
    for r in reqs:
        scheduler.add_request(r)
    run_all(scheduler, cache)
    assert all(r.finished and len(r.output_token_ids) == 6 for r in reqs)
    assert all(alloc.num_used == 0 for alloc in cache.allocators)


def test_stats():
    scheduler, cache = make()
    scheduler.add_request(request("a", 5, 2))
    stats = scheduler.stats()
    assert stats["num_waiting"] == 1 and stats["num_running"] == 0 and stats["free_blocks"] == 63


def test_single_token_layout_matches_the_general_planner():
    """The array-built layout of a padded decode step equals the looped one."""
    import numpy as np

    from velox_b200.ops import attention_plan as ap

    rng = np.random.default_rng(0)
    for trial in range(60):
        group = int(rng.choice([1, 2, 6, 8, 16]))
        kv_heads = int(rng.choice([1, 2, 5]))
        window = None if trial % 3 else int(rng.choice([1, 24, 300]))
        use_f32 = bool(trial % 2)
        bucket = int(rng.choice([1, 2, 4, 8]))
        n = int(rng.integers(0, bucket + 1))
        splits = int(rng.choice([1, 2, 3, 7, 19]))
        kv_lens = rng.integers(1, 3000, n)
        opt = ap.PlanOptions(num_kv_heads=kv_heads, group=group, window=window, use_f32=use_f32)
        slow = ap.pad_plan(ap.plan_attention([1] * n, kv_lens.tolist(), opt, fixed_splits=splits), bucket, splits, opt)
        kind, items, merges, partial_rows = ap.plan_single_tokens(kv_lens, bucket, splits, opt)
        assert list(slow.items) == [kind]
        assert np.array_equal(slow.items[kind], items), (trial, slow.items[kind][:4], items[:4])
        if splits > 1:
            assert np.array_equal(slow.merge_items, merges)
            assert slow.partial_rows == partial_rows
        else:
            assert merges is None and len(slow.merge_items) == 0


def test_attention_plan_covers_every_visible_key_exactly_once():
    """Whatever the step, the options and the splits: for every row tile, the key ranges of its
    items are disjoint, tile-aligned inside, and their union is what the tile's rows may see."""
    import numpy as np

    from velox_b200.ops import attention_plan as ap

    rng = np.random.default_rng(1)
    for trial in range(80):
        group = int(rng.choice([1, 3, 6, 7, 16, 20]))
        kv_heads = int(rng.choice([1, 2, 4]))
        window = None if trial % 4 else int(rng.choice([5, 64, 500]))
        opt = ap.PlanOptions(
            num_kv_heads=kv_heads, group=group, window=window, use_f32=bool(trial % 3 == 0),
            min_split_keys=int(rng.choice([32, 256])), target_ctas=int(rng.choice([16, 296, 5000])),
            narrow_max_cluster=int(rng.choice([1, 4, 8])), narrow_global_split_keys=int(rng.choice([32, 1024])),
            narrow_cluster_limits=((8, 15), (4, 37), (2, 74)) if trial % 2 else (),
            wide_on_tensor_memory=bool(trial % 5 == 0),
        )
        n = int(rng.integers(1, 7))
        q_lens = [int(rng.choice([1, 1, 2, 9, 70, 300])) for _ in range(n)]
        kv_lens = [q + int(rng.integers(0, 3000)) for q in q_lens]
        plan = ap.plan_attention(q_lens, kv_lens, opt)
        assert plan.cluster in (1, 2, 4, 8) and plan.cluster <= opt.narrow_max_cluster
        covered = {}
        for kind, items in plan.items.items():
            height = ap.TILE_ROWS[kind]
            for seq, row_begin, row_count, lo, hi, partial_base, merge_index, splits in items.tolist():
                assert 0 < row_count <= height and row_begin % height == 0
                assert (partial_base >= 0) == (splits > 1)
                covered.setdefault((seq, row_begin, row_count), []).append((lo, hi))
        tiles = 0
        for seq, (q_len, kv_len) in enumerate(zip(q_lens, kv_lens)):
            rows = q_len * group
            kinds = [k for k, items in plan.items.items() if (items[:, 0] == seq).any()]
            assert len(kinds) == 1
            height = ap.TILE_ROWS[kinds[0]]
            for row_begin in range(0, rows, height):
                row_count = min(height, rows - row_begin)
                ranges = sorted(r for r in covered[(seq, row_begin, row_count)] if r[1] > r[0])
                ctx = kv_len - q_len
                hi_want = ctx + (row_begin + row_count - 1) // group + 1
                lo_want = max(0, ctx + row_begin // group - window + 1) if window else 0
                assert ranges[0][0] == lo_want and ranges[-1][1] == hi_want, (trial, ranges, lo_want, hi_want)
                for (a_lo, a_hi), (b_lo, b_hi) in zip(ranges, ranges[1:]):
                    assert a_hi == b_lo and a_hi % ap.KEY_TILE == 0
                tiles += 1
        assert tiles == len(covered)


def test_cluster_size_fits_in_one_wave():
    from velox_b200.ops import attention_plan as ap

    limits = ((8, 15), (4, 37), (2, 74))
    opt = ap.PlanOptions(num_kv_heads=2, group=6, window=None, use_f32=False, narrow_max_cluster=8,
                         narrow_cluster_limits=limits)
    assert ap.choose_cluster(opt, pairs=2, wanted=74) == 8
    assert ap.choose_cluster(opt, pairs=16, wanted=9) == 4      # sixteen clusters of eight do not fit
    assert ap.choose_cluster(opt, pairs=16, wanted=3) == 2
    assert ap.choose_cluster(opt, pairs=64, wanted=2) == 2
    assert ap.choose_cluster(opt, pairs=128, wanted=2) == 1     # more pairs than clusters of two fit
    assert ap.choose_cluster(opt, pairs=4, wanted=1) == 1
    unlimited = ap.PlanOptions(num_kv_heads=2, group=6, window=None, use_f32=False, narrow_max_cluster=8)
    assert ap.choose_cluster(unlimited, pairs=500, wanted=9) == 8


def test_request_keeps_its_tokens_and_tells_its_listeners():
    r = Request("q", (4, 5, 6), SamplingParams(temperature=0.0, max_tokens=2, stop_token_ids=[9]))
    heard = []
    r.add_listener(lambda req, kind, token: heard.append((kind, token)))
    r.add_listener(lambda req, kind, token: 1 / 0)  # a listener that raises does not stop anything
    assert r.prompt_token_ids == [4, 5, 6] and r.output_token_ids == [] and r.num_tokens == 3
    assert r.num_computed_tokens == 0 and r.num_uncomputed_tokens == 3 and not r.is_decoding
    assert r.block_table == [] and r.seq_index is None and not r.finished
    r.append_token(7)
    assert r.all_token_ids == [4, 5, 6, 7] and r.output_token_ids == [7] and r.num_output_tokens == 1
    assert r.should_stop(7, frozenset()) is None
    assert r.should_stop(9, frozenset()) is FinishReason.STOP and r.should_stop(3, frozenset({3})) is FinishReason.STOP
    r.append_token(8)
    assert r.should_stop(8, frozenset()) is FinishReason.LENGTH
    r.finish(FinishReason.LENGTH)
    r.finish(FinishReason.ABORT)  # the first reason stands
    assert r.finished and r.finish_reason is FinishReason.LENGTH and r.status is RequestStatus.FINISHED
    assert heard == [("token", 7), ("token", 8), ("finish", None)]
    assert r.time_to_first_token is not None and r.time_to_first_token >= 0.0
    quiet = Request("e", [1], SamplingParams(max_tokens=5, ignore_eos=True, stop_token_ids=[2]))
    quiet.append_token(2)
    assert quiet.should_stop(2, frozenset({2})) is None  # ignore_eos: only the length ends it
    aborted = Request("a", [1])
    aborted.finish(FinishReason.ABORT)
    assert aborted.status is RequestStatus.ABORTED


@pytest.mark.parametrize("bad", [dict(n=2), dict(temperature=-0.1), dict(top_p=0.0), dict(top_p=1.01), dict(top_k=-1),
                                 dict(repetition_penalty=0.0), dict(max_tokens=0)])
def test_sampling_params_ranges(bad):
    with pytest.raises(ValueError, match=next(iter(bad))):
        SamplingParams(**bad)
    p = SamplingParams(temperature=0.0, top_k=3, presence_penalty=0.1)
    assert p.is_greedy and p.filters_candidates and p.has_penalties
    q = SamplingParams()
    assert not q.is_greedy and not q.filters_candidates and not q.has_penalties


def test_planner_with_arrays_equals_the_plain_one():
    """Long steps are laid out with arrays: the same items, merges and cluster as tile by tile."""
    import random

    import numpy as np

    from velox_b200.ops import attention_plan as ap

    rng = random.Random(5)
    for _ in range(300):
        opt = ap.PlanOptions(
            num_kv_heads=rng.choice([1, 2, 4]), group=rng.choice([1, 2, 6, 8, 20]), window=rng.choice([None, 8, 100]),
            use_f32=rng.random() < 0.2, target_ctas=rng.choice([8, 64, 296]), min_split_keys=rng.choice([64, 256]),
            max_splits=rng.choice([1, 4, 64]), narrow_max_rows=rng.choice([16, 64]), tc_min_split_keys=rng.choice([64, 1024]),
            narrow_target_ctas=rng.choice([None, 148]), narrow_max_cluster=rng.choice([1, 2, 8]),
            narrow_cluster_limits=rng.choice([(), ((8, 16), (4, 37), (2, 74))]),
            narrow_global_split_keys=rng.choice([256, 1024]), wide_on_tensor_memory=rng.random() < 0.5)
        q = [rng.choice([0, 1, 1, 2, 5, 17, 64, 300, 700]) for _ in range(rng.randint(0, 9))]
        kv = [n + rng.choice([0, 3, 100, 2000, 9000]) for n in q]
        plain, fast = ap.plan_attention_plain(q, kv, opt), ap._plan_with_arrays(q, kv, opt)
        assert (plain.partial_rows, plain.cluster, list(plain.items)) == (fast.partial_rows, fast.cluster, list(fast.items))
        for kind in plain.items:
            assert np.array_equal(plain.items[kind], fast.items[kind]) and fast.items[kind].dtype == np.int32
        assert np.array_equal(plain.merge_items, fast.merge_items) and plain.merge_items.shape == fast.merge_items.shape
        # and the public entry picks one of the two
        both = ap.plan_attention(q, kv, opt)
        assert all(np.array_equal(plain.items[kind], both.items[kind]) for kind in plain.items)


def test_rounded_plans_only_add_padding():
    import numpy as np

    from velox_b200.engine.runner import ModelRunner
    from velox_b200.ops import attention_plan as ap

    assert [ModelRunner._round_tokens(n) for n in (1, 16, 17, 128, 129, 520, 1024, 1025, 2048)] == \
        [16, 16, 32, 128, 160, 544, 1024, 1088, 2048]
    assert [ModelRunner._round_count(n) for n in (0, 1, 3, 8, 9, 24, 25)] == [0, 1, 4, 8, 16, 24, 32]
    opt = ap.PlanOptions(num_kv_heads=2, group=6, window=None, use_f32=False, target_ctas=64, narrow_max_cluster=1)
    plan = ap.plan_attention([300, 1, 1, 5], [900, 700, 64, 5], opt)
    rounded = ap.round_plan(plan, ModelRunner._round_count)
    assert rounded.partial_rows == plan.partial_rows and rounded.cluster == plan.cluster
    for kind, items in plan.items.items():
        padded = rounded.items[kind]
        assert len(padded) == ModelRunner._round_count(len(items)) and padded.dtype == np.int32
        assert np.array_equal(padded[: len(items)], items)
        assert (padded[len(items):, 0] == -1).all() and (padded[len(items):, 5] == -1).all()
    assert np.array_equal(rounded.merge_items[: len(plan.merge_items)], plan.merge_items)
    assert (rounded.merge_items[len(plan.merge_items):, 0] == -1).all()


class FakeReadback:
    """Stands in for the pinned-memory read-back: the fake sampler's values, handed over later."""

    def begin(self, tokens):
        return tokens.tolist()

    def end(self, ticket):
        return list(ticket)


class FakeTokens:
    def __init__(self, values):
        self.values = values

    def tolist(self):
        return list(self.values)


def fake_engine(scheduler, cache, runner, sampler, pipeline=True, eos=()):
    """An ``Engine`` around stand-ins for everything that needs a device."""
    from types import SimpleNamespace

    from velox_b200.engine.engine import Engine

    engine = Engine.__new__(Engine)
    engine.scheduler, engine.cache, engine.runner, engine.sampler = scheduler, cache, runner, sampler
    engine.readback, engine._flight = FakeReadback(), None
    engine.config = SimpleNamespace(pipeline_decode=pipeline)
    engine.eos_token_ids = frozenset(eos)
    engine.stats = {name: [] for name in ("scheduler_ms", "prepare_ms", "gpu_ms", "cpu_sync_wait_ms", "sampling_ms", "step_ms")}
    engine.num_steps, engine._timing = 0, False
    return engine


@pytest.mark.parametrize("pipeline", [False, True])
def test_engine_loop_with_a_fake_model(pipeline):
    """``Engine.generate`` around a runner and a sampler that are stand-ins, one step at a time
    and pipelined: portions reach the runner in order, the last token of a prompt asks for
    logits, sampled tokens come back to their requests, stop tokens and lengths end them, and
    every page returns.  Pipelined, a decoded token is fed as the stand-in that names its row in
    the step before, and a stop token costs one extra step whose token is thrown away."""
    scheduler, cache = make(num_pages=40, page_size=4, max_num_seqs=3, budget=16, chunk=8, max_model_len=64)
    seen = []
    heard = []

    class FakeRunner:
        def step(self, chunks, capture=True):
            seen.append([(c.seq.seq_id, list(c.tokens), tuple(c.want)) for c in chunks])
            return [c.seq.seq_id for c in chunks if c.want]

    class FakeSampler:
        def sample(self, logits, params, names, draw_indices, slots=None, history_lengths=None, status=None):
            assert status is None and logits == names and all(s is not None for s in slots)
            # request "s" draws its stop token as its second token; the others count upwards
            return FakeTokens([99 if name == "s" and index == 1 else 10 + index for name, index in zip(names, draw_indices)])

    engine = fake_engine(scheduler, cache, FakeRunner(), FakeSampler(), pipeline=pipeline)
    a = Request("a", list(range(1, 12)), SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
    s = Request("s", [5, 6], SamplingParams(temperature=0.0, max_tokens=9, stop_token_ids=[99]))
    for request in (a, s):
        request.add_listener(lambda r, kind, token: heard.append((r.request_id, kind, token)))
    engine.generate([a, s])
    assert a.output_token_ids == [10, 11, 12] and a.finish_reason is FinishReason.LENGTH
    assert s.output_token_ids == [10, 99] and s.finish_reason is FinishReason.STOP
    assert a.all_token_ids == list(range(1, 12)) + [10, 11, 12] and s.all_token_ids == [5, 6, 10, 99]
    # every token is announced once and in order, the end after the last token
    assert [h for h in heard if h[0] == "a"] == [("a", "token", 10), ("a", "token", 11), ("a", "token", 12), ("a", "finish", None)]
    assert [h for h in heard if h[0] == "s"] == [("s", "token", 10), ("s", "token", 99), ("s", "finish", None)]
    # first step: 8 tokens of a (a portion, no logits wanted), the whole of s (logits at its last token)
    assert seen[0] == [("a", list(range(1, 9)), ()), ("s", [5, 6], (1,))]
    # second step: prompt portions first, decoded tokens after them; s's first token was row 0
    # of the first step's sampled rows
    assert seen[1] == [("a", [9, 10, 11], (2,)), ("s", [-1 if pipeline else 10], (0,))]
    assert all(len(tokens) == 1 for step in seen[2:] for _, tokens, _ in step)
    if pipeline:
        # third step: both decode; their tokens are rows 0 (a) and 1 (s) of the second step
        assert seen[2] == [("a", [-1], (0,)), ("s", [-2], (0,))]
        # s's stop token became known after the third step had been queued with s in it; the
        # fourth step was scheduled without it
        assert [name for name, _, _ in seen[3]] == ["a"]
    else:
        assert seen[2] == [("a", [10], (0,))]
    scheduler.schedule()  # the last finished request is reaped at the next schedule()
    assert cache.num_free_pages() == cache.num_total_pages and cache.num_free_slots == 3
    assert engine.num_steps == len(seen) and not engine.has_work()


def test_pipelined_steps_deliver_one_call_later_and_drain():
    """``step_pipelined`` hands out a step's tokens during the next call; ``drain`` (and a plain
    ``step``) first finish what is on its way.  Aborting a request between two calls drops the
    token that is on its way to it."""
    scheduler, cache = make(num_pages=40, page_size=4, max_num_seqs=3, budget=16, chunk=8, max_model_len=64)

    class FakeRunner:
        def step(self, chunks, capture=True):
            return [c.seq.seq_id for c in chunks if c.want]

    class FakeSampler:
        def sample(self, logits, params, names, draw_indices, slots=None, history_lengths=None, status=None):
            return FakeTokens([100 * (1 + "abcd".index(name)) + index for name, index in zip(names, draw_indices)])

    engine = fake_engine(scheduler, cache, FakeRunner(), FakeSampler())
    a, b, c = (Request(name, [1, 2, 3], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)) for name in "abc")
    for request in (a, b, c):
        engine.add_request(request)
    d = Request("d", [1, 2, 3], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    # when a hears its second token, it takes c out: c's token of the same step is on its way
    a.add_listener(lambda r, kind, token: engine.abort_request("c") if token == 101 else None)
    engine.step_pipelined()
    assert a.output_token_ids == [] and a.num_output_tokens == 0 and engine.has_work()
    engine.step_pipelined()
    # the first step's tokens are here; the second step is queued and nothing of it is booked yet
    assert a.output_token_ids == [100] and a.num_output_tokens == 1 and a.num_computed_tokens == 3
    assert engine.abort_request("b")
    engine.step_pipelined()
    # the second step is booked and handed out; b's token of it is thrown away, c's too
    assert b.output_token_ids == [200] and b.finish_reason is FinishReason.ABORT and b.all_token_ids == [1, 2, 3, 200]
    assert c.output_token_ids == [300] and c.finish_reason is FinishReason.ABORT and c.all_token_ids == [1, 2, 3, 300]
    assert a.output_token_ids == [100, 101] and a.num_output_tokens == 2
    engine.drain()
    assert a.output_token_ids == [100, 101, 102] and a.num_output_tokens == 3 and engine._flight is None
    engine.add_request(d)
    engine.step()  # a plain step after pipelined ones: start to end
    assert a.output_token_ids == [100, 101, 102, 103] and d.output_token_ids == [400]
    engine.generate([])
    assert a.output_token_ids == [100, 101, 102, 103, 104] and a.finish_reason is FinishReason.LENGTH
    scheduler.schedule()
    assert cache.num_free_pages() == cache.num_total_pages and not engine.has_work()
    cache.assert_consistent()


def test_pipelined_requests_with_penalties_get_their_tokens_first():
    """A request whose sampler history is rebuilt from the host's token list never has a
    stand-in in that list when a step is scheduled."""
    scheduler, cache = make(num_pages=40, page_size=4, max_num_seqs=3, budget=16, chunk=8, max_model_len=64)
    fed = []

    class FakeRunner:
        def step(self, chunks, capture=True):
            fed.extend(t for c in chunks for t in c.tokens)
            return [c.seq.seq_id for c in chunks if c.want]

    class FakeSampler:
        def sample(self, logits, params, names, draw_indices, slots=None, history_lengths=None, status=None):
            return FakeTokens([7 + index for index in draw_indices])

    engine = fake_engine(scheduler, cache, FakeRunner(), FakeSampler())
    a = Request("a", [1, 2, 3], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True, repetition_penalty=1.2))
    engine.generate([a])
    assert a.output_token_ids == [7, 8, 9, 10] and all(t >= 0 for t in fed)


def test_pipelined_preemption_refeeds_the_stand_in():
    """Pages run out while a token is on its way: the victim is recomputed, and if it is taken
    up again in the very same step its portion ends with the stand-in for that token."""
    scheduler, cache = make(num_pages=7, page_size=4, max_num_seqs=2, budget=32, chunk=32, max_model_len=24)
    seen = []

    class FakeRunner:
        def step(self, chunks, capture=True):
            seen.append([(c.seq.seq_id, list(c.tokens)) for c in chunks])
            return [c.seq.seq_id for c in chunks if c.want]

    class FakeSampler:
        def sample(self, logits, params, names, draw_indices, slots=None, history_lengths=None, status=None):
            return FakeTokens([50 + index for index in draw_indices])

    for pipeline in (False, True):
        seen.clear()
        engine = fake_engine(scheduler, cache, FakeRunner(), FakeSampler(), pipeline=pipeline)
        a = Request("a" + str(pipeline), list(range(1, 10)), SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
        b = Request("b" + str(pipeline), list(range(1, 10)), SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
        engine.generate([a, b])
        assert a.output_token_ids == list(range(50, 58)) and b.output_token_ids == list(range(50, 58))
        assert scheduler.num_preemptions > 0
        # whatever was fed for a position, resolved: the prompt and then the tokens drawn
        for request in (a, b):
            assert request.all_token_ids == list(range(1, 10)) + list(range(50, 58))
        scheduler.schedule()
        assert cache.num_free_pages() == cache.num_total_pages
        cache.assert_consistent()


def test_engine_step_raises_when_the_status_word_comes_back_set():
    """The device status word rides behind the sampled tokens; a non-zero word stops the step
    before any token reaches a request, and the word is cleared."""
    from velox_b200.engine.engine import Engine

    scheduler, cache = make(num_pages=40, page_size=4, max_num_seqs=3, budget=16, chunk=8, max_model_len=64)

    class FakeTokens:
        def __init__(self, values):
            self.values = values

        def tolist(self):
            return list(self.values)

    class FakeRunner:
        status = "the-device-word"
        word = 0
        cleared = 0

        def step(self, chunks, capture=True):
            return [c.seq.seq_id for c in chunks if c.want]

        def raise_for_status(self, word):
            FakeRunner.cleared += 1
            FakeRunner.word = 0
            raise RuntimeError(f"a kernel of the step refused an access: word {word}")

    class FakeSampler:
        def sample(self, logits, params, names, draw_indices, slots=None, history_lengths=None, status=None):
            assert status == "the-device-word"
            return FakeTokens([11] * len(names) + [FakeRunner.word])

    engine = fake_engine(scheduler, cache, FakeRunner(), FakeSampler())
    a = Request("a", [1, 2, 3], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    engine.add_request(a)
    engine.step()
    assert a.output_token_ids == [11]
    FakeRunner.word = 4 | 16
    with pytest.raises(RuntimeError, match="word 20"):
        engine.step()
    assert a.output_token_ids == [11] and FakeRunner.cleared == 1
    engine.step()
    assert a.output_token_ids == [11, 11]


def test_pipelined_status_error_gives_up_the_steps_on_their_way():
    """Pipelined, a status word that comes back set belongs to a step that is already booked,
    with another queued behind it: the requests of both are taken out, whoever was not part of
    them goes on, and every page comes back."""
    scheduler, cache = make(num_pages=40, page_size=4, max_num_seqs=3, budget=16, chunk=8, max_model_len=64)
    heard = []

    class FakeRunner:
        status = "the-device-word"
        word = 0

        def step(self, chunks, capture=True):
            return [c.seq.seq_id for c in chunks if c.want]

        def raise_for_status(self, word):
            FakeRunner.word = 0
            raise RuntimeError(f"a kernel of the step refused an access: word {word}")

    class FakeSampler:
        def sample(self, logits, params, names, draw_indices, slots=None, history_lengths=None, status=None):
            return FakeTokens([11] * len(names) + [FakeRunner.word])

    engine = fake_engine(scheduler, cache, FakeRunner(), FakeSampler())
    a = Request("a", [1, 2, 3], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    b = Request("b", [1, 2, 3], SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True))
    for request in (a, b):
        request.add_listener(lambda r, kind, token: heard.append((r.request_id, kind, token)))
        engine.add_request(request)
    engine.step_pipelined()
    FakeRunner.word = 16
    engine.step_pipelined()  # the second step carries the word; the first is handed out
    assert a.output_token_ids == [11] and b.output_token_ids == [11]
    late = Request("late", [4, 5], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    with pytest.raises(RuntimeError, match="word 16"):
        engine.step_pipelined()
    # a had reached its length with the token that never came; b was in both steps
    assert a.finish_reason is FinishReason.ABORT and b.finish_reason is FinishReason.ABORT
    assert a.output_token_ids == [11] and a.all_token_ids == [1, 2, 3, 11] and b.all_token_ids == [1, 2, 3, 11]
    assert heard.count(("a", "finish", None)) == 1 and heard.count(("b", "finish", None)) == 1
    assert engine._flight is None
    engine.generate([late])
    assert late.output_token_ids == [11, 11] and late.finish_reason is FinishReason.LENGTH
    scheduler.schedule()
    assert cache.num_free_pages() == cache.num_total_pages and not engine.has_work()
    cache.assert_consistent()


def test_split_and_chunk_choices_fill_the_gpu_without_overfilling():
    """How many CTAs share an output tile (cluster split K) or a K range (chunks): pure
    arithmetic on the sizes, checked at the three model sizes the benchmarks use."""
    from velox_b200.ops import linear

    linear._NUM_SMS = 148
    try:
        # (out, in): 1.5B QKV / O / down, 7B, 14B
        few = {(2048, 1536): 8, (1536, 1536): 8, (1536, 8960): 8, (4608, 3584): 4, (3584, 3584): 8, (3584, 18944): 8,
               (7168, 5120): 4, (5120, 5120): 4, (5120, 13824): 4, (151936, 1536): 1}
        for (n, k), want in few.items():
            assert linear.choose_splits(n, k, 8) == want, (n, k)
            tiles = -(-n // 128)
            assert tiles * linear.choose_splits(n, k, 8) <= 148 * 8 // 5 or want == 1
            # wider token tiles: one CTA per SM
            assert tiles * linear.choose_splits(n, k, 64) <= 148 or linear.choose_splits(n, k, 64) == 1
        for (n, k) in few:
            for rows, per_sm in ((8, 2), (32, 2), (64, 1), (200, 1)):
                chunks = linear.choose_chunks(n, k, rows)
                token_tiles = 1 if rows <= 64 else -(-rows // (128 if rows <= 128 else 256))
                tiles = -(-n // 128) * token_tiles
                assert chunks >= 1 and (chunks == 1 or tiles * chunks <= 148 * per_sm)
                assert chunks == 1 or -(-k // 64) // chunks >= 2  # at least two K blocks a chunk
    finally:
        linear._NUM_SMS = None


def test_benchmark_command_line_options():
    from velox_b200.cli.benchmark import build_prompts, parse_args

    args = parse_args(["--model-size", "7b", "--prompt-range", "128,2048", "--rounds", "2", "--max-tokens", "256",
                       "--num-requests", "64", "--max-prefill-chunk-size", "512"])
    assert args.prompt_range == "128,2048" and args.rounds == 2 and args.model_size == "7b"
    prompts = build_prompts("mixed", 40, 1000, 4096, 3, length_range=args.prompt_range)
    lengths = [len(p) for p in prompts]
    assert len(prompts) == 40 and min(lengths) >= 128 and max(lengths) <= 2048 and len(set(lengths)) > 20
    assert all(0 <= t < 1000 for p in prompts for t in p)
    assert build_prompts("mixed", 40, 1000, 4096, 3, length_range=args.prompt_range) == prompts  # seeded
    assert [len(p) for p in build_prompts("short", 5, 50, 30, 1, fixed_len=77)] == [30] * 5  # cut to the limit
    with pytest.raises(SystemExit):
        parse_args(["--model-size", "7b", "--model", "x"])


def test_roofline_command_counts_a_layers_bytes():
    """The bytes a decode step must read of one layer: its five matrices once in bfloat16, and
    keys and values of every live request."""
    from velox_b200.cli import roofline
    from velox_b200.config.presets import model_size

    weights, cached = roofline.layer_bytes(model_size("1.5b"), batch=8, context=4096)
    assert weights == 2 * (1536 * 2048 + 1536 * 1536 + 3 * 1536 * 8960)
    assert cached == 8 * 4096 * 2 * 128 * 2 * 2
    weights, cached = roofline.layer_bytes(model_size("0.5b"), batch=1, context=10)
    assert weights == 2 * (896 * (14 + 4) * 64 + 896 * 896 + 3 * 896 * 4864) and cached == 10 * 2 * 64 * 4
    args = roofline.parse_args(["--model-size", "7b", "--batch", "1,8", "--context", "512"])
    assert (args.model_size, args.batch, args.context, args.layers, args.block_size) == ("7b", "1,8", "512", "2,6", 16)


def test_splits_through_memory_start_coarse_and_go_fine():
    import numpy as np

    from velox_b200.ops import attention_plan as ap

    opt = ap.PlanOptions(num_kv_heads=2, group=6, window=None, use_f32=False)
    assert (opt.narrow_global_split_keys, opt.narrow_global_fine_keys) == (1024, 512)
    # a cluster of eight: no split below 16,384 keys, then one per 4,096
    assert [ap.splits_through_memory(n, 8, opt) for n in (100, 8192, 16383, 16384, 32768)] == [1, 1, 1, 4, 8]
    assert ap.splits_through_memory(np.array([100, 16384, 40000]), 8, opt).tolist() == [1, 4, 9]
    assert ap.splits_through_memory(4096, 2, opt) == 4 and ap.splits_through_memory(4095, 2, opt) == 1
    # a finer start than the fine size: the start decides both
    tight = ap.PlanOptions(num_kv_heads=2, group=6, window=None, use_f32=False, narrow_global_split_keys=256)
    assert ap.splits_through_memory(4096, 8, tight) == 2 and ap.splits_through_memory(4095, 8, tight) == 1


@pytest.mark.parametrize("seed", range(6))
def test_pipelined_equals_step_by_step_under_random_traffic(seed):
    """Requests of random lengths arriving while others run, stop tokens, lengths, a pool that
    forces preemptions: the pipelined loop hands every request the tokens that one step at a
    time hands it, tells its listeners the same things in the same order, and gives every page
    back.  (The stand-in sampler draws a token from the request's name and the token's index, as
    a seeded request does.)"""
    import random

    def token_for(name, index):
        return (hash((name, index, seed)) % 50) + 1  # 1..50; 7 is everybody's stop token

    class FakeRunner:
        def __init__(self):
            self.fed = 0

        def step(self, chunks, capture=True):
            self.fed += sum(len(c.tokens) for c in chunks)
            return [c.seq.seq_id for c in chunks if c.want]

    class FakeSampler:
        def sample(self, logits, params, names, draw_indices, slots=None, history_lengths=None, status=None):
            return FakeTokens([token_for(name, index) for name, index in zip(names, draw_indices)])

    def run(pipeline):
        rng = random.Random(seed)
        scheduler, cache = make(num_pages=24, page_size=4, max_num_seqs=4, budget=24, chunk=8, max_model_len=80)
        engine = fake_engine(scheduler, cache, FakeRunner(), FakeSampler(), pipeline=pipeline)
        heard = {}
        arrivals = []
        for i in range(14):
            prompt = [rng.randrange(1, 50) for _ in range(rng.randrange(1, 30))]
            params = SamplingParams(temperature=0.0, max_tokens=rng.randrange(1, 25), stop_token_ids=[7],
                                    ignore_eos=rng.random() < 0.3)
            arrivals.append((rng.randrange(0, 40), Request(f"q{i}", prompt, params)))
        arrivals.sort(key=lambda pair: pair[0])
        requests = [r for _, r in arrivals]
        for r in requests:
            heard[r.request_id] = []
            r.add_listener(lambda req, kind, token: heard[req.request_id].append((kind, token)))
        step = engine.step_pipelined if pipeline else engine.step
        tick, waiting = 0, list(arrivals)
        while waiting or engine.has_work():
            while waiting and waiting[0][0] <= tick:
                engine.add_request(waiting.pop(0)[1])
            step()
            tick += 1
            assert tick < 5000
        engine.drain()
        scheduler.schedule()
        cache.assert_consistent()
        assert cache.num_free_pages() == cache.num_total_pages and cache.num_free_slots == 4
        return requests, heard, scheduler.num_preemptions

    want, want_heard, _ = run(False)
    got, got_heard, preemptions = run(True)
    for a, b in zip(got, want):
        assert a.request_id == b.request_id
        assert a.output_token_ids == b.output_token_ids and a.all_token_ids == b.all_token_ids, a.request_id
        assert a.finish_reason is b.finish_reason
        assert got_heard[a.request_id] == want_heard[b.request_id]
        assert all(t > 0 for t in a.all_token_ids)
        assert got_heard[a.request_id][-1] == ("finish", None)


def test_planner_splits_tensor_memory_tiles_only_into_long_ranges():
    """The 128-row family walks 64 keys in less than a microsecond and merges a split through
    memory in about ten: a 512-token portion alone in the cache is not split at all, one behind
    7,680 keys is split into ranges of at least 1,024 keys."""
    from velox_b200.ops import attention_plan as ap

    opt = ap.PlanOptions(num_kv_heads=2, group=6, window=None, use_f32=False, wide_on_tensor_memory=True,
                         narrow_max_cluster=8, target_ctas=296)
    alone = ap.plan_attention([512], [512], opt)
    assert list(alone.items) == [ap.KIND_BF16_TC] and len(alone.merge_items) == 0 and len(alone.items[ap.KIND_BF16_TC]) == 24
    behind = ap.plan_attention([512], [8192], opt)
    items = behind.items[ap.KIND_BF16_TC]
    assert len(behind.merge_items) == 24 and len(items) > 24
    spans = items[:, 4] - items[:, 3]
    assert spans.min() >= 1024 - 64 and len(items) * 2 <= 296 + 48
    # the 16-row family keeps its own, finer rule
    narrow = ap.plan_attention([1], [2048], ap.PlanOptions(num_kv_heads=2, group=6, window=None, use_f32=False,
                                                           target_ctas=296, narrow_max_cluster=1))
    assert len(narrow.merge_items) == 1 and len(narrow.items[ap.KIND_BF16_NARROW]) == 8
    # The count follows the expected time of the launch, not what fits at once: 192 CTAs with
    # 31,000 keys each run 38 % faster as three thirds in two rounds; behind 2,048 keys the merge
    # costs more than the rounds save; the 160 CTAs of a 512-token portion with 8 KV heads, which
    # would leave 136 places idle, are cut in seven (four rounds of a seventh of the length).
    assert ap.tc_uniform_splits(96, 31024.0, opt) == 3
    assert ap.tc_uniform_splits(96, 3072.0, opt) == 1
    wide = ap.PlanOptions(num_kv_heads=8, group=5, window=None, use_f32=False, wide_on_tensor_memory=True,
                          target_ctas=296)
    assert ap.tc_uniform_splits(20, 30256.0, wide) == 7
    # a merge that costs nothing: as many ranges as the least length allows
    free = ap.PlanOptions(num_kv_heads=2, group=6, window=None, use_f32=False, wide_on_tensor_memory=True,
                          target_ctas=10_000, tc_min_split_keys=64, min_split_keys=64, tc_merge_us=0.0)
    assert ap.tc_uniform_splits(12, 1200.0, free) > 4


def test_pipelined_step_that_cannot_be_queued_keeps_the_step_before():
    """The runner refuses a step (here: once, by raising): the error goes to the caller, the step
    that was on its way is still handed out by ``drain``, and the loop can go on."""
    scheduler, cache = make(num_pages=40, page_size=4, max_num_seqs=3, budget=16, chunk=8, max_model_len=64)

    class FakeRunner:
        fail_at = 2
        calls = 0

        def step(self, chunks, capture=True):
            FakeRunner.calls += 1
            if FakeRunner.calls == FakeRunner.fail_at:
                raise ValueError("no room for this step")
            return [c.seq.seq_id for c in chunks if c.want]

    class FakeSampler:
        def sample(self, logits, params, names, draw_indices, slots=None, history_lengths=None, status=None):
            return FakeTokens([30 + index for index in draw_indices])

    engine = fake_engine(scheduler, cache, FakeRunner(), FakeSampler())
    a = Request("a", [1, 2, 3], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    engine.add_request(a)
    engine.step_pipelined()
    with pytest.raises(ValueError, match="no room"):
        engine.step_pipelined()
    assert engine._flight is not None and a.output_token_ids == []
    engine.drain()
    assert a.output_token_ids == [30]
    engine.generate([])
    assert a.output_token_ids == [30, 31, 32, 33] and a.finish_reason is FinishReason.LENGTH
    scheduler.schedule()
    assert cache.num_free_pages() == cache.num_total_pages


def test_roofline_command_counts_a_portions_operations():
    """Two operations per weight and token, four per query, key and head dimension under the
    causal mask (a token sees the context and, on average, half of its own portion)."""
    from velox_b200.cli import roofline

    cfg = {"hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 160, "head_dim": 32}
    weights = 64 * (4 + 2 * 2) * 32 + 4 * 32 * 64 + 3 * 64 * 160
    assert roofline.layer_flops(cfg, 10, 0) == 2.0 * 10 * weights + 4.0 * 10 * 5.5 * 4 * 32
    assert roofline.layer_flops(cfg, 10, 100) - roofline.layer_flops(cfg, 10, 0) == 4.0 * 10 * 100 * 4 * 32


def test_timeline_command_groups_ctas_into_launches():
    """The trace is one event a CTA; a launch is as many events of one (kernel, grid) as the
    grid has CTAs, in the order the CTAs started, whatever other kernels' CTAs lie between."""
    import numpy as np

    from velox_b200.cli import timeline

    layout = np.dtype([("t0", "<u8"), ("t1", "<u8"), ("kernel", "<i4"), ("grid", "<i4"), ("block", "<i4"),
                       ("sm", "<i4"), ("m0", "<u8"), ("m1", "<u8"), ("m2", "<u8"), ("m3", "<u8")])
    assert layout.itemsize == timeline.EVENT_BYTES
    rows = [(10, 20, 12, 2, 0, 0), (11, 30, 21, 3, 0, 1), (12, 22, 12, 2, 1, 2), (13, 31, 21, 3, 1, 3),
            (14, 33, 21, 3, 2, 4), (40, 50, 12, 2, 0, 0), (41, 52, 12, 2, 1, 1), (60, 61, 21, 3, 0, 0)]
    events = np.zeros(len(rows), dtype=layout)
    for event, (t0, t1, kernel, grid, block, sm) in zip(events, rows):
        event["t0"], event["t1"], event["kernel"], event["grid"], event["block"], event["sm"] = t0, t1, kernel, grid, block, sm
    launches = timeline.group_launches(events)
    # two whole launches of kernel 12, one of kernel 21; the lone CTA of an unfinished launch is left out
    assert [(key, len(group)) for key, group in launches] == [((12, 2), 2), ((21, 3), 3), ((12, 2), 2)]
    assert [int(e["t0"]) for e in launches[1][1]] == [11, 13, 14]
    assert set(timeline.KERNEL_NAMES) >= {1, 2, 3, 10, 11, 12, 13, 14, 15, 20, 21, 22, 23}


def test_bench_refuses_more_than_one_gpu():
    """The engine is for one GPU: for N > 1 the benchmark prints one line that says so and exits with 2."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    done = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1"],
                          capture_output=True, text=True, timeout=300)
    assert done.returncode == 2
    assert len((done.stdout + done.stderr).strip().splitlines()) == 1 and "one GPU" in done.stdout + done.stderr
