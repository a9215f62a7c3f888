"""Trace replay against the plain implementation: the same requests whole, with the last 32
tokens decoded one by one, in portions of changing size down to two tokens, and mixed with
other requests in a pool so small that pages are used again; in float32 and in bfloat16, on
tiny configurations that differ in every size and option."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model
import tiny_configs
from helpers import check_logits, random_prompts, read_tensors, write_model

pytestmark = pytest.mark.gpu

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# name -> (config, page size, request lengths)
CASES = {
    "tiny_a": (tiny_configs.TINY_A, 4, (5, 11, 17, 60, 100)),
    "tiny_b": (tiny_configs.TINY_B, 8, (1, 9, 33, 70, 150)),
    "tiny_w": (tiny_configs.TINY_W, 16, (40, 3, 90, 130, 64)),
    "tiny_c": (tiny_configs.TINY_C, 16, (77, 2, 35, 200, 129)),
    "tiny_d": (tiny_configs.TINY_D, 64, (130, 3, 65, 300, 64)),
}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """Model folders (bfloat16 storage, so both dtypes see the same weights) and plain logits."""
    out = {}
    for name, (cfg, page, lengths) in CASES.items():
        folder = str(tmp_path_factory.mktemp(name))
        write_model(folder, cfg, seed=21 + len(name), dtype="bfloat16")
        tensors = read_tensors(folder)
        prompts = random_prompts(cfg["vocab_size"], lengths, seed=77)
        want = [plain_model.forward_logits(tensors, cfg, p, dtype=torch.float64) for p in prompts]
        out[name] = (folder, cfg, page, prompts, want)
    return out


def make_replayer(folder, dtype, max_tokens, page, **kw):
    from velox_b200.engine.replay import TraceReplayer

    return TraceReplayer(folder, dtype, max_tokens, block_size=page, **kw)


def check(got_rows, want_rows, dtype, what):
    check_logits(got_rows, want_rows, dtype, what)


def replay_one(replayer, name, tokens, cuts):
    """Feed ``tokens`` of one request in portions ``cuts``; logits at every position."""
    rows, start = [], 0
    for step, n in enumerate(cuts):
        rec = {"step": step, "entries": [{"id": name, "tokens": tokens[start : start + n], "want": list(range(n))}],
               "end": [name] if start + n == len(tokens) else []}
        rows.append(replayer.run_step(rec))
        start += n
    assert start == len(tokens)
    return np.concatenate(rows, axis=0)


def changing_cuts(total):
    sizes = [7, 2, 16, 3, 2, 5, 33, 2, 9, 64, 4, 2, 21]
    cuts, left, i = [], total, 0
    while left > 0:
        n = min(sizes[i % len(sizes)], left)
        if left - n == 1:  # never leave a single token as a "portion": it is covered elsewhere
            n = left
        cuts.append(n)
        left -= n
        i += 1
    return cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(CASES))
def test_whole_then_decode_then_portions(models, case, dtype):
    folder, cfg, page, prompts, want = models[case]
    longest = max(len(p) for p in prompts)
    replayer = make_replayer(folder, dtype, max_tokens=max(256, -(-longest // 64) * 64), page=page)
    for index, (tokens, ref) in enumerate(zip(prompts, want)):
        L = len(tokens)
        whole = replay_one(replayer, f"w{index}", tokens, [L])
        check(whole, ref, dtype, f"{case} request {index} whole")
        tail = min(32, L - 1)
        if tail > 0:
            decoded = replay_one(replayer, f"d{index}", tokens, [L - tail] + [1] * tail)
            check(decoded, ref, dtype, f"{case} request {index} last {tail} one by one")
            if dtype == "float32":
                # same kernels, same order of sums: no split below 512 keys
                assert np.array_equal(decoded, whole), "decode differs from the whole prompt in float32"
        if L > 2:
            portions = replay_one(replayer, f"p{index}", tokens, changing_cuts(L))
            check(portions, ref, dtype, f"{case} request {index} in portions")
            if dtype == "float32":
                assert np.array_equal(portions, whole), "portions differ from the whole prompt in float32"
    replayer.cache.assert_consistent()
    assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages


def mixed_trace(prompts, rng, max_live=4):
    """Up to ``max_live`` live requests; each step feeds a portion of some and single tokens of
    others.  Returns (steps, for each request the (step, row range) of every position)."""
    progress = [0] * len(prompts)
    waiting = list(range(len(prompts)))
    live, steps = [], []
    step = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        entries, ends = [], []
        for r in list(live):
            left = len(prompts[r]) - progress[r]
            if rng.random() < 0.2 and len(live) > 1:
                continue  # this request sits the step out
            decoding = left <= 12 or rng.random() < 0.3
            n = 1 if decoding else min(left, int(rng.choice([2, 3, 5, 8, 13, 30])))
            if left - n == 0:
                ends.append(r)
            entries.append((r, progress[r], n))
            progress[r] += n
        if not entries:
            continue
        steps.append((step, entries, ends))
        for r in ends:
            live.remove(r)
        step += 1
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(CASES))
def test_mixed_batches_with_page_reuse(models, case, dtype):
    folder, cfg, page, prompts, want = models[case]
    # Twice over the requests, so that later ones run in pages earlier ones gave back.
    order = list(range(len(prompts))) * 2
    seqs = [prompts[i] for i in order]
    rng = np.random.default_rng(5)
    steps = mixed_trace(seqs, rng)
    # The four longest requests rounded up to 64 must fit; nothing more is given.
    need = sum(sorted((-(-len(p) // 64) * 64 for p in prompts), reverse=True)[:4])
    replayer = make_replayer(folder, dtype, max_tokens=need, page=page)
    used_pages = set()
    got = [np.zeros((len(p), cfg["vocab_size"]), np.float32) for p in seqs]
    for step, entries, ends in steps:
        rec = {"step": step, "end": [f"r{r}" for r in ends],
               "entries": [{"id": f"r{r}", "tokens": seqs[r][s : s + n], "want": list(range(n))} for r, s, n in entries]}
        before = {name: list(seq.tables[0]) for name, seq in replayer.live.items()}
        out = replayer.run_step(rec)
        row = 0
        for r, s, n in entries:
            got[r][s : s + n] = out[row : row + n]
            row += n
        for table in before.values():
            used_pages.update(table)
        replayer.cache.assert_consistent()
    for r, ref_index in enumerate(order):
        check(got[r], want[ref_index], dtype, f"{case} mixed request {r}")
    if dtype == "float32":
        # the second pass of a request ran in other pages beside other neighbours
        for r in range(len(prompts)):
            assert np.array_equal(got[r], got[r + len(prompts)]), f"request {r}: pages or neighbours changed its logits"
    assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
    assert len(used_pages) <= replayer.cache.num_total_pages + 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decode_with_split_key_ranges(models, dtype):
    """Decode far past the point where key ranges are split and merged."""
    folder, cfg, page, _, _ = models["tiny_c"]
    tensors = read_tensors(folder)
    tokens = random_prompts(cfg["vocab_size"], [600], seed=4)[0]
    ref = plain_model.forward_logits(tensors, cfg, tokens, dtype=torch.float64)
    replayer = make_replayer(folder, dtype, max_tokens=640, page=page,
                             plan_overrides={"min_split_keys": 64, "target_ctas": 4096})
    rows = replay_one(replayer, "long", tokens, [40] + [1] * 560)
    check(rows, ref, dtype, "long decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens(models, dtype):
    """A request's very first tokens: position 0 alone, then 1, then two at once."""
    folder, cfg, page, prompts, want = models["tiny_b"]
    replayer = make_replayer(folder, dtype, max_tokens=64, page=page)
    tokens, ref = prompts[3][:6], want[3][:6]
    rows = replay_one(replayer, "f", tokens, [1, 1, 2, 2])
    check(rows, ref, dtype, "first tokens")


def test_want_subset_and_skipped_steps(models):
    folder, cfg, page, prompts, want = models["tiny_a"]
    replayer = make_replayer(folder, "float32", max_tokens=256, page=page)
    a, b = prompts[3], prompts[2]
    out0 = replayer.run_step({"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]},
                                                     {"id": "b", "tokens": b[:5], "want": []}], "end": []})
    assert out0.shape == (2, cfg["vocab_size"])
    out1 = replayer.run_step({"step": 1, "entries": [{"id": "b", "tokens": b[5:], "want": [len(b) - 6]}], "end": ["b"]})
    out2 = replayer.run_step({"step": 2, "entries": [{"id": "a", "tokens": a[30:], "want": []}], "end": []})
    assert out2 is None
    check(out0, want[3][[0, 29]], "float32", "subset")
    check(out1, want[2][[len(b) - 1]], "float32", "after a skipped step")


def test_out_of_pages_is_an_error(models):
    folder, cfg, page, prompts, _ = models["tiny_a"]
    replayer = make_replayer(folder, "float32", max_tokens=64, page=page)
    replayer.run_step({"step": 0, "entries": [{"id": "a", "tokens": prompts[3][:60], "want": []}], "end": []})
    with pytest.raises(RuntimeError, match="no pages left"):
        replayer.run_step({"step": 1, "entries": [{"id": "b", "tokens": prompts[2], "want": []}], "end": []})


def test_trace_run_program(models, tmp_path):
    """The program itself, as a user runs it: JSON lines in, .f32 files and 'done' lines out."""
    folder, cfg, page, prompts, want = models["tiny_b"]
    a, b = prompts[2], prompts[1]
    lines = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [19]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[20:], "want": list(range(len(a) - 20))},
                                {"id": "b", "tokens": b, "want": [0, len(b) - 1]}], "end": ["a", "b"]},
        {"step": 2, "entries": [{"id": "c", "tokens": b[:2], "want": []}], "end": ["c"]},
    ]
    for dtype in ("float32", "bfloat16"):
        out_dir = tmp_path / dtype
        proc = subprocess.run(
            [os.path.join(REPO, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out_dir),
             "--max-tokens", "128"],
            input="\n".join(json.dumps(line) for line in lines) + "\n", capture_output=True, text=True, timeout=600,
        )
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [line for line in proc.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
        V = cfg["vocab_size"]
        s0 = np.fromfile(out_dir / "0.f32", dtype="<f4").reshape(-1, V)
        s1 = np.fromfile(out_dir / "1.f32", dtype="<f4").reshape(-1, V)
        assert not (out_dir / "2.f32").exists()
        check(s0, want[2][[19]], dtype, "trace_run step 0")
        expect1 = torch.cat([want[2][20:], want[1][[0, len(b) - 1]]])
        check(s1, expect1, dtype, "trace_run step 1")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_whole_and_in_large_portions(models, dtype):
    """600 tokens at once and as 300 + 300: steps above the small-step limit of the projections
    (library GEMM in bfloat16) and attention tiles far from the start of the sequence."""
    folder, cfg, page, _, _ = models["tiny_c"]
    tensors = read_tensors(folder)
    tokens = random_prompts(cfg["vocab_size"], [600], seed=14)[0]
    ref = plain_model.forward_logits(tensors, cfg, tokens, dtype=torch.float64)
    replayer = make_replayer(folder, dtype, max_tokens=640, page=page)
    check(replay_one(replayer, "whole", tokens, [600]), ref, dtype, "600 tokens whole")
    check(replay_one(replayer, "halves", tokens, [300, 300]), ref, dtype, "600 tokens as 300 + 300")


def test_decode_as_cuda_graph_matches_eager(models):
    """Single-token steps replayed as a captured graph against the same steps run eagerly:
    batches of 1 to 3 requests of different lengths, requests leaving and joining."""
    folder, cfg, page, prompts, want = models["tiny_b"]
    outs = {}
    for graphs in (True, False):
        replayer = make_replayer(folder, "bfloat16", max_tokens=512, page=page, enable_graphs=graphs)
        seqs = {"a": prompts[4], "b": prompts[3], "c": prompts[2]}
        rows = {name: [] for name in seqs}
        done = {name: 0 for name in seqs}
        heads = {"a": 100, "b": 40, "c": 20}
        replayer.run_step({"step": 0, "end": [], "entries": [
            {"id": n, "tokens": seqs[n][: heads[n]], "want": []} for n in seqs]})
        for n in seqs:
            done[n] = heads[n]
        step = 1
        while any(done[n] < len(seqs[n]) for n in seqs):
            live = [n for n in seqs if done[n] < len(seqs[n])]
            rec = {"step": step, "end": [n for n in live if done[n] + 1 == len(seqs[n])],
                   "entries": [{"id": n, "tokens": [seqs[n][done[n]]], "want": [0]} for n in live]}
            out = replayer.run_step(rec)
            for i, n in enumerate(live):
                rows[n].append(out[i])
                done[n] += 1
            step += 1
        outs[graphs] = {n: np.stack(r) for n, r in rows.items()}
        if graphs:
            assert replayer.runner._graphs and not replayer.runner._graphs_broken
    for n, ref_index in (("a", 4), ("b", 3), ("c", 2)):
        head = {"a": 100, "b": 40, "c": 20}[n]
        check(outs[True][n], want[ref_index][head:], "bfloat16", f"graph decode {n}")
        check(outs[False][n], want[ref_index][head:], "bfloat16", f"eager decode {n}")


@pytest.mark.parametrize("case", ["tiny_w", "tiny_d"])
def test_padded_step_staging_equals_prepare(models, case):
    """The captured decode step reads its arrays from fixed places; the fast path that fills
    them (it rewrites only what has changed since the same host copy was last used) must leave
    on the device exactly what the general ``prepare`` writes, step after step, while requests
    join, leave, sit steps out, grow new pages and (with a window) give pages back."""
    from velox_b200.engine.runner import StepChunk

    folder, cfg, page, prompts, _ = models[case]
    replayer = make_replayer(folder, "bfloat16", max_tokens=1024, page=page, max_live=4)
    runner, cache = replayer.runner, replayer.cache
    rng = np.random.default_rng(3)
    vocab = cfg["vocab_size"]
    heads = {"a": 70, "b": 3, "c": 33, "d": 120}
    replayer.run_step({"step": 0, "end": [], "entries": [
        {"id": name, "tokens": rng.integers(0, vocab, n).tolist(), "want": []} for name, n in heads.items()]})
    live = dict(replayer.live)
    compared = 0
    for step in range(150):
        if step == 60:  # one leaves, another of the same name comes with other pages
            seq = live.pop("b")
            cache.free(seq)
            cache.release_slot(seq)
            replayer.live.pop("b")
            replayer.run_step({"step": 1000, "end": [], "entries": [{"id": "b", "tokens": rng.integers(0, vocab, 40).tolist(), "want": []}]})
            live["b"] = replayer.live["b"]
        names = [name for name in sorted(live) if rng.random() < 0.75] or ["a"]
        chunks = []
        for name in names:
            assert cache.append_slots(live[name], 1)
            chunks.append(StepChunk(live[name], [int(rng.integers(0, vocab))], (0,)))
        bucket = runner._bucket(len(chunks))
        reach = runner._reaches[-1]
        entry = runner._graphs.get((bucket, reach))
        if entry is None or entry[2] != (runner.workspace.generation, runner._meta_generation):
            entry = runner._graphs[(bucket, reach)] = runner._capture(bucket, reach)
        where, plan_where, size = entry[3]
        # The arrays of the step; between them lie a few ints of alignment that nobody writes.
        used = torch.zeros(size, dtype=torch.bool, device="cuda")
        pieces = list(where.values())
        for entry_where, merge_where in plan_where.values():
            pieces.extend(entry_where.values())
            if merge_where is not None:
                pieces.append(merge_where)
        for offset, shape in pieces:
            used[offset : offset + int(np.prod(shape))] = True
        assert runner._fill_padded(entry, bucket, chunks)
        torch.cuda.synchronize()
        fast = runner._device_meta[:size][used]
        runner.prepare(chunks, pad_to=bucket)
        torch.cuda.synchronize()
        assert runner._last_layout[2] == size
        plain = runner._device_meta[:size][used]
        assert torch.equal(fast, plain), (step, names, torch.nonzero(fast != plain).flatten().tolist()[:10])
        compared += 1
        for name in names:
            cache.advance(live[name], 1)
    assert compared == 150


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_layouts_by_reach(models, dtype):
    """Captured single-token steps come in two layouts: one without splits through memory for
    steps whose sequences are all short, one cut for the longest sequence the engine allows.
    With the thresholds moved down to tiny sizes both are captured and used, alone and together,
    and the logits are the plain ones either way."""
    folder, cfg, page, prompts, want = models["tiny_d"]
    overrides = dict(short_reach=128, narrow_global_split_keys=32, narrow_global_fine_keys=16)
    replayer = make_replayer(folder, dtype, max_tokens=1024, page=page, plan_overrides=overrides)
    runner = replayer.runner
    assert runner._reaches == [128, 1024]
    long_index, short_index, tail = 3, 2, 12          # 300 and 65 tokens
    got = {long_index: [], short_index: []}
    step = 0

    def feed(entries, end=()):
        nonlocal step
        record = {"step": step, "end": list(end), "entries": [
            {"id": f"r{i}", "tokens": prompts[i][a:b], "want": list(range(b - a)) if b - a == 1 else []}
            for i, a, b in entries]}
        out = replayer.run_step(record)
        step += 1
        row = 0
        for i, a, b in entries:
            if b - a == 1:
                got[i].append((a, out[row]))
                row += 1

    L, S = len(prompts[long_index]), len(prompts[short_index])
    feed([(long_index, 0, L - tail), (short_index, 0, S - tail)])
    for k in range(tail // 2):                        # both: the long layout, two sequences
        feed([(long_index, L - tail + k, L - tail + k + 1), (short_index, S - tail + k, S - tail + k + 1)])
    for k in range(tail // 2, tail):                  # each alone: long and short layout, one sequence
        feed([(long_index, L - tail + k, L - tail + k + 1)])
        feed([(short_index, S - tail + k, S - tail + k + 1)])
    for index in (long_index, short_index):
        places = [a for a, _ in got[index]]
        assert places == list(range(len(prompts[index]) - tail, len(prompts[index])))
        check(np.stack([row for _, row in got[index]]), want[index][places], dtype, f"tiny_d {dtype} request {index}")
    assert not runner._graphs_broken
    if dtype == "bfloat16":  # float32 steps are not captured
        assert {key for key in runner._graphs} >= {(1, 128), (1, 1024), (2, 1024)}
        # the long layout splits through memory, the short one does not
        opt = runner._plan_options(runner._signatures[0][1])
        assert runner._padded_splits(1, opt, 1024)[0] > 1 and runner._padded_splits(1, opt, 128)[0] == 1
    runner.check_status()


@pytest.mark.parametrize("case", ["tiny_d", "tiny_w"])
def test_mixed_steps_replayed_as_graphs(models, case):
    """Steps of any shape are laid out with rounded extents and, from the second time a shape
    comes, captured and replayed.  The same mixed trace three times over: the third pass runs
    on replayed graphs and must give the logits of the plain implementation, like the first."""
    folder, cfg, page, prompts, want = models[case]
    seqs = [prompts[i] for i in (0, 2, 3, 4)]
    refs = [want[i] for i in (0, 2, 3, 4)]
    need = sum(-(-len(p) // 64) * 64 for p in seqs)
    replayer = make_replayer(folder, "bfloat16", max_tokens=need, page=page)
    runner = replayer.runner
    assert runner._mixed_graphs_on
    steps = mixed_trace(seqs, np.random.default_rng(9))
    passes = []
    for round_index in range(3):
        replayed_before = runner.kernels_replayed
        got = [np.zeros((len(p), cfg["vocab_size"]), np.float32) for p in seqs]
        for step, entries, ends in steps:
            rec = {"step": step, "end": [f"r{r}" for r in ends],
                   "entries": [{"id": f"r{r}", "tokens": seqs[r][s : s + n], "want": list(range(n))} for r, s, n in entries]}
            out = replayer.run_step(rec)
            row = 0
            for r, s, n in entries:
                got[r][s : s + n] = out[row : row + n]
                row += n
        for r, ref in enumerate(refs):
            check(got[r], ref, "bfloat16", f"{case} pass {round_index} request {r}")
        passes.append(runner.kernels_replayed - replayed_before)
        assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
    assert len(runner._mixed_graphs) > 0
    # every step of the third pass was a replay: as many kernels as steps x launches, none eager
    assert passes[2] > passes[1] > passes[0] >= 0
