"""Generation through the Python entry point: greedy tokens against the plain implementation,
batched against one at a time, preemption under page pressure, seeded sampling, limits."""
import numpy as np
import os

import pytest
import torch

import plain_model
import tiny_configs
from helpers import random_prompts, read_tensors, write_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in (("tiny_a", tiny_configs.TINY_A), ("tiny_b", tiny_configs.TINY_B), ("tiny_w", tiny_configs.TINY_W),
                      ("tiny_d", tiny_configs.TINY_D)):
        folder = str(tmp_path_factory.mktemp(name))
        write_model(folder, cfg, seed=31, dtype="bfloat16")
        out[name] = (folder, cfg, read_tensors(folder))
    return out


def build_engine(folder, dtype="float32", **kw):
    from velox_b200.config import EngineConfig
    from velox_b200.engine.engine import Engine

    options = dict(model=folder, dtype=dtype, max_model_len=128, max_num_seqs=4, max_num_batched_tokens=64,
                   max_prefill_chunk_size=16, block_size=4, num_gpu_blocks=200, seed=0)
    options.update(kw)
    return Engine.from_pretrained(EngineConfig(**options))


def make_requests(prompts, **params):
    from velox_b200.engine.request import Request
    from velox_b200.sampling.params import SamplingParams

    return [Request(f"r{i}", p, SamplingParams(ignore_eos=True, **params)) for i, p in enumerate(prompts)]


def teacher_forced_argmax(tensors, cfg, request):
    """What greedy decoding must have produced, given what it did produce before each token."""
    full = request.all_token_ids
    logits = plain_model.forward_logits(tensors, cfg, full[:-1], dtype=torch.float64)
    return logits[request.num_prompt_tokens - 1 :].argmax(-1).tolist()


@pytest.mark.parametrize("case,page,chunk", [("tiny_a", 4, 32), ("tiny_a", 4, 3), ("tiny_b", 8, 16), ("tiny_w", 16, 7)])
def test_greedy_generation_matches_plain(folders, case, page, chunk):
    folder, cfg, tensors = folders[case]
    engine = build_engine(folder, "float32", block_size=page, max_prefill_chunk_size=chunk)
    prompts = random_prompts(cfg["vocab_size"], (5, 11, 17, 40), seed=1)
    requests = make_requests(prompts, temperature=0.0, max_tokens=8)
    engine.generate(requests)
    for request in requests:
        assert request.finish_reason.value == "length"
        assert len(request.output_token_ids) == 8
        assert request.output_token_ids == teacher_forced_argmax(tensors, cfg, request)
    engine.scheduler.schedule()  # reaps the finished requests
    engine.cache.assert_consistent()
    assert engine.cache.num_free_pages() == engine.cache.num_total_pages
    assert engine.cache.num_free_slots == engine.config.max_num_seqs


def test_greedy_generation_bfloat16_tracks_plain(folders):
    folder, cfg, tensors = folders["tiny_b"]
    engine = build_engine(folder, "bfloat16", block_size=8)
    prompts = random_prompts(cfg["vocab_size"], (9, 33, 70), seed=2)
    requests = make_requests(prompts, temperature=0.0, max_tokens=12)
    engine.generate(requests)
    for request in requests:
        full = request.all_token_ids
        logits = plain_model.forward_logits(tensors, cfg, full[:-1], dtype=torch.float64)
        rows = logits[request.num_prompt_tokens - 1 :]
        for row, token in zip(rows, request.output_token_ids):
            # the chosen token is the plain argmax, or within bfloat16 noise of it
            assert row[token] >= row.max() - 3e-2 * row.abs().max()


def within_bfloat16_noise_of_plain_argmax(tensors, cfg, request):
    """Every generated token, given the tokens before it, is the plain argmax or within
    bfloat16 noise of it."""
    full = request.all_token_ids
    logits = plain_model.forward_logits(tensors, cfg, full[:-1], dtype=torch.float64)
    rows = logits[request.num_prompt_tokens - 1 :]
    assert len(rows) == len(request.output_token_ids)
    for index, (row, token) in enumerate(zip(rows, request.output_token_ids)):
        assert row[token] >= row.max() - 3e-2 * row.abs().max(), (request.request_id, index)


@pytest.mark.parametrize("case,page,pages,lengths,tokens", [
    # Heads of 128 dims: the fused projection / rotation / cache write, the norm inside the
    # projections, the one-kernel feed-forward, clusters in captured graphs.  64-key pages;
    # every request ends with about 230 tokens = 4 pages, and 11 usable pages cannot hold four.
    ("tiny_d", 64, 12, (150, 130, 171, 140), 70),
    ("tiny_b", 8, 41, (60, 56, 52, 66), 80),
])
def test_bfloat16_preemption_with_graphs(folders, case, page, pages, lengths, tokens):
    folder, cfg, tensors = folders[case]
    prompts = random_prompts(cfg["vocab_size"], lengths, seed=12)
    longest = max(lengths) + tokens
    engine = build_engine(folder, "bfloat16", block_size=page, num_gpu_blocks=pages, max_model_len=-(-longest // page) * page,
                          max_num_batched_tokens=128, max_prefill_chunk_size=64, enable_cuda_graphs=True)
    assert engine.runner.enable_graphs
    requests = make_requests(prompts, temperature=0.0, max_tokens=tokens)
    engine.generate(requests)
    assert engine.scheduler.num_preemptions > 0
    assert engine.runner._graphs and not engine.runner._graphs_broken and engine.runner.kernels_replayed > 0
    for request in requests:
        assert len(request.output_token_ids) == tokens and request.finish_reason.value == "length"
        within_bfloat16_noise_of_plain_argmax(tensors, cfg, request)
    engine.scheduler.schedule()
    engine.cache.assert_consistent()
    assert engine.cache.num_free_pages() == engine.cache.num_total_pages
    assert engine.cache.num_free_slots == engine.config.max_num_seqs
    engine.runner.check_status()


def test_bfloat16_seeded_temperature_workload(folders):
    """Prompts of 1, 9, 33 and 70 tokens, portions of 16 mixed with decoding, 12 tokens at
    temperature 0.8 under fixed seeds: the same tokens on a second run, and for each request
    alone as in the batch (its draws depend on its seed and token index only; its logits on
    the batch only within bfloat16 rounding)."""
    folder, cfg, _ = folders["tiny_b"]
    prompts = random_prompts(cfg["vocab_size"], (1, 9, 33, 70), seed=5)
    from velox_b200.engine.request import Request
    from velox_b200.sampling.params import SamplingParams

    def run(engine, subset):
        requests = [
            Request(f"s{i}", prompts[i], SamplingParams(temperature=0.8, seed=7 + i, max_tokens=12, ignore_eos=True))
            for i in subset
        ]
        engine.generate(requests)
        return {i: r.output_token_ids for i, r in zip(subset, requests)}

    engine = build_engine(folder, "bfloat16", block_size=8, max_model_len=192, max_prefill_chunk_size=16)
    together = run(engine, [0, 1, 2, 3])
    assert all(len(v) == 12 for v in together.values())
    # Three of four, not four: the one-kernel feed-forward of small steps adds its shares in no
    # fixed order, so the last bit of a bfloat16 logit can differ between runs, and a draw
    # whose two best scores sit within that bit may then fall the other way.
    again = run(engine, [0, 1, 2, 3])
    assert sum(again[i] == together[i] for i in range(4)) >= 3, "a second run drew different tokens"
    agree = sum(run(engine, [i])[i] == together[i] for i in range(4))
    assert agree >= 3, "alone and in the batch, seeded requests drew different tokens"


def test_bfloat16_generation_at_head_size_128(folders):
    folder, cfg, tensors = folders["tiny_d"]
    engine = build_engine(folder, "bfloat16", block_size=64, num_gpu_blocks=40, max_model_len=512,
                          max_num_batched_tokens=256, max_prefill_chunk_size=128)
    prompts = random_prompts(cfg["vocab_size"], (3, 70, 129, 300), seed=13)
    requests = make_requests(prompts, temperature=0.0, max_tokens=24)
    engine.generate(requests)
    for request in requests:
        within_bfloat16_noise_of_plain_argmax(tensors, cfg, request)
    assert engine.runner.kernels_replayed > 0


def test_status_word_reaches_generation(folders):
    """A kernel that refuses an access only sets a bit; generation reads the word with the
    sampled tokens and stops instead of going on with tokens that mean nothing."""
    folder, cfg, _ = folders["tiny_a"]
    engine = build_engine(folder, "float32")
    request = make_requests([[3, 4, 5]], temperature=0.0, max_tokens=4)[0]
    engine.add_request(request)
    engine.step()
    assert len(request.output_token_ids) == 1
    engine.runner.status[0] = 4  # as a kernel would have left it
    with pytest.raises(RuntimeError, match="a cache slot outside the pool"):
        engine.step()
    assert int(engine.runner.status[0].item()) == 0
    engine.step()
    assert len(request.output_token_ids) == 2


def test_batched_equals_one_at_a_time(folders):
    folder, cfg, _ = folders["tiny_a"]
    prompts = random_prompts(cfg["vocab_size"], (3, 20, 9, 31, 14), seed=3)
    engine = build_engine(folder, "float32")
    together = make_requests(prompts, temperature=0.0, max_tokens=20)
    engine.generate(together)
    for index, prompt in enumerate(prompts):
        alone = make_requests([prompt], temperature=0.0, max_tokens=20)
        engine.generate(alone)
        assert alone[0].output_token_ids == together[index].output_token_ids


def test_preemption_recomputes_and_gives_same_tokens(folders):
    folder, cfg, tensors = folders["tiny_a"]
    prompts = random_prompts(cfg["vocab_size"], (30, 28, 26, 33), seed=4)
    roomy = build_engine(folder, "float32", num_gpu_blocks=200)
    want = make_requests(prompts, temperature=0.0, max_tokens=40)
    roomy.generate(want)
    assert roomy.scheduler.num_preemptions == 0
    # 4-token pages: every request ends with 70 tokens = 18 pages; 40 usable pages cannot hold four.
    tight = build_engine(folder, "float32", num_gpu_blocks=41)
    got = make_requests(prompts, temperature=0.0, max_tokens=40)
    tight.generate(got)
    assert tight.scheduler.num_preemptions > 0
    for a, b in zip(got, want):
        assert len(a.output_token_ids) == 40
        assert a.output_token_ids == b.output_token_ids
    tight.scheduler.schedule()
    tight.cache.assert_consistent()
    assert tight.cache.num_free_pages() == tight.cache.num_total_pages


def test_seeded_temperature_is_reproducible_and_independent_of_the_batch(folders):
    folder, cfg, _ = folders["tiny_b"]
    prompts = random_prompts(cfg["vocab_size"], (1, 9, 33, 70), seed=5)
    from velox_b200.engine.request import Request
    from velox_b200.sampling.params import SamplingParams

    def run(engine, subset):
        requests = [
            Request(f"s{i}", prompts[i], SamplingParams(temperature=0.8, seed=7 + i, max_tokens=12, ignore_eos=True))
            for i in subset
        ]
        engine.generate(requests)
        return {i: r.output_token_ids for i, r in zip(subset, requests)}

    engine = build_engine(folder, "float32", block_size=8, max_model_len=192)
    all_together = run(engine, [0, 1, 2, 3])
    assert run(engine, [0, 1, 2, 3]) == all_together
    for i in range(4):
        assert run(engine, [i])[i] == all_together[i]
    assert len({tuple(v) for v in all_together.values()}) == 4
    # temperature changes what is drawn
    greedy = make_requests([prompts[2]], temperature=0.0, max_tokens=12)
    engine.generate(greedy)
    assert greedy[0].output_token_ids != all_together[2]


def test_greedy_row_is_not_disturbed_by_sampled_neighbours(folders):
    folder, cfg, _ = folders["tiny_a"]
    prompts = random_prompts(cfg["vocab_size"], (12, 12, 12), seed=6)
    from velox_b200.engine.request import Request
    from velox_b200.sampling.params import SamplingParams

    engine = build_engine(folder, "float32")
    alone = make_requests([prompts[0]], temperature=0.0, max_tokens=10)
    engine.generate(alone)
    mixed = [
        Request("g", prompts[0], SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)),
        Request("h1", prompts[1], SamplingParams(temperature=1.5, max_tokens=10, ignore_eos=True, top_k=20)),
        Request("h2", prompts[2], SamplingParams(temperature=1.5, max_tokens=10, ignore_eos=True, top_p=0.7,
                                                 repetition_penalty=1.2, presence_penalty=0.1, frequency_penalty=0.1)),
    ]
    engine.generate(mixed)
    assert mixed[0].output_token_ids == alone[0].output_token_ids
    assert all(len(r.output_token_ids) == 10 for r in mixed)


def test_stop_tokens_max_tokens_and_limits(folders):
    folder, cfg, tensors = folders["tiny_a"]
    from velox_b200.engine.request import Request
    from velox_b200.sampling.params import SamplingParams

    engine = build_engine(folder, "float32")
    prompt = random_prompts(cfg["vocab_size"], (10,), seed=8)[0]
    free_run = make_requests([prompt], temperature=0.0, max_tokens=6)
    engine.generate(free_run)
    tokens = free_run[0].output_token_ids
    stopper = Request("stop", prompt, SamplingParams(temperature=0.0, max_tokens=6, stop_token_ids=[tokens[2]]))
    engine.generate([stopper])
    first = tokens.index(tokens[2])
    assert stopper.output_token_ids == tokens[: first + 1]
    assert stopper.finish_reason.value == "stop"
    with pytest.raises(ValueError):
        engine.add_request(Request("long", [1] * 128, SamplingParams(max_tokens=1)))
    with pytest.raises(ValueError):
        engine.add_request(Request("long2", [1] * 100, SamplingParams(max_tokens=40)))


@pytest.mark.parametrize("dtype,case", [("float32", "tiny_a"), ("float32", "tiny_w"), ("bfloat16", "tiny_d")])
def test_pipelined_generation_equals_step_by_step(folders, dtype, case, monkeypatch):
    """``generate`` queues a step before it has read the tokens of the one before and feeds
    them on the device; the tokens, the reasons for ending and what the listeners hear are
    those of one step at a time: greedy and seeded requests, a stop token in the middle of
    decoding, penalties, prompts cut into portions, and a pool so small that requests are
    preempted while a token is on its way.  Two runs are compared token by token, so the
    bfloat16 case runs with every sum in a fixed order (what VELOX_B200_DETERMINISTIC=1 sets):
    sums that meet at the L2 in any order can move a draw that sits on the last bit."""
    from velox_b200.engine.request import Request
    from velox_b200.ops import linear
    from velox_b200.parts import mlp
    from velox_b200.sampling.params import SamplingParams

    monkeypatch.setattr(linear, "_CHUNKED_SPLITK", False)
    monkeypatch.setattr(mlp, "_FUSE_MLP", False)

    folder, cfg, _ = folders[case]
    prompts = random_prompts(cfg["vocab_size"], (30, 3, 41, 17, 26, 9), seed=12)

    def run(pipeline, stop_on=None):
        engine = build_engine(folder, dtype, num_gpu_blocks=45, pipeline_decode=pipeline)
        heard = []
        requests = [
            Request("greedy", prompts[0], SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True)),
            Request("stops", prompts[1], SamplingParams(temperature=0.0, max_tokens=30,
                                                        stop_token_ids=[] if stop_on is None else [stop_on])),
            Request("seeded", prompts[2], SamplingParams(temperature=0.9, seed=5, max_tokens=25, ignore_eos=True)),
            Request("filtered", prompts[3], SamplingParams(temperature=1.1, seed=6, top_k=12, top_p=0.8, max_tokens=33,
                                                           ignore_eos=True)),
            Request("penalised", prompts[4], SamplingParams(temperature=0.7, seed=7, repetition_penalty=1.3,
                                                            frequency_penalty=0.2, max_tokens=20, ignore_eos=True)),
            Request("short", prompts[5], SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)),
        ]
        for request in requests:
            request.add_listener(lambda r, kind, token: heard.append((r.request_id, kind, token)))
        engine.generate(requests)
        assert not engine.has_work()
        engine.scheduler.schedule()
        engine.cache.assert_consistent()
        assert engine.cache.num_free_pages() == engine.cache.num_total_pages
        assert all(t >= 0 for r in requests for t in r.all_token_ids)
        per_request = {r.request_id: [h[1:] for h in heard if h[0] == r.request_id] for r in requests}
        return requests, per_request, engine.scheduler.num_preemptions

    free, _, _ = run(False)
    stop_on = free[1].output_token_ids[11]
    want, want_heard, want_preemptions = run(False, stop_on)
    got, got_heard, got_preemptions = run(True, stop_on)
    assert want_preemptions > 0 and got_preemptions > 0
    for a, b in zip(got, want):
        assert a.output_token_ids == b.output_token_ids, a.request_id
        assert a.finish_reason is b.finish_reason
        assert got_heard[a.request_id] == want_heard[b.request_id]
        assert got_heard[a.request_id][-1] == ("finish", None)
        assert [t for kind, t in got_heard[a.request_id] if kind == "token"] == a.output_token_ids
    first = free[1].output_token_ids.index(stop_on)
    assert got[1].finish_reason.value == "stop" and got[1].output_token_ids == free[1].output_token_ids[: first + 1]
    assert got[5].finish_reason.value == "length" and len(got[5].output_token_ids) == 1


def test_llm_entry_point(folders):
    folder, cfg, tensors = folders["tiny_a"]
    from velox_b200.engine.engine import LLM
    from velox_b200.sampling.params import SamplingParams

    llm = LLM(folder, dtype="float32", max_model_len=128, max_num_seqs=4, max_num_batched_tokens=64,
              max_prefill_chunk_size=16, block_size=4, num_gpu_blocks=100)
    prompts = random_prompts(cfg["vocab_size"], (6, 13), seed=9)
    outputs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    for prompt, output in zip(prompts, outputs):
        assert output == plain_model.greedy_generate(tensors, cfg, prompt, 5, dtype=torch.float64)


@pytest.mark.parametrize("pipeline", [False, True], ids=["step_by_step", "pipelined"])
def test_bfloat16_soak_many_requests_tight_pool(folders, pipeline):
    """Two dozen requests of random lengths through a pool that cannot hold four of them:
    portions beside decoded tokens, preemptions and recomputes, captured decode steps and
    captured steps of other shapes, slots and pages used again and again.  Every token must be
    the plain argmax given its prefix (or within bfloat16 noise of it), everything must finish,
    and everything must come back.  Step by step, steps with prompt portions take the
    captured-graph route; pipelined, they are queued launch by launch behind the running step."""
    folder, cfg, tensors = folders["tiny_d"]
    rng = np.random.default_rng(17)
    lengths = [int(n) for n in rng.integers(1, 260, 24)]
    budgets = [int(n) for n in rng.integers(8, 60, 24)]
    prompts = random_prompts(cfg["vocab_size"], lengths, seed=23)
    engine = build_engine(folder, "bfloat16", block_size=64, num_gpu_blocks=8, max_model_len=320, max_num_seqs=4,
                          max_num_batched_tokens=128, max_prefill_chunk_size=64, pipeline_decode=pipeline)
    from velox_b200.engine.request import Request
    from velox_b200.sampling.params import SamplingParams

    requests = [Request(f"q{i}", p, SamplingParams(temperature=0.0, max_tokens=b, ignore_eos=True))
                for i, (p, b) in enumerate(zip(prompts, budgets))]
    before = dict(engine.runner.mixed_step_counts)  # the warm-up's own steps
    engine.generate(requests, max_steps=5000)
    assert all(r.finished and len(r.output_token_ids) == b for r, b in zip(requests, budgets))
    for request in requests:
        within_bfloat16_noise_of_plain_argmax(tensors, cfg, request)
    counts = engine.runner.mixed_step_counts
    assert engine.scheduler.num_preemptions > 0
    assert engine.runner.kernels_replayed > 0
    assert (counts["eager"] + counts["replayed"] > before["eager"] + before["replayed"]) == (not pipeline)
    engine.scheduler.schedule()
    engine.cache.assert_consistent()
    assert engine.cache.num_free_pages() == engine.cache.num_total_pages
    assert engine.cache.num_free_slots == engine.config.max_num_seqs
    engine.runner.check_status()


def test_command_lines_run_on_tiny_sizes(tmp_path, capsys):
    """The benchmark and the roofline command lines, start to end, on the tiny named sizes:
    pipelined and one step at a time, greedy and with candidate filters, and the JSON they write."""
    import json

    from velox_b200.cli import benchmark, roofline

    out = tmp_path / "bench.json"
    common = ["--model-size", "tiny-b", "--num-requests", "6", "--max-tokens", "12", "--max-model-len", "128",
              "--max-num-seqs", "4", "--max-num-batched-tokens", "64", "--max-prefill-chunk-size", "16",
              "--block-size", "8", "--workload", "short", "--seed", "3"]
    assert benchmark.main(common + ["--temperature", "0", "--output-json", str(out)]) == 0
    first = capsys.readouterr().out
    assert "decode throughput" in first and "GPU-busy fraction" in first
    record = json.loads(out.read_text())
    assert record
    assert benchmark.main(common + ["--temperature", "0.8", "--top-p", "0.9", "--top-k", "20", "--no-pipeline"]) == 0
    assert "decode throughput" in capsys.readouterr().out
    table = tmp_path / "roofline.json"
    assert roofline.main(["--model-size", "tiny-b", "--batch", "1,3", "--context", "20,60", "--layers", "1,3",
                          "--steps", "4", "--warmup", "1", "--block-size", "8", "--output-json", str(table)]) == 0
    rows = json.loads(table.read_text())
    assert [(r["batch"], r["context"]) for r in rows] == [(1, 20), (1, 60), (3, 20), (3, 60)]
    assert all(r["us_by_bytes"] > 0 and r["size"] == "tiny-b" for r in rows)
    assert roofline.main(["--model-size", "tiny-b", "--prefill", "24,70", "--context", "0,50", "--layers", "1,3",
                          "--warmup", "1", "--block-size", "8", "--output-json", str(table)]) == 0
    rows = json.loads(table.read_text())
    assert [(r["tokens"], r["context"]) for r in rows] == [(24, 0), (24, 50), (70, 0), (70, 50)]
    assert all(r["tflops"] >= 0 for r in rows)


def test_timeline_command_line_runs_on_a_tiny_size():
    """The timeline build (kernels compiled with their CTA trace) through its command line, in a
    process of its own because the build flag is read when the libraries are loaded: a decode
    step and a prompt portion, every launch listed with its CTAs."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for mode in (["--batch", "3", "--context", "40"], ["--prefill", "70", "--context", "30"]):
        done = subprocess.run([sys.executable, "-m", "velox_b200.cli.timeline", "--model-size", "tiny-b", "--layers", "2",
                               "--block-size", "8"] + mode, cwd=root, capture_output=True, text=True, timeout=600)
        assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
        assert "launches" in done.stdout and "by kernel and grid" in done.stdout
        assert "attn" in done.stdout and "gemm" in done.stdout
