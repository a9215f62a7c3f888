"""Benchmark: decode tokens/s (batch 8 by default; batch 1 and 64 as extra points) and prefill
tokens/s at 2,048 tokens, at Qwen2.5-1.5B layer sizes with random weights, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second of the step function (device time
of K decode steps queued back to back, CUDA events; each step is fed the tokens the step
before it sampled, on the device); ``e2e`` is the same through the Python entry point (the
loop of ``Engine.generate``: every step's arrays go up through pinned memory and its sampled
tokens are read back, one step behind).  ``prefill`` is one 2,048-token prompt in one step; ``roofline`` is the decode step's
bytes (every weight once, the live requests' cache) over its time against the measured copy
bandwidth.  With --gpus N > 1 it says that the engine is single-GPU and exits with 2.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Qwen2.5-1.5B layer sizes (the benchmark's third configuration).
MODEL_1P5B = {
    "architectures": ["Qwen2ForCausalLM"],
    "model_type": "qwen2",
    "num_hidden_layers": 28,
    "hidden_size": 1536,
    "num_attention_heads": 12,
    "num_key_value_heads": 2,
    "intermediate_size": 8960,
    "vocab_size": 151936,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True,
    "use_sliding_window": False,
    "max_position_embeddings": 32768,
    "hidden_act": "silu",
}
FULL_LAYERS = 28
CONTEXT = 4096
PREFILL_TOKENS = 2048
# Untimed decode steps in front of every timed decode region, beyond --warmup, in both arms: the
# first few dozen steps after a pause of the device run some 5 % slower than the ones that follow
# (measured: 1.45, 1.38, then 1.355 ms a step over three windows of 20 steps in a row).
SETTLE_STEPS = 40
# Keys per cache page: the benchmark configuration's (and the reference's default).  The engine's own
# default is 64; a point with 64-key pages is reported beside the main numbers.
BLOCK_SIZE = 16
ENGINE_DEFAULT_BLOCK_SIZE = 64

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as handle:
            peaks = json.load(handle)
        peaks["source"] = "measured"
        return peaks
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self._proc = None
        self._thread = None

    def start(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            return
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()

    def _read(self):
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        sm, reasons, sm_max = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for parts in self.samples:
            try:
                sm.append(float(parts[0]))
                sm_max = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {
            "sm_mhz": sm[len(sm) // 2] if sm else None,
            "sm_max_mhz": sm_max,
            "reasons": sorted(reasons),
            "samples": len(sm),
        }


def model_bytes(cfg, layers):
    E, H, G, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                     cfg["intermediate_size"], cfg["vocab_size"])
    D = E // H
    per_layer = ((H + 2 * G) * D * E + E * H * D + 3 * I * E) * 2 + ((H + 2 * G) * D + 2 * E) * 4
    head = V * E * 2
    return layers * per_layer + head + E * 4, 2 * G * D * 2 * layers  # weight bytes, KV bytes per token


def model_flops_per_token(cfg, layers, context):
    """Multiply-add flops of one token at a given number of visible keys."""
    E, H, G, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                     cfg["intermediate_size"], cfg["vocab_size"])
    D = E // H
    gemm = 2 * ((H + 2 * G) * D * E + E * H * D + 3 * I * E)
    attn = 4 * H * D * context
    return layers * (gemm + attn)


def run_own(args):
    import numpy as np
    import torch

    from velox_b200.config import EngineConfig
    from velox_b200.engine.engine import Engine
    from velox_b200.engine.request import Request
    from velox_b200.engine.runner import StepChunk
    from velox_b200.ops import kernels
    from velox_b200.sampling.params import SamplingParams
    from velox_b200.weights import write_random_model

    peaks = load_peaks()
    layers = args.layers
    cfg = dict(MODEL_1P5B, num_hidden_layers=layers)
    folder = tempfile.mkdtemp(prefix="velox_bench_")
    t0 = time.time()
    write_random_model(folder, cfg, seed=0, dtype="bfloat16")
    print(f"[bench] wrote random {layers}-layer model in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)

    max_batch = max(args.batch, 64 if args.points else args.batch)
    block_size = args.block_size
    pages_per_seq = CONTEXT // block_size + 1
    engine = Engine.from_pretrained(EngineConfig(
        model=folder, dtype="bfloat16", max_model_len=CONTEXT + 16, max_num_seqs=max_batch,
        max_num_batched_tokens=max(PREFILL_TOKENS, max_batch), max_prefill_chunk_size=PREFILL_TOKENS,
        block_size=block_size, num_gpu_blocks=max_batch * pages_per_seq + 8, seed=0,
    ))
    import shutil

    runner, cache, sampler = engine.runner, engine.cache, engine.sampler
    vocab = cfg["vocab_size"]
    rng = np.random.default_rng(0)
    weight_bytes, kv_bytes_per_token = model_bytes(cfg, layers)

    def fill(batch, context, runner=runner, cache=cache):
        """``batch`` sequences with ``context`` tokens in the cache, through the step function."""
        seqs = []
        for b in range(batch):
            seq = cache.new_sequence(f"bench{b}")
            assert cache.acquire_slot(seq)
            seqs.append(seq)
            done = 0
            while done < context:
                n = min(PREFILL_TOKENS, context - done)
                assert cache.append_slots(seq, n)
                runner.step([StepChunk(seq, rng.integers(0, vocab, n).tolist(), ())])
                cache.advance(seq, n)
                done += n
        torch.cuda.synchronize()
        return seqs

    def release(seqs, cache=cache):
        for seq in seqs:
            cache.free(seq)
            cache.release_slot(seq)

    def decode_steps(seqs, steps, warmup, runner=runner, cache=cache, sampler=sampler):
        """Device time (ms) of ``steps`` decode steps after ``warmup`` untimed ones, and the
        launches they made.  The timed steps are queued back to back, as ``Engine.generate``
        queues them: each step's token ids are stand-ins that the embedding resolves from the
        tokens the step before it sampled on the device, so the host prepares a step while the
        device runs the one before; one pair of events brackets all of them."""
        batch = len(seqs)
        tokens = rng.integers(0, vocab, batch).tolist()
        params = [SamplingParams(temperature=0.0, max_tokens=1)] * batch
        names = [s.seq_id for s in seqs]
        runner.fed_tokens = sampler.tokens

        def one_step(ids):
            chunks = []
            for seq, token in zip(seqs, ids):
                assert cache.append_slots(seq, 1)
                chunks.append(StepChunk(seq, [token], (0,)))
            logits = runner.step(chunks)
            out = sampler.sample(logits, params, names, [0] * batch)
            for seq in seqs:
                cache.advance(seq, 1)
            return out

        for _ in range(warmup):
            tokens = one_step(tokens).tolist()
        fed = [-1 - row for row in range(batch)]
        for _ in range(SETTLE_STEPS):
            one_step(fed)
        launches_before = kernels.launch_count + runner.kernels_replayed
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            out = one_step(fed)
        end.record()
        torch.cuda.synchronize()
        assert all(0 <= t < vocab for t in out.tolist())
        runner.check_status()
        return [start.elapsed_time(end) / steps] * steps, kernels.launch_count + runner.kernels_replayed - launches_before

    def decode_point(batch, steps, warmup, engine=engine):
        context = CONTEXT - steps - warmup - SETTLE_STEPS - 1
        seqs = fill(batch, context, engine.runner, engine.cache)
        times, launches = decode_steps(seqs, steps, warmup, engine.runner, engine.cache, engine.sampler)
        release(seqs, engine.cache)
        ms = sum(times) / len(times)
        return batch * 1000.0 / ms, ms, launches, context + warmup + SETTLE_STEPS + steps // 2

    E, H, G, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                     cfg["intermediate_size"], cfg["vocab_size"])
    D = E // H
    # Bytes every launch of a kind has to read: its matrix once (the cache for attention).
    kind_bytes = {"qkv": (H + 2 * G) * D * E * 2, "o": E * H * D * 2, "feed_forward": 3 * I * E * 2, "lm_head": V * E * 2}
    kind_of = {"gemm_bf16_qkv_rope": "qkv", "rope_cache_write": "qkv", "attention": "attention", "attention_merge": "attention",
               "gemm_bf16_add_mirrored": "o", "mlp_fused": "feed_forward", "swiglu": "feed_forward"}

    def kernel_breakdown(batch, repeats=5):
        """Device time of each kind of kernel in one decode step of ``batch`` requests at the
        benchmark's context: the step is laid out as the captured step is, but launched kernel
        by kernel behind a queued delay with an event after every launch."""
        context = CONTEXT - 8
        seqs = fill(batch, context)
        chunks = []
        for seq in seqs:
            assert cache.append_slots(seq, 1)
            chunks.append(StepChunk(seq, [int(rng.integers(0, vocab))], (0,)))
        bucket = runner._bucket(batch)
        totals = []
        for _ in range(repeats):
            ctx, ids, rows, count = runner.prepare(chunks, pad_to=bucket)
            torch.cuda.synchronize()
            torch.cuda._sleep(40_000_000)  # about 20 ms: the host queues the whole step meanwhile
            first = torch.cuda.Event(enable_timing=True)
            first.record()
            kernels.launch_events = []
            try:
                runner.model.forward(ctx, runner.layer_caches, ids, rows, count)
            finally:
                events, kernels.launch_events = kernels.launch_events, None
            torch.cuda.synchronize()
            per_kind, previous, last_gemm = {}, first, None
            for index, (name, event) in enumerate(events):
                took = previous.elapsed_time(event) * 1000.0
                previous = event
                kind = kind_of.get(name)
                if name.startswith("gemm_bf16") and kind is None:
                    last_gemm = index
                    kind = "o" if name == "gemm_bf16" else "feed_forward"  # settled below for the last one
                per_kind.setdefault(kind or "other", []).append((index, took))
            flat = {}
            for kind, entries in per_kind.items():
                for index, took in entries:
                    real = "lm_head" if index == last_gemm else kind
                    flat[real] = flat.get(real, 0.0) + took
            totals.append(flat)
        release(seqs)
        out = {}
        for kind in sorted({k for t in totals for k in t}):
            values = sorted(t.get(kind, 0.0) for t in totals)
            out[kind] = values[len(values) // 2]
        return out, context + 1

    def kernel_report(times_us, batch, keys):
        report = {}
        for kind, us in times_us.items():
            per_step = kind_bytes.get(kind)
            if kind == "attention":
                per_step = batch * keys * kv_bytes_per_token
            elif per_step is not None and kind != "lm_head":
                per_step *= layers
            entry = {"us": round(us, 1)}
            if per_step:
                gbs = per_step / (us * 1e-6) / 1e9
                entry.update({"gbs": round(gbs, 1), "frac": round(gbs / peaks["hbm_gbs"], 3)})
            report[kind] = entry
        return report

    clocks = ClockSampler()
    clocks.start()
    value, ms_per_step, launches, mean_context = decode_point(args.batch, args.steps, args.warmup)
    clock_summary = clocks.stop()

    step_bytes = weight_bytes + args.batch * mean_context * kv_bytes_per_token
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peaks["source"]}

    # Prefill: one 2,048-token prompt in one step.
    prefill_times = []
    for i in range(3 + 3):
        seq = cache.new_sequence(f"prefill{i}")
        assert cache.acquire_slot(seq) and cache.append_slots(seq, PREFILL_TOKENS)
        ids = rng.integers(0, vocab, PREFILL_TOKENS).tolist()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepChunk(seq, ids, (PREFILL_TOKENS - 1,))])
        end.record()
        torch.cuda.synchronize()
        cache.advance(seq, PREFILL_TOKENS)
        release([seq])
        if i >= 3:
            prefill_times.append(start.elapsed_time(end))
    prefill_ms = sum(prefill_times) / len(prefill_times)
    prefill_flops = sum(model_flops_per_token(cfg, layers, t + 1) for t in range(PREFILL_TOKENS))
    prefill_flops += 2 * cfg["vocab_size"] * cfg["hidden_size"]  # one row of logits
    prefill = {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}

    # The same prompt as four portions of 512, one step each.
    split_times = []
    for i in range(2 + 3):
        seq = cache.new_sequence(f"prefill4_{i}")
        assert cache.acquire_slot(seq)
        ids = rng.integers(0, vocab, PREFILL_TOKENS).tolist()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for part in range(4):
            assert cache.append_slots(seq, 512)
            runner.step([StepChunk(seq, ids[512 * part : 512 * (part + 1)], (511,) if part == 3 else ())])
            cache.advance(seq, 512)
        end.record()
        torch.cuda.synchronize()
        release([seq])
        if i >= 2:
            split_times.append(start.elapsed_time(end))
    split_ms = sum(split_times) / len(split_times)
    prefill_4x512 = {"value": round(PREFILL_TOKENS * 1000.0 / split_ms, 1), "ms": round(split_ms, 3),
                     "frac": round(prefill_flops / (split_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}

    points = {}
    kernel_times = {}
    if args.points:
        for batch in (1, 64):
            tok_s, _, _, _ = decode_point(batch, max(8, args.steps // 2), 3)
            points[f"decode_b{batch}"] = round(tok_s, 1)
        times8, keys8 = kernel_breakdown(args.batch)
        kernel_times = kernel_report(times8, args.batch, keys8)
        times64, keys64 = kernel_breakdown(64)
        kernel_times["attention_b64"] = kernel_report({"attention": times64["attention"]}, 64, keys64)["attention"]
        kernel_times["method"] = ("one decode step launched kernel by kernel behind a queued delay, a CUDA event after every "
                                  "launch; us summed over the layers, bytes = the matrices (the cache) each kind must read")
        # The other page size (the engine's default of 64 keys, or 16 if the run itself uses
        # 64): a second engine on the same weights.
        other = ENGINE_DEFAULT_BLOCK_SIZE if block_size != ENGINE_DEFAULT_BLOCK_SIZE else 16
        other_pages = Engine.from_pretrained(EngineConfig(
            model=folder, dtype="bfloat16", max_model_len=CONTEXT + 16, max_num_seqs=args.batch,
            max_num_batched_tokens=max(PREFILL_TOKENS, args.batch), max_prefill_chunk_size=PREFILL_TOKENS,
            block_size=other, num_gpu_blocks=args.batch * (CONTEXT // other + 2) + 8, seed=0,
        ))
        tok_s, _, _, _ = decode_point(args.batch, args.steps, args.warmup, engine=other_pages)
        points[f"decode_b{args.batch}_block{other}"] = round(tok_s, 1)
        del other_pages
    shutil.rmtree(folder, ignore_errors=True)

    # End to end through the entry point, host tokens in and out.  Prompts are
    # prefilled in turn, so the first request decodes while the others still prefill (two
    # portions each); max_tokens leaves every request alive until the timed steps are over.
    head_start = 2 * args.batch
    budget = args.steps + args.warmup + SETTLE_STEPS + head_start + 8
    prompts = [rng.integers(0, vocab, CONTEXT - budget).tolist() for _ in range(args.batch)]
    requests = [Request(f"e2e{i}", p, SamplingParams(temperature=0.0, max_tokens=budget, ignore_eos=True))
                for i, p in enumerate(prompts)]
    for request in requests:
        engine.add_request(request)
    while any(not r.is_decoding or r.num_output_tokens < 1 for r in requests):
        engine.step()
    for _ in range(args.warmup + SETTLE_STEPS):
        engine.step_pipelined()
    engine.drain()
    torch.cuda.synchronize()
    produced_before = sum(r.num_output_tokens for r in requests)
    meta_bytes = 0
    t_start = time.perf_counter()
    # The loop of Engine.generate: every call queues a step (its arrays go up in one copy from
    # pinned memory) and reads the tokens of the step before from pinned memory; drain() reads
    # the last step's.
    for _ in range(args.steps):
        engine.step_pipelined()
        meta_bytes = max(meta_bytes, runner.last_meta_bytes)
    engine.drain()
    torch.cuda.synchronize()
    e2e_seconds = time.perf_counter() - t_start
    produced = sum(r.num_output_tokens for r in requests) - produced_before
    if produced != args.steps * args.batch:
        raise RuntimeError(f"e2e: {produced} tokens in {args.steps} steps of {args.batch} requests")
    for request in requests:
        engine.abort_request(request.request_id)
    e2e = {"value": round(produced / e2e_seconds, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": meta_bytes, "d2h_bytes_per_step": 4 * args.batch}

    line = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Qwen2.5-1.5B)",
        "value": round(value, 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True,
        "scaling": "weak",
        # The reference's only published batch-8 figure: 226 tok/s on an RTX 4050 Mobile.
        "vs_baseline": round(value / 226.0, 2),
        "dtype": "bf16",
        "data": "synthetic: seeded random weights, uniform-random token ids",
        "config": {
            "model": "Qwen2.5-1.5B layer sizes", "layers": layers, "layers_full_model": FULL_LAYERS,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "global_batch": args.batch, "seq_len": CONTEXT, "prefill_tokens": PREFILL_TOKENS,
            "kv_block_size": block_size, "kv_block_size_engine_default": ENGINE_DEFAULT_BLOCK_SIZE, "tied_embeddings": True, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (weights streamed every step)",
            "decode_steps": "queued back to back; each is fed the tokens the step before sampled, on the device; 40 more untimed steps before the timed ones", "gemm": "decode: own tcgen05 kernels; prefill: cuBLAS (library)",
        },
        "clocks": clock_summary,
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill,
        "prefill_4x512": prefill_4x512,
        "roofline": roofline,
        "points": points,
        "kernels": kernel_times,
    }
    print(json.dumps(line))
    return 0


def run_reference(args):
    """The unmodified reference engine from ``baseline/_ref`` (a plain copy of its source tree:
    it has no packaging, and imports as ``engine`` / ``src`` from its root) on the same random
    model folder, batch and context, through its own ``Engine.from_pretrained`` and ``step``
    (engine/engine.py:106-172,276-369 of that project) with its defaults: 16-key pages, CUDA
    graphs, prefix caching.  Nothing of this package runs on that path except the writer of the
    random-weights folder."""
    ref_root = os.environ.get("VELOX_REFERENCE_TREE") or os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isfile(os.path.join(ref_root, "engine", "engine.py")):
        print(json.dumps({"impl": "reference",
                          "unavailable": f"no copy of the reference's source tree at {os.path.relpath(ref_root, ROOT)}"}))
        return 0
    log_dir = os.environ.get("VELOX_BENCH_LOG_DIR") or tempfile.gettempdir()
    try:
        line = _reference_numbers(args, ref_root)
    except Exception as exc:  # the reference's own code failed here: say why, keep the traceback
        import traceback

        text = traceback.format_exc()
        try:
            os.makedirs(log_dir, exist_ok=True)
            with open(os.path.join(log_dir, "reference_arm_failure.log"), "w") as handle:
                handle.write(text)
        except OSError:
            pass
        print(text, file=sys.stderr)
        reason = f"{type(exc).__name__}: {exc}".replace("\n", " ")[:300]
        print(json.dumps({"impl": "reference", "unavailable": "the reference's engine failed on this box: " + reason}))
        return 0
    print(json.dumps(line))
    return 0


def _reference_numbers(args, ref_root):
    import numpy as np
    import torch

    from velox_b200.weights import write_random_model

    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    cfg = dict(MODEL_1P5B, num_hidden_layers=args.layers)
    folder = tempfile.mkdtemp(prefix="velox_bench_ref_")
    write_random_model(folder, cfg, seed=0, dtype="bfloat16")

    sys.path.insert(0, ref_root)
    from engine.config import EngineConfig as RefEngineConfig  # the reference's
    from engine.engine import Engine as RefEngine
    from engine.request import Request as RefRequest
    from engine.utils import SamplingParams as RefSamplingParams

    ref_block = RefEngineConfig().block_size
    rng = np.random.default_rng(0)
    vocab = cfg["vocab_size"]

    def build(max_batch, total_requests):
        # Its prefix cache (on by default) keeps the pages of requests that have ended and counts
        # only the leaves of its tree as free again, so the pool holds every request of the run.
        return RefEngine.from_pretrained(RefEngineConfig(
            model=folder, dtype="bfloat16", device="cuda", max_model_len=CONTEXT + 16, max_num_seqs=max_batch,
            max_num_batched_tokens=max(PREFILL_TOKENS, max_batch), max_prefill_chunk_size=PREFILL_TOKENS,
            num_gpu_blocks=total_requests * (CONTEXT // ref_block + 2) + 64, seed=0,
        ))

    def decode_point(engine, batch, steps, warmup):
        """``batch`` requests brought to the benchmark's context through the engine's own loop,
        then ``steps`` decode steps timed on the device (events around ``step``) and ``steps``
        more by the wall clock."""
        head_start = 2 * batch
        budget = 2 * steps + warmup + SETTLE_STEPS + head_start + 8
        requests = [RefRequest(request_id=f"ref{batch}_{i}", prompt_token_ids=rng.integers(0, vocab, CONTEXT - budget).tolist(),
                               sampling_params=RefSamplingParams(temperature=0.0, max_tokens=budget, ignore_eos=True))
                    for i in range(batch)]
        for request in requests:
            engine.add_request(request)
        guard = 0
        while any(r.num_output_tokens < 1 or r.num_computed_tokens < r.num_tokens - 1 for r in requests):
            engine.step()
            guard += 1
            if guard > 100 * batch:
                raise RuntimeError("the reference's engine did not reach pure decoding")
        for _ in range(warmup + SETTLE_STEPS):
            engine.step()
        times = []
        for _ in range(steps):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            before = sum(r.num_output_tokens for r in requests)
            start.record()
            engine.step()
            end.record()
            torch.cuda.synchronize()
            if sum(r.num_output_tokens for r in requests) - before != batch:
                raise RuntimeError("a timed step of the reference was not a pure decode step of the whole batch")
            times.append(start.elapsed_time(end))
        torch.cuda.synchronize()
        before = sum(r.num_output_tokens for r in requests)
        t_start = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t_start
        produced = sum(r.num_output_tokens for r in requests) - before
        for request in requests:
            engine.abort_request(request.request_id)
        engine.step()  # lets the scheduler reap them
        ms = sum(times) / len(times)
        return batch * 1000.0 / ms, ms, produced / seconds

    max_batch = max(args.batch, 64 if args.points else args.batch)
    engine = build(max_batch, args.batch + 6 + (1 + 64 if args.points else 0))
    import shutil

    shutil.rmtree(folder, ignore_errors=True)
    clocks = ClockSampler()
    clocks.start()
    value, ms_per_step, e2e_value = decode_point(engine, args.batch, args.steps, args.warmup)
    clock_summary = clocks.stop()

    # Prefill: a 2,048-token prompt in one step, to its first token.
    prefill_times = []
    for i in range(3 + 3):
        request = RefRequest(request_id=f"refprefill{i}", prompt_token_ids=rng.integers(0, vocab, PREFILL_TOKENS).tolist(),
                             sampling_params=RefSamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
        engine.add_request(request)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step()
        end.record()
        torch.cuda.synchronize()
        if request.num_output_tokens != 1:
            raise RuntimeError("the reference did not prefill the prompt in one step")
        engine.step()
        if i >= 3:
            prefill_times.append(start.elapsed_time(end))
    prefill_ms = sum(prefill_times) / len(prefill_times)

    points = {}
    if args.points:
        for batch in (1, 64):
            tok_s, _, _ = decode_point(engine, batch, max(8, args.steps // 2), 3)
            points[f"decode_b{batch}"] = round(tok_s, 1)

    return {
        "impl": "reference",
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Qwen2.5-1.5B)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / 226.0, 2), "dtype": "bf16",
        "data": "synthetic: seeded random weights, uniform-random token ids",
        "config": {
            "model": "Qwen2.5-1.5B layer sizes", "layers": args.layers, "layers_full_model": FULL_LAYERS,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "global_batch": args.batch, "seq_len": CONTEXT, "prefill_tokens": PREFILL_TOKENS,
            "kv_block_size": ref_block, "tied_embeddings": True, "parallelism": "single GPU",
            "timing": "CUDA events around each Engine.step of the reference (its host work included); 40 more untimed steps before the timed ones",
        },
        "clocks": clock_summary,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s"},
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3)},
        "points": points,
    }


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers of the same sizes (reported)")
    parser.add_argument("--block-size", type=int, default=BLOCK_SIZE, help="keys per cache page of the main engine (reported)")
    parser.add_argument("--impl", default="own", choices=["own", "reference"])
    parser.add_argument("--no-points", dest="points", action="store_false", help="skip the batch 1 / 64 points")
    args = parser.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 or world > 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py: this engine runs on one GPU; --gpus {max(args.gpus, world)} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    return run_own(args)


if __name__ == "__main__":
    sys.exit(main())
