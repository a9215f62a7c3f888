"""End-to-end benchmark command line, in the manner of the reference's ``benchmark.py``.

    python -m velox_b200.cli.benchmark --model DIR [--workload mixed] [--num-requests 16] ...

Option names and meanings are the reference's where it has them (benchmark.py:349-388 of that
project): ``--model``, ``--workload {short,long,mixed}``, ``--num-requests``, ``--max-tokens``,
``--temperature``, ``--top-p``, ``--max-model-len``, ``--max-num-seqs``,
``--max-num-batched-tokens``, ``--max-prefill-chunk-size``, ``--block-size``,
``--num-gpu-blocks``, ``--gpu-memory-utilization``, ``--sweep-batch-size``, ``--show-outputs``,
``--output-json``, ``--seed``.  The reference builds its prompts from English text through a
tokenizer; there is no tokenizer here, so prompts are seeded uniform-random token ids whose
lengths follow the workload (short: 16-64, long: 512-1536, mixed: both).  Added: ``--dtype``,
``--random-weights CONFIG_JSON`` with ``--weights-seed`` (writes the model folder first), and
``--top-k``, ``--model-size NAME`` (random weights with a named configuration's layer sizes,
``--layers N`` of them), ``--prompt-len`` / ``--decode-len`` (fixed lengths), ``--prompt-range
LOW,HIGH`` (lengths uniform in that range), ``--rounds N`` (the reference's option: the same
requests N times on one engine; here it also says whether every round gave the same tokens),
``--batch 1,8,64``
(that many requests and sequences per run) and a roofline line (bytes the steps had to read
over GPU-busy time).  It prints what the reference prints: wall time, steps, prompt and generated
tokens, decode tokens/s (generated / wall), time to first token and inter-token latency
percentiles, the per-stage time of a step, and the sweep table.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import tempfile
import time
from typing import Dict, List, Optional

WORKLOADS = {"short": [(16, 64)], "long": [(512, 1536)], "mixed": [(16, 64), (512, 1536), (128, 384)]}


def parse_args(argv: Optional[List[str]] = None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", default=None, help="model folder (config.json + model.safetensors)")
    parser.add_argument("--random-weights", default=None, metavar="CONFIG_JSON",
                        help="write a random-weights model folder from this config.json first")
    parser.add_argument("--model-size", default=None, metavar="NAME",
                        help="random weights with the layer sizes of a named configuration "
                             "(tiny-a, tiny-b, 0.5b, 1.5b, 3b, 7b, 14b)")
    parser.add_argument("--layers", type=int, default=None,
                        help="with --model-size / --random-weights: build only this many layers")
    parser.add_argument("--weights-seed", type=int, default=0)
    parser.add_argument("--prompt-len", type=int, default=None,
                        help="every prompt has this many tokens (instead of the workload's lengths)")
    parser.add_argument("--prompt-range", default=None, metavar="LOW,HIGH",
                        help="prompt lengths uniform in [LOW, HIGH] (instead of the workload's lengths)")
    parser.add_argument("--rounds", type=int, default=1, help="run the same requests this many times on one engine")
    parser.add_argument("--decode-len", type=int, default=None, help="the same as --max-tokens")
    parser.add_argument("--batch", default=None,
                        help="comma-separated batch sizes: for each, that many requests and max_num_seqs")
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--workload", default="mixed", choices=sorted(WORKLOADS))
    parser.add_argument("--num-requests", type=int, default=16)
    parser.add_argument("--max-tokens", type=int, default=128)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--top-k", type=int, default=0)
    parser.add_argument("--max-model-len", type=int, default=2048)
    parser.add_argument("--max-num-seqs", type=int, default=32)
    parser.add_argument("--max-num-batched-tokens", type=int, default=2048)
    parser.add_argument("--max-prefill-chunk-size", type=int, default=512)
    parser.add_argument("--block-size", type=int, default=64, help="keys per cache page (a power of two)")
    parser.add_argument("--num-gpu-blocks", type=int, default=None)
    parser.add_argument("--gpu-memory-utilization", type=float, default=0.85)
    parser.add_argument("--no-cuda-graphs", action="store_true")
    parser.add_argument("--no-pipeline", action="store_true",
                        help="one step at a time: read a step's tokens before the next step is queued")
    parser.add_argument("--sweep-batch-size", default=None, help="comma-separated max_num_seqs values to sweep")
    parser.add_argument("--show-outputs", action="store_true")
    parser.add_argument("--output-json", default=None)
    parser.add_argument("--seed", type=int, default=0)
    args = parser.parse_args(argv)
    if sum(v is not None for v in (args.model, args.random_weights, args.model_size)) != 1:
        parser.error("give exactly one of --model, --random-weights and --model-size")
    if args.decode_len is not None:
        args.max_tokens = args.decode_len
    if args.batch is not None and args.sweep_batch_size is not None:
        parser.error("--batch and --sweep-batch-size exclude each other")
    return args


def build_prompts(workload: str, count: int, vocab: int, limit: int, seed: int,
                  fixed_len: Optional[int] = None, length_range: Optional[str] = None) -> List[List[int]]:
    import numpy as np

    rng = np.random.default_rng(seed)
    ranges = WORKLOADS[workload] if fixed_len is None else [(fixed_len, fixed_len)]
    if length_range is not None:
        low, high = (int(v) for v in length_range.split(","))
        ranges = [(low, high)]
    prompts = []
    for index in range(count):
        low, high = ranges[index % len(ranges)]
        length = int(min(rng.integers(low, high + 1), limit))
        prompts.append(rng.integers(0, vocab, length).tolist())
    return prompts


def percentile(values: List[float], q: float) -> float:
    if not values:
        return float("nan")
    ordered = sorted(values)
    return ordered[min(len(ordered) - 1, int(q * len(ordered)))]


def run_workload(engine, prompts, args, round_index: int = 0) -> Dict[str, object]:
    from ..engine.request import Request
    from ..sampling.params import SamplingParams

    token_times: Dict[str, List[float]] = {}
    requests = []
    for index, prompt in enumerate(prompts):
        params = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                                max_tokens=args.max_tokens, ignore_eos=True, seed=args.seed + index)
        request = Request(f"bench-{round_index}-{index}", prompt, params)
        token_times[request.request_id] = []
        request.add_listener(
            lambda r, kind, token: token_times[r.request_id].append(time.perf_counter()) if kind == "token" else None
        )
        requests.append(request)
    start = time.perf_counter()
    for request in requests:
        request.arrival_time = time.time()
        engine.add_request(request)
    steps = 0
    live_tokens = 0  # keys the steps' attention reads, summed over the steps
    one_step = engine.step_pipelined if engine.config.pipeline_decode else engine.step
    while engine.has_work():
        live_tokens += sum(r.num_tokens for r in engine.scheduler.running)
        one_step()
        steps += 1
    engine.drain()
    wall = time.perf_counter() - start
    generated = sum(r.num_output_tokens for r in requests)
    ttft = [times[0] - start for times in token_times.values() if times]
    itl = [b - a for times in token_times.values() for a, b in zip(times, times[1:])]
    return {
        "wall_s": wall,
        "steps": steps,
        "prompt_tokens": sum(len(p) for p in prompts),
        "generated_tokens": generated,
        "decode_tok_s": generated / wall if wall > 0 else 0.0,
        "ttft_mean_s": statistics.mean(ttft) if ttft else float("nan"),
        "ttft_p50_s": percentile(ttft, 0.5),
        "ttft_p99_s": percentile(ttft, 0.99),
        "itl_p50_ms": 1000 * percentile(itl, 0.5),
        "itl_p95_ms": 1000 * percentile(itl, 0.95),
        "preemptions": engine.scheduler.num_preemptions,
        "stages_ms": {name: (statistics.mean(v) if v else 0.0) for name, v in engine.stats.items()},
        "blocks_used_peak": None,
        "live_tokens": live_tokens,
        "requests": requests,
    }


def streamed_bytes(model) -> int:
    """Bytes of the matrices a step reads once: every block's and the head's (an embedding that
    is also the head counts once; one that is only looked up does not count)."""
    seen = {}
    parts = [model.lm_head]
    for block in model.blocks:
        parts.extend(getattr(block, name) for name in ("mixer", "feed_forward") if hasattr(block, name))
    for part in parts:
        for tensor in getattr(part, "weights", {}).values():
            if tensor is not None and tensor.dim() == 2:
                seen[tensor.data_ptr()] = tensor.numel() * tensor.element_size()
    return sum(seen.values())


def _measured_peak(key: str, fallback: float) -> float:
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        with open(path, "r", encoding="utf-8") as handle:
            return float(json.load(handle)[key])
    except (OSError, KeyError, ValueError):
        return fallback


def hbm_peak_gbs() -> float:
    """The measured copy bandwidth (``hbm_gbs`` of a ``MEASURED_PEAKS.json`` at the repository's
    root) if that file exists, else 6,650 GB/s, an earlier measurement on a B200."""
    return _measured_peak("hbm_gbs", 6650.0)


def bf16_peak_tflops() -> float:
    """The measured library bf16 matrix-product rate (``bf16_tflops`` of the same file), else
    1,590 TFLOP/s, an earlier measurement on a B200."""
    return _measured_peak("bf16_tflops", 1590.0)


def roofline(engine, result: Dict[str, object]) -> Dict[str, float]:
    """Bytes the run's steps had to read (every matrix once a step, the cache of the live
    requests) over the time the GPU was busy, against the copy bandwidth."""
    gpu_ms = engine.stats.get("gpu_ms", [])
    busy = sum(gpu_ms) / 1000.0
    total_pages = max(1, engine.cache.num_pages)
    per_token = engine.runner.kv_cache_bytes() / (total_pages * engine.cache.page_size)
    needed = streamed_bytes(engine.model) * result["steps"] + per_token * result["live_tokens"]
    achieved = needed / busy / 1e9 if busy > 0 else 0.0
    peak = hbm_peak_gbs()
    return {"hbm_gbs": achieved, "hbm_peak_gbs": peak, "hbm_frac": achieved / peak}


def report(result: Dict[str, object], label: str) -> None:
    print(f"== {label}")
    print(f"wall time          {result['wall_s']:.3f} s   steps {result['steps']}")
    print(f"prompt tokens      {result['prompt_tokens']}   generated tokens {result['generated_tokens']}")
    print(f"decode throughput  {result['decode_tok_s']:.1f} tok/s")
    print(f"TTFT mean / p50 / p99   {result['ttft_mean_s']:.4f} / {result['ttft_p50_s']:.4f} / {result['ttft_p99_s']:.4f} s")
    print(f"ITL p50 / p95      {result['itl_p50_ms']:.3f} / {result['itl_p95_ms']:.3f} ms")
    print(f"preemptions        {result['preemptions']}")
    stages = result["stages_ms"]
    print("per-step stage (mean ms): " + "  ".join(f"{k}={v:.3f}" for k, v in stages.items()))
    if stages.get("step_ms"):
        print(f"GPU-busy fraction  {stages.get('gpu_ms', 0.0) / stages['step_ms']:.2f}")
    if "hbm_gbs" in result:
        print(f"HBM roofline       {result['hbm_gbs']:.0f} of {result['hbm_peak_gbs']:.0f} GB/s = {result['hbm_frac']:.2f} "
              "(weights once a step + cache of the live requests, over GPU-busy time)")


def main(argv: Optional[List[str]] = None) -> int:
    args = parse_args(argv)
    from ..config import EngineConfig
    from ..engine.engine import Engine

    model_dir = args.model
    holder = None
    if args.random_weights is not None or args.model_size is not None:
        from ..weights import write_random_model

        if args.model_size is not None:
            from ..config.presets import model_size

            config_json = model_size(args.model_size)
        else:
            with open(args.random_weights, "r", encoding="utf-8") as handle:
                config_json = json.load(handle)
        if args.layers is not None:
            config_json["num_hidden_layers"] = args.layers
        holder = tempfile.TemporaryDirectory(prefix="velox_model_")
        model_dir = holder.name
        write_random_model(model_dir, config_json, seed=args.weights_seed, dtype="bfloat16")

    sweep = [int(v) for v in args.sweep_batch_size.split(",")] if args.sweep_batch_size else [args.max_num_seqs]
    if args.batch is not None:
        sweep = [int(v) for v in args.batch.split(",")]
    table = []
    for max_num_seqs in sweep:
        num_requests = max_num_seqs if args.batch is not None else args.num_requests
        engine = Engine.from_pretrained(EngineConfig(
            model=model_dir, dtype=args.dtype, max_model_len=args.max_model_len, max_num_seqs=max_num_seqs,
            max_num_batched_tokens=max(args.max_num_batched_tokens, max_num_seqs),
            max_prefill_chunk_size=args.max_prefill_chunk_size, block_size=args.block_size,
            num_gpu_blocks=args.num_gpu_blocks, gpu_memory_utilization=args.gpu_memory_utilization,
            enable_cuda_graphs=not args.no_cuda_graphs, pipeline_decode=not args.no_pipeline, seed=args.seed,
        ))
        limit = engine.max_model_len - args.max_tokens - 1
        prompts = build_prompts(args.workload, num_requests, engine.model.vocab_size, limit, args.seed,
                                fixed_len=args.prompt_len, length_range=args.prompt_range)
        outputs = []
        for round_index in range(max(1, args.rounds)):
            for values in engine.stats.values():
                values.clear()
            preemptions_before = engine.scheduler.num_preemptions
            result = run_workload(engine, prompts, args, round_index)
            result["preemptions"] -= preemptions_before
            result.update(roofline(engine, result))
            suffix = f" round={round_index + 1}" if args.rounds > 1 else ""
            report(result, f"max_num_seqs={max_num_seqs} workload={args.workload} dtype={args.dtype}{suffix}")
            outputs.append([r.output_token_ids for r in result["requests"]])
        if args.rounds > 1:
            same = sum(outputs[0][i] == later[i] for later in outputs[1:] for i in range(len(prompts)))
            print(f"rounds             {same} of {(len(outputs) - 1) * len(prompts)} requests repeated their first round's tokens")
            result["rounds_same_tokens"] = same
        if args.show_outputs:
            for request in result["requests"]:
                print(request.request_id, request.output_token_ids)
        stats = engine.snapshot()
        print("steps with prompt portions: " + ", ".join(
            f"{int(stats.get('mixed_steps_' + how, 0))} {how}" for how in ("replayed", "eager", "captured")))
        table.append({"max_num_seqs": max_num_seqs, **{k: v for k, v in result.items() if k != "requests"},
                      "total_blocks": stats["total_blocks"]})
        del engine
    if len(table) > 1:
        print("== sweep")
        print("max_num_seqs  decode tok/s  TTFT p50 s  preemptions  HBM roofline")
        for row in table:
            print(f"{row['max_num_seqs']:>12}  {row['decode_tok_s']:>12.1f}  {row['ttft_p50_s']:>10.4f}  "
                  f"{row['preemptions']:>11}  {row['hbm_frac']:>12.2f}")
    if args.output_json:
        with open(args.output_json, "w", encoding="utf-8") as handle:
            json.dump(table, handle, indent=1)
    if holder is not None:
        holder.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
