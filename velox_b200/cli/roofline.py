"""How close decode steps come to the memory roofline, and prompt portions to the matrix-product
peak, per layer, over sizes, batches and contexts.

    python -m velox_b200.cli.roofline --model-size 1.5b,7b --batch 1,8,64 --context 512,4096,32000
    python -m velox_b200.cli.roofline --model-size 1.5b,7b --prefill 512,2048 --context 0,8192,30000

For every named configuration two models with random weights are built, with ``--layers A,B``
layers (2 and 6 unless told otherwise); for every batch and context each runs decode steps whose
sequences hold that many keys, and the difference of the two step times over B - A is what one
layer costs: embedding, head, sampling and the host's share of a step cancel.  A layer has to read
its matrices once and the keys and values of the live requests; those bytes over the layer's time,
against the measured copy bandwidth, is the fraction printed.  The reference has no counterpart;
its benchmark reports tokens per second only (benchmark.py:233-262 of that project).

The cache is not filled through the model (the keys are whatever the pool holds): the step's work
does not depend on their values.  Steps are queued back to back, each fed the tokens the step
before it sampled (on the device), so the device never waits for the host.

With ``--prefill T,...`` the steps are portions of T prompt tokens of one sequence behind
``--context`` keys instead: a layer's floating-point operations (two per weight and token, four
per query, key and head dimension under the causal mask) over its time, against the measured
library bf16 rate.
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile
from typing import Dict, List, Optional, Tuple


def parse_args(argv: Optional[List[str]] = None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model-size", default="1.5b", help="named configurations, comma separated")
    parser.add_argument("--batch", default="1,8,64")
    parser.add_argument("--context", default="512,4096")
    parser.add_argument("--prefill", default=None, metavar="T,...",
                        help="time prompt portions of so many tokens behind --context keys instead of decode steps")
    parser.add_argument("--layers", default="2,6", help="the two layer counts whose difference is taken")
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--steps", type=int, default=24)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--output-json", default=None)
    return parser.parse_args(argv)


def layer_bytes(config_json: Dict, batch: int, context: int) -> Tuple[int, int]:
    """(bytes of one layer's matrices in bfloat16, bytes of ``batch`` x ``context`` keys and
    values of one layer)."""
    width, heads, kv_heads = config_json["hidden_size"], config_json["num_attention_heads"], config_json["num_key_value_heads"]
    inner = config_json["intermediate_size"]
    head_dim = config_json.get("head_dim") or width // heads
    weights = 2 * (width * (heads + 2 * kv_heads) * head_dim + heads * head_dim * width + 3 * width * inner)
    cache = batch * context * kv_heads * head_dim * 2 * 2
    return weights, cache


def layer_flops(config_json: Dict, tokens: int, context: int) -> float:
    """Floating-point operations of one layer on a portion of ``tokens`` behind ``context`` keys."""
    width, heads, kv_heads = config_json["hidden_size"], config_json["num_attention_heads"], config_json["num_key_value_heads"]
    inner = config_json["intermediate_size"]
    head_dim = config_json.get("head_dim") or width // heads
    weights = width * (heads + 2 * kv_heads) * head_dim + heads * head_dim * width + 3 * width * inner
    return 2.0 * tokens * weights + 4.0 * tokens * (context + (tokens + 1) / 2.0) * heads * head_dim


def portion_times(config_json: Dict, layers: int, portions: List[int], contexts: List[int], args) -> Dict[Tuple[int, int], float]:
    """Milliseconds of a step that is one portion of a prompt, for every (portion, context)."""
    import torch

    from ..config import EngineConfig
    from ..engine.engine import Engine
    from ..engine.runner import StepChunk
    from ..weights import write_random_model

    most_tokens, most_keys = max(portions), max(contexts) + max(portions) + 8
    with tempfile.TemporaryDirectory(prefix="velox_roofline_") as folder:
        write_random_model(folder, dict(config_json, num_hidden_layers=layers), seed=0, dtype="bfloat16")
        engine = Engine.from_pretrained(EngineConfig(
            model=folder, dtype="bfloat16", max_model_len=most_keys, max_num_seqs=2,
            max_num_batched_tokens=most_tokens, max_prefill_chunk_size=most_tokens, block_size=args.block_size,
            num_gpu_blocks=2 * (-(-most_keys // args.block_size) + 1) + 8, seed=0))
    runner, cache = engine.runner, engine.cache
    times: Dict[Tuple[int, int], float] = {}
    for tokens in portions:
        ids = [1 + (i % 97) for i in range(tokens)]
        for context in contexts:
            measured = []
            for repeat in range(args.warmup + 3):
                seq = cache.new_sequence(f"p{tokens}_{context}_{repeat}")
                if not (cache.acquire_slot(seq) and cache.append_slots(seq, context + tokens)):
                    raise RuntimeError(f"the pool does not hold {context + tokens} keys")
                cache.advance(seq, context)
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                start.record()
                runner.step([StepChunk(seq, ids, (tokens - 1,))])
                end.record()
                torch.cuda.synchronize()
                cache.free(seq)
                cache.release_slot(seq)
                if repeat >= args.warmup:
                    measured.append(start.elapsed_time(end))
            times[(tokens, context)] = sorted(measured)[len(measured) // 2]
    runner.check_status()
    del engine, runner, cache
    torch.cuda.empty_cache()
    return times


def step_times(config_json: Dict, layers: int, batches: List[int], contexts: List[int], args) -> Dict[Tuple[int, int], float]:
    """Milliseconds of a decode step for every (batch, context), with ``layers`` layers."""
    import torch

    from ..config import EngineConfig
    from ..engine.engine import Engine
    from ..engine.runner import StepChunk
    from ..sampling.params import SamplingParams
    from ..weights import write_random_model

    most_seqs, most_keys = max(batches), max(contexts) + args.steps + args.warmup + 2
    with tempfile.TemporaryDirectory(prefix="velox_roofline_") as folder:
        write_random_model(folder, dict(config_json, num_hidden_layers=layers), seed=0, dtype="bfloat16")
        engine = Engine.from_pretrained(EngineConfig(
            model=folder, dtype="bfloat16", max_model_len=most_keys, max_num_seqs=most_seqs,
            max_num_batched_tokens=max(256, most_seqs), max_prefill_chunk_size=256, block_size=args.block_size,
            num_gpu_blocks=most_seqs * (-(-most_keys // args.block_size) + 1) + 8, seed=0))
    runner, cache, sampler = engine.runner, engine.cache, engine.sampler
    times: Dict[Tuple[int, int], float] = {}
    for batch in batches:
        params = [SamplingParams(temperature=0.0, max_tokens=1)] * batch
        names = [f"s{i}" for i in range(batch)]
        for context in contexts:
            seqs = []
            for name in names:
                seq = cache.new_sequence(name)
                if not (cache.acquire_slot(seq) and cache.append_slots(seq, context)):
                    raise RuntimeError(f"the pool does not hold {batch} sequences of {context} keys")
                cache.advance(seq, context)
                seqs.append(seq)

            def one_step(ids):
                chunks = []
                for seq, token in zip(seqs, ids):
                    cache.append_slots(seq, 1)
                    chunks.append(StepChunk(seq, [token], (0,)))
                logits = runner.step(chunks)
                sampler.sample(logits, params, names, [0] * batch)
                for seq in seqs:
                    cache.advance(seq, 1)

            for _ in range(args.warmup):
                one_step([1] * batch)
            fed = [-1 - row for row in range(batch)]
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(args.steps):
                one_step(fed)
            end.record()
            torch.cuda.synchronize()
            times[(batch, context)] = start.elapsed_time(end) / args.steps
            for seq in seqs:
                cache.free(seq)
                cache.release_slot(seq)
    runner.check_status()
    del engine, runner, cache, sampler
    torch.cuda.empty_cache()
    return times


def main(argv: Optional[List[str]] = None) -> int:
    args = parse_args(argv)
    from ..config.presets import model_size
    from .benchmark import bf16_peak_tflops, hbm_peak_gbs

    batches = [int(v) for v in args.batch.split(",")]
    contexts = [int(v) for v in args.context.split(",")]
    few, many = (int(v) for v in args.layers.split(","))
    if not 0 < few < many:
        raise SystemExit("--layers A,B needs 0 < A < B")
    rows = []
    if args.prefill:
        portions = [int(v) for v in args.prefill.split(",")]
        rate = bf16_peak_tflops()
        print(f"{'size':>6} {'tokens':>6} {'context':>7} {'us/layer':>9} {'TFLOP/s':>8} {'fraction':>8}")
        for name in args.model_size.split(","):
            config_json = model_size(name)
            short = portion_times(config_json, few, portions, contexts, args)
            long = portion_times(config_json, many, portions, contexts, args)
            for tokens in portions:
                for context in contexts:
                    seconds = (long[(tokens, context)] - short[(tokens, context)]) / (many - few) * 1e-3
                    achieved = layer_flops(config_json, tokens, context) / seconds / 1e12 if seconds > 0 else 0.0
                    row = {"size": name, "tokens": tokens, "context": context, "us_per_layer": round(seconds * 1e6, 1),
                           "tflops": round(achieved, 1), "bf16_frac": round(achieved / rate, 3), "bf16_peak_tflops": rate,
                           "kv_block_size": args.block_size}
                    rows.append(row)
                    print(f"{name:>6} {tokens:>6} {context:>7} {row['us_per_layer']:>9.1f} {row['tflops']:>8.1f} "
                          f"{row['bf16_frac']:>8.3f}", flush=True)
        if args.output_json:
            with open(args.output_json, "w", encoding="utf-8") as handle:
                json.dump(rows, handle, indent=1)
        return 0
    peak = hbm_peak_gbs()
    print(f"{'size':>6} {'batch':>5} {'context':>7} {'us/layer':>9} {'by bytes':>9} {'fraction':>8}  cache share")
    for name in args.model_size.split(","):
        config_json = model_size(name)
        short = step_times(config_json, few, batches, contexts, args)
        long = step_times(config_json, many, batches, contexts, args)
        for batch in batches:
            for context in contexts:
                # the sequences grow while they are timed: count the keys of the middle step
                keys = context + args.warmup + args.steps // 2
                weights, cached = layer_bytes(config_json, batch, keys)
                seconds = (long[(batch, context)] - short[(batch, context)]) / (many - few) * 1e-3
                ideal = (weights + cached) / (peak * 1e9)
                row = {"size": name, "batch": batch, "context": context, "us_per_layer": round(seconds * 1e6, 1),
                       "us_by_bytes": round(ideal * 1e6, 1), "hbm_frac": round(ideal / seconds, 3) if seconds > 0 else None,
                       "cache_share": round(cached / (weights + cached), 2), "hbm_peak_gbs": peak,
                       "kv_block_size": args.block_size}
                rows.append(row)
                print(f"{name:>6} {batch:>5} {context:>7} {row['us_per_layer']:>9.1f} {row['us_by_bytes']:>9.1f} "
                      f"{row['hbm_frac']:>8.3f}  {row['cache_share']:.2f}", flush=True)
    if args.output_json:
        with open(args.output_json, "w", encoding="utf-8") as handle:
            json.dump(rows, handle, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
