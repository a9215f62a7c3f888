"""How close decode steps come to the memory roofline, per layer, over sizes, batches and contexts.

    python -m velox_b200.cli.roofline --model-size 1.5b,7b --batch 1,8,64 --context 512,4096,32000

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
    from .benchmark import hbm_peak_gbs

    batches = [int(v) for v in args.batch.split(",")]
    contexts = [int(v) for v in args.context.split(",")]
    few, many = (int(v) for v in args.layers.split(","))
    if not 0 < few < many:
        raise SystemExit("--layers A,B needs 0 < A < B")
    peak = hbm_peak_gbs()
    rows = []
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
