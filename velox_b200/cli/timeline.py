"""Where the time of a step goes, CTA by CTA, from the timeline build of the kernels.

    python -m velox_b200.cli.timeline --model-size 1.5b --layers 2 --batch 8 --context 4096
    python -m velox_b200.cli.timeline --model-size 1.5b --layers 2 --prefill 8192

With ``VELOX_B200_TRACE=1`` (set here, before anything is loaded) the libraries are built a second
time with ``-DVX_TRACE``: every CTA then appends (kernel, grid, block, SM, start, end, four marks)
to a buffer, read through ``vx_*_trace_setup`` / ``vx_*_trace_count``.  This program runs one
decode step (``--batch`` sequences of ``--context`` keys) or one prompt portion (``--prefill``
tokens behind ``--context`` keys) of a model with random weights and prints, launch by launch,
when its first CTA started and its last ended, how much later it ended than everything before
it, the median CTA and the medians between the marks.  For the tensor-memory attention the marks
are cycle counts instead (low words: the softmax threads' four phases; high words: the MMA
issuer's waits, first products, second products and commits), printed as shares.  The
counters slow the kernels by a tenth to a fifth: the shares are what to read, not the totals.
The reference has nothing of the kind (its profiling is torch.profiler around whole steps,
benchmark.py:233-262 of that project).
"""
from __future__ import annotations

import argparse
import collections
import ctypes
import os
import sys
import tempfile
from typing import List, Optional

KERNEL_NAMES = {
    1: "embed", 2: "norm", 3: "rope/swiglu", 10: "gemm bf16 out", 11: "gemm f32 out", 12: "gemm += stream",
    13: "gemm swiglu", 14: "gemm qkv+rope", 15: "mlp one kernel", 20: "attn mma.sync", 21: "attn narrow",
    22: "attn merge", 23: "attn tcgen05",
}
TC_ATTENTION = 23
EVENT_BYTES = 64


def parse_args(argv: Optional[List[str]] = None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model-size", default="1.5b")
    parser.add_argument("--layers", type=int, default=2)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--prefill", type=int, default=0, metavar="T",
                        help="one prompt portion of T tokens of one sequence instead of a decode step")
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--launches", type=int, default=40, help="launches to list")
    parser.add_argument("--capacity", type=int, default=200000, help="events a buffer holds")
    return parser.parse_args(argv)


def read_events(lib, prefix: str, buffer, capacity: int):
    import numpy as np

    layout = np.dtype([("t0", "<u8"), ("t1", "<u8"), ("kernel", "<i4"), ("grid", "<i4"), ("block", "<i4"),
                       ("sm", "<i4"), ("m0", "<u8"), ("m1", "<u8"), ("m2", "<u8"), ("m3", "<u8")])
    assert layout.itemsize == EVENT_BYTES
    count = ctypes.c_uint(0)
    if getattr(lib, prefix + "_trace_count")(ctypes.byref(count)) != 0:
        raise RuntimeError(f"{prefix}_trace_count failed")
    return np.frombuffer(buffer.cpu().numpy().tobytes(), dtype=layout)[: min(count.value, capacity)]


def group_launches(events):
    """Events in start order, cut into launches: a launch is `grid` events of one (kernel, grid)."""
    pending = collections.defaultdict(list)
    launches = []
    for event in events:
        key = (int(event["kernel"]), int(event["grid"]))
        pending[key].append(event)
        if len(pending[key]) == key[1]:
            launches.append((key, pending.pop(key)))
    launches.sort(key=lambda item: min(int(e["t0"]) for e in item[1]))
    return launches


def main(argv: Optional[List[str]] = None) -> int:
    args = parse_args(argv)
    os.environ["VELOX_B200_TRACE"] = "1"
    import numpy as np
    import torch

    from ..config import EngineConfig
    from ..config.presets import model_size
    from ..engine.engine import Engine
    from ..engine.runner import StepChunk
    from ..ops import kernels
    from ..weights import write_random_model

    config_json = dict(model_size(args.model_size), num_hidden_layers=args.layers)
    tokens = max(args.prefill, 1)
    seqs = 1 if args.prefill else args.batch
    most_keys = args.context + tokens + 16
    with tempfile.TemporaryDirectory(prefix="velox_timeline_") as folder:
        write_random_model(folder, config_json, seed=0, dtype="bfloat16")
        engine = Engine.from_pretrained(EngineConfig(
            model=folder, dtype="bfloat16", max_model_len=most_keys, max_num_seqs=max(seqs, 1),
            max_num_batched_tokens=max(256, tokens, seqs), max_prefill_chunk_size=max(256, tokens),
            block_size=args.block_size, num_gpu_blocks=seqs * (-(-most_keys // args.block_size) + 1) + 8, seed=0))
    runner, cache = engine.runner, engine.cache
    head_dim = config_json.get("head_dim") or config_json["hidden_size"] // config_json["num_attention_heads"]

    def one_step():
        held = []
        chunks = []
        for index in range(seqs):
            seq = cache.new_sequence(f"t{index}")
            if not (cache.acquire_slot(seq) and cache.append_slots(seq, args.context + tokens)):
                raise RuntimeError("the pool is too small for this step")
            cache.advance(seq, args.context)
            held.append(seq)
            ids = [1 + (i % 97) for i in range(tokens)]
            chunks.append(StepChunk(seq, ids, (tokens - 1,)))
        runner.step(chunks)
        torch.cuda.synchronize()
        for seq in held:
            cache.free(seq)
            cache.release_slot(seq)

    for _ in range(4):
        one_step()
    libraries = {"vx_core": kernels.core(), "vx_gemm": kernels.core(), "vx_attn": kernels.attention_lib(head_dim)}
    buffers = {}
    for prefix, lib in libraries.items():
        buffers[prefix] = torch.zeros(args.capacity * EVENT_BYTES, dtype=torch.uint8, device="cuda")
        if getattr(lib, prefix + "_trace_setup")(ctypes.c_void_p(buffers[prefix].data_ptr()),
                                                 ctypes.c_uint(args.capacity)) != 0:
            raise RuntimeError(f"{prefix}_trace_setup failed")
    torch.cuda.synchronize()
    one_step()
    events = np.concatenate([read_events(lib, prefix, buffers[prefix], args.capacity)
                             for prefix, lib in libraries.items()])
    runner.check_status()
    if len(events) == 0:
        print("no events: the libraries were not built with VX_TRACE")
        return 1
    events = events[np.argsort(events["t0"], kind="stable")]
    launches = group_launches(events)
    base = min(int(e["t0"]) for _, group in launches for e in group)
    what = (f"a portion of {args.prefill} tokens behind {args.context} keys" if args.prefill
            else f"a decode step of {args.batch} sequences of {args.context} keys")
    print(f"{args.model_size}, {args.layers} layers, {what}: {len(events)} CTAs in {len(launches)} launches, "
          f"{(max(int(e['t1']) for e in events) - base) / 1e3:.1f} us from the first start to the last end")
    print(f"{'start':>9} {'end':>9} {'adds':>7} {'CTA':>7}  {'kernel':>15} {'grid':>6} {'SMs':>4}  between the marks (us)")
    latest = base
    for key, group in launches[: args.launches]:
        first, last = min(int(e["t0"]) for e in group), max(int(e["t1"]) for e in group)
        median = float(np.median([int(e["t1"]) - int(e["t0"]) for e in group]))
        line = (f"{(first - base) / 1e3:9.2f} {(last - base) / 1e3:9.2f} {(last - latest) / 1e3:7.2f} {median / 1e3:7.2f}  "
                f"{KERNEL_NAMES.get(key[0], str(key[0])):>15} {key[1]:6d} {len(set(int(e['sm']) for e in group)):4d}  ")
        if key[0] != TC_ATTENTION:
            points = ["t0", "m0", "m1", "m2", "m3", "t1"]
            gaps = []
            for a, b in zip(points, points[1:]):
                values = [int(e[b]) - int(e[a]) for e in group if e[a] and e[b]]
                gaps.append(f"{np.median(values) / 1e3:5.2f}" if values else "    -")
            line += " ".join(gaps)
        print(line)
        latest = max(latest, last)
    totals = collections.defaultdict(lambda: [0, 0.0])
    for key, group in launches:
        entry = totals[(KERNEL_NAMES.get(key[0], str(key[0])), key[1])]
        entry[0] += 1
        entry[1] += (max(int(e["t1"]) for e in group) - min(int(e["t0"]) for e in group)) / 1e3
    print("by kernel and grid (first start to last end, summed over the launches):")
    for (name, grid), (count, total) in sorted(totals.items(), key=lambda item: -item[1][1]):
        print(f"  {name:>15} grid {grid:6d}: {count:4d} launches, {total:9.1f} us, {total / count:7.2f} each")
    walked = [e for e in events if int(e["kernel"]) == TC_ATTENTION and (int(e["m0"]) & 0xffffffff) > 0]
    if walked:
        low = np.array([[int(e[f"m{i}"]) & 0xffffffff for i in range(4)] for e in walked], dtype=np.float64)
        high = np.array([[int(e[f"m{i}"]) >> 32 for i in range(4)] for e in walked], dtype=np.float64)
        share = low.sum(0) / low.sum()
        print("tensor-memory attention, cycles summed over all CTAs and key tiles:")
        print("  softmax threads: waiting for scores %.0f %%, scores into registers %.0f %%, masks and maximum %.0f %%, "
              "exponentials and P %.0f %%" % tuple(100 * share))
        print("  MMA issuer, as shares of the softmax threads' cycles: waiting %.0f %%, issuing first products %.0f %%, "
              "second products %.0f %%, commits %.0f %%" % tuple(100 * high.sum(0) / low.sum()))
    return 0


if __name__ == "__main__":
    sys.exit(main())
