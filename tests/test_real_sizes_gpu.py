"""The layer sizes that are benchmarked and served, composed: Qwen2.5-0.5B, 1.5B, 3B, 7B and 14B
widths, head counts, inner widths and vocabularies with two layers and random weights, replayed through
the engine with the work laid out as the runner itself chooses (no planner overrides) and
compared with the plain implementation in float64 on the same device.

The tiny configurations pin the arithmetic; these runs pin what only real sizes reach: the
split-K choices of the projections, the LM head over 150k rows, the fused QKV / rotation /
cache-write kernel at 16 clusters, the one-kernel feed-forward (and its refusal at a width of
5,120, where the step must take the two-kernel route), tensor-memory attention over a
2,048-row prompt, library GEMMs with the stand-alone SwiGLU, and cluster-of-eight decode
attention beyond 2,048 keys.  The reference checks its full-size model the same way: every
position of a long prompt fed as one portion, and portions against decoding
(tests/test_engine_e2e.py:127-158,406-441 of that project).
"""
import numpy as np
import pytest
import torch

import plain_model
from helpers import check_logits, random_prompts, read_tensors, write_model

pytestmark = pytest.mark.gpu

PROMPT = 2048
TAIL = 32
# Sums of up to 18,944 float32 terms on both sides.
F32_TOLERANCE = 1e-4

# name -> page size of the cache (the reference's default and this engine's)
SIZES = {"0.5b": 16, "1.5b": 64, "3b": 64, "7b": 16, "14b": 64}
# 0.5B has heads of 64 dims, seven to a KV head (kernels of another head size, a group that does
# not fill a tile of eight); 3B has eight to a KV head and a width of 2,048.
MIXED_LENGTHS = (2300, 700, 150, 333)


def wanted(length):
    """Every 64th position and all of the last 40."""
    return sorted(set(range(0, length, 64)) | set(range(max(0, length - 40), length)))


@pytest.fixture(scope="module", params=list(SIZES))
def sized(request, tmp_path_factory):
    """(name, folder, config, page size, prompts, plain logits at the wanted places)."""
    from velox_b200.config.presets import model_size

    name = request.param
    cfg = dict(model_size(name), num_hidden_layers=2, max_position_embeddings=4096)
    folder = str(tmp_path_factory.mktemp("real_" + name.replace(".", "p")))
    write_model(folder, cfg, seed=31, dtype="bfloat16")
    device = torch.device("cuda:0")
    tensors = {key: value.to(device) for key, value in read_tensors(folder).items()}
    prompts = random_prompts(cfg["vocab_size"], (PROMPT,) + MIXED_LENGTHS, seed=7)
    want = []
    with torch.no_grad():
        for tokens in prompts:
            rows = wanted(len(tokens))
            if len(tokens) == PROMPT:
                rows = sorted(set(rows) | set(range(PROMPT - TAIL, PROMPT)))
            want.append((rows, plain_model.forward_logits(tensors, cfg, tokens, dtype=torch.float64, rows=rows).cpu()))
    del tensors
    torch.cuda.empty_cache()
    yield name, folder, cfg, SIZES[name], prompts, want
    torch.cuda.empty_cache()
    # Gigabytes of weights: not left for pytest's own clean-up, which keeps the last runs.
    import shutil

    shutil.rmtree(folder, ignore_errors=True)


def replay(replayer, name, tokens, cuts, rows):
    """Feed ``tokens`` in portions ``cuts``; logits at the positions ``rows`` (sorted).
    Also returns whether any step split a key range through memory."""
    out, start, split = [], 0, False
    for step, n in enumerate(cuts):
        here = [r - start for r in rows if start <= r < start + n]
        got = replayer.run_step({"step": step, "end": [name] if start + n == len(tokens) else [],
                                 "entries": [{"id": name, "tokens": tokens[start : start + n], "want": here}]})
        if got is not None:
            out.append(got)
        layout = getattr(replayer.runner, "_last_layout", None)
        if layout is not None:
            split = split or any(merge is not None for _, merge in layout[1].values())
        start += n
    assert start == len(tokens)
    return np.concatenate(out, axis=0), split


def changing_cuts(total):
    sizes = [7, 2, 300, 16, 3, 2, 513, 33, 2, 9, 64, 700, 4, 2, 21, 129]
    cuts, left, i = [], total, 0
    while left > 0:
        n = min(sizes[i % len(sizes)], left)
        if left - n == 1:
            n = left
        cuts.append(n)
        left -= n
        i += 1
    return cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_every_way_of_cutting(sized, dtype, monkeypatch):
    from velox_b200.engine.replay import TraceReplayer
    from velox_b200.ops import kernels

    name, folder, cfg, page, prompts, want = sized
    fused_answers = []
    real_mlp_fused = kernels.mlp_fused

    def spying_mlp_fused(*args, **kwargs):
        answer = real_mlp_fused(*args, **kwargs)
        fused_answers.append((args[6], answer))  # (rows of the step, taken or refused)
        return answer

    monkeypatch.setattr(kernels, "mlp_fused", spying_mlp_fused)
    tokens, (rows, ref) = prompts[0], want[0]
    replayer = TraceReplayer(folder, dtype, max_tokens=PROMPT, block_size=page)

    def check(got, what):
        check_logits(got, ref, dtype, f"{name} {dtype} {what}", f32_tolerance=F32_TOLERANCE)

    whole, whole_split = replay(replayer, "whole", tokens, [PROMPT], rows)
    check(whole, "2,048 tokens whole")
    quarters, quarters_split = replay(replayer, "quarters", tokens, [512] * 4, rows)
    check(quarters, "as 4 x 512")
    decoded, decoded_split = replay(replayer, "decoded", tokens, [PROMPT - TAIL] + [1] * TAIL, rows)
    check(decoded, "2,016 at once, the last 32 one by one")
    portions, portions_split = replay(replayer, "portions", tokens, changing_cuts(PROMPT), rows)
    check(portions, "in portions of changing size")

    if dtype == "float32":
        # Same kernels, same order of every sum: equal bits wherever no key range was split
        # through memory, float32 rounding of the merge where one was.
        scale = float(np.abs(whole).max())
        for other, split, what in ((quarters, quarters_split, "4 x 512"), (decoded, decoded_split, "decoded tail"),
                                   (portions, portions_split, "portions")):
            if not (split or whole_split):
                assert np.array_equal(other, whole), f"{name}: {what} differs from the whole prompt in float32"
            else:
                assert float(np.abs(other - whole).max()) <= 1e-5 * scale, f"{name}: {what} is far from the whole prompt"
    else:
        # The single-token steps ran as captured graphs with the fused kernels of small steps.
        assert replayer.runner._graphs and not replayer.runner._graphs_broken
        assert fused_answers, "no small step reached the one-kernel feed-forward"
        # A step's tile of 16 or 32 tokens needs (1 + width / 128) x tile columns of tensor
        # memory out of 512: all small steps at 896 and 1,536, steps of up to 16 tokens at 2,048
        # and 3,584, none at 5,120, where the step must take the two-kernel route (and still
        # match, above).
        width = cfg["hidden_size"]
        for rows_of_step, taken in fused_answers:
            tile = 16 if rows_of_step <= 16 else 32
            assert taken == ((1 + width // 128) * tile <= 512), (width, rows_of_step, taken)
        assert any(taken for _, taken in fused_answers) == (width < 5120)
    replayer.cache.assert_consistent()
    assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages


def mixed_trace(lengths, rng, max_live=4):
    """Up to four live requests; a step feeds portions of some (2 to 512 tokens) beside single
    tokens of others, and some requests sit steps out."""
    progress = [0] * len(lengths)
    waiting = list(range(len(lengths)))
    live, steps = [], []
    while waiting or live:
        while waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        entries, ends = [], []
        for r in list(live):
            left = lengths[r] - progress[r]
            if rng.random() < 0.15 and len(live) > 1:
                continue
            single = left <= 20 or rng.random() < 0.3
            n = 1 if single else min(left, int(rng.choice([2, 3, 17, 64, 200, 512])))
            if left - n == 0:
                ends.append(r)
            entries.append((r, progress[r], n))
            progress[r] += n
        if not entries:
            continue
        steps.append((entries, ends))
        for r in ends:
            live.remove(r)
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_requests_with_page_reuse(sized, dtype):
    from velox_b200.engine.replay import TraceReplayer

    name, folder, cfg, page, prompts, want = sized
    # Each request twice, so that the second pass runs in pages the first gave back; the pool
    # holds the four longest requests (rounded up to 64) and nothing more.
    order = [1, 2, 3, 4, 2, 1, 4, 3]
    seqs = [prompts[i] for i in order]
    need = sum(sorted((-(-len(p) // 64) * 64 for p in seqs), reverse=True)[:4])
    replayer = TraceReplayer(folder, dtype, max_tokens=need, block_size=page)
    steps = mixed_trace([len(p) for p in seqs], np.random.default_rng(11))
    got = [dict() for _ in seqs]
    for step, (entries, ends) in enumerate(steps):
        record = {"step": step, "end": [f"r{r}" for r in ends], "entries": []}
        places = []
        for r, start, n in entries:
            here = [w - start for w in want[order[r]][0] if start <= w < start + n]
            record["entries"].append({"id": f"r{r}", "tokens": seqs[r][start : start + n], "want": here})
            places.extend((r, start + w) for w in here)
        out = replayer.run_step(record)
        for index, (r, position) in enumerate(places):
            got[r][position] = out[index]
        replayer.cache.assert_consistent()
    for r, source in enumerate(order):
        rows, ref = want[source]
        check_logits(np.stack([got[r][w] for w in rows]), ref, dtype, f"{name} {dtype} mixed request {r} ({len(seqs[r])} tokens)",
                     f32_tolerance=F32_TOLERANCE)
    assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
