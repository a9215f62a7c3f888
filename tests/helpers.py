"""Shared helpers of the tests: model folders in temporary places, prompts, tensors by name."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Sequence

import numpy as np
import torch


def write_model(folder: str, cfg: Dict[str, Any], seed: int, dtype: str = "float32") -> None:
    from velox_b200.weights import write_random_model

    write_random_model(folder, cfg, seed=seed, dtype=dtype)


def read_tensors(folder: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return load_file(os.path.join(folder, "model.safetensors"))


def read_config(folder: str) -> Dict[str, Any]:
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as handle:
        return json.load(handle)


def random_prompt(vocab: int, length: int, seed: int) -> List[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=gen).tolist()


def random_prompts(vocab: int, lengths: Sequence[int], seed: int) -> List[List[int]]:
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in lengths]


F32_TOLERANCE = 2e-5
BF16_TOLERANCE = 3e-2
BF16_MIN_COSINE = 0.999
BF16_MIN_ARGMAX_AGREEMENT = 0.95


def check_logits(got_rows, want_rows, dtype: str, what: str, f32_tolerance: float = F32_TOLERANCE) -> None:
    """Engine logits against the plain implementation's (float64), row by row.

    float32: both sides round differently in sums of a few hundred to a few thousand terms; the
    largest error must stay below ``f32_tolerance`` of the logits' scale, and the argmax must
    agree wherever the plain top two are further apart than twice that.

    bfloat16: activations are rounded to 8 bits of mantissa about six times per layer, which
    over a few layers is about 1e-2 of the activations' scale (3 sigma: 3e-2).  Three checks,
    each per row, so that a row of small logits cannot hide behind a large one elsewhere: the
    largest error against 3e-2 of the row's own largest logit, the cosine between the two rows
    (at least 0.999), and the argmax, which must agree in at least 95 % of the rows whose plain
    top two are further apart than the row's tolerance."""
    got = torch.from_numpy(np.ascontiguousarray(np.asarray(got_rows))).double()
    want = want_rows.detach().double().cpu()
    assert got.shape == want.shape, (what, tuple(got.shape), tuple(want.shape))
    assert torch.isfinite(got).all(), f"{what}: logits are not finite"
    err = (got - want).abs().amax(-1)
    top2 = want.topk(2, dim=-1).values
    gap = top2[:, 0] - top2[:, 1]
    same = got.argmax(-1) == want.argmax(-1)
    if dtype == "float32":
        scale = max(want.abs().max().item(), 1e-3)
        worst = err.max().item()
        assert worst <= f32_tolerance * scale, f"{what}: max abs error {worst:.3e}, logit scale {scale:.3e}"
        clear = gap > 2 * f32_tolerance * scale
        assert bool(same[clear].all()), f"{what}: argmax differs at rows {torch.nonzero(clear & ~same).flatten().tolist()[:8]}"
        return
    row_scale = want.abs().amax(-1).clamp_min(1e-3)
    ratio = err / row_scale
    worst_row = int(ratio.argmax())
    assert ratio[worst_row].item() <= BF16_TOLERANCE, (
        f"{what}: row {worst_row}: max abs error {err[worst_row].item():.3e}, its largest logit {row_scale[worst_row].item():.3e}")
    cosine = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert cosine.min().item() >= BF16_MIN_COSINE, f"{what}: row {int(cosine.argmin())}: cosine {cosine.min().item():.5f}"
    clear = gap > BF16_TOLERANCE * row_scale
    if int(clear.sum()) > 0:
        agreement = same[clear].double().mean().item()
        assert agreement >= BF16_MIN_ARGMAX_AGREEMENT, f"{what}: argmax agrees in {agreement:.3f} of {int(clear.sum())} clear rows"
