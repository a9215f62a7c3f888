"""The plain implementation against the reference's own model code (golden files) and itself."""
import os

import numpy as np
import pytest
import torch

import plain_model
import tiny_configs
from helpers import read_tensors, write_model

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("case", ["tiny_a", "tiny_b"])
def test_plain_matches_reference_golden(case, tmp_path):
    data = np.load(os.path.join(GOLDEN, f"{case}.npz"))
    cfg = tiny_configs.ALL[case]
    write_model(str(tmp_path), cfg, seed=int(data["weights_seed"]), dtype="float32")
    tensors = read_tensors(str(tmp_path))
    index = 0
    while f"ids_{index}" in data:
        ids = data[f"ids_{index}"].tolist()
        want = torch.from_numpy(data[f"logits_{index}"])
        got = plain_model.forward_logits(tensors, cfg, ids, dtype=torch.float32)
        assert got.shape == want.shape
        scale = want.abs().max().item()
        # Both sides are float32 with different summation orders.
        assert (got - want).abs().max().item() <= 2e-5 * max(scale, 1.0)
        assert torch.equal(got.argmax(-1), want.argmax(-1))
        index += 1
    assert index >= 3


def test_plain_is_causal(tmp_path):
    cfg = tiny_configs.TINY_A
    write_model(str(tmp_path), cfg, seed=3, dtype="float32")
    tensors = read_tensors(str(tmp_path))
    ids = list(range(20))
    full = plain_model.forward_logits(tensors, cfg, ids, dtype=torch.float64)
    short = plain_model.forward_logits(tensors, cfg, ids[:9], dtype=torch.float64)
    assert torch.allclose(full[:9], short, atol=1e-12)


def test_plain_window_hides_old_keys():
    T, H, D = 12, 2, 8
    gen = torch.Generator().manual_seed(0)
    q = torch.randn(T, H, D, generator=gen, dtype=torch.float64)
    k = torch.randn(T, H, D, generator=gen, dtype=torch.float64)
    v = torch.randn(T, H, D, generator=gen, dtype=torch.float64)
    windowed = plain_model.causal_attention(q, k, v, 0.3, window=4)
    # The last query sees keys 8..11 only: changing key/value 7 must not matter, 8 must.
    k2, v2 = k.clone(), v.clone()
    k2[7] += 5.0
    v2[7] -= 3.0
    assert torch.allclose(plain_model.causal_attention(q, k2, v2, 0.3, window=4)[-1], windowed[-1])
    v3 = v.clone()
    v3[8] += 1.0
    assert not torch.allclose(plain_model.causal_attention(q, k, v3, 0.3, window=4)[-1], windowed[-1])
    # A window as long as the sequence is plain causal attention.
    assert torch.allclose(
        plain_model.causal_attention(q, k, v, 0.3, window=T), plain_model.causal_attention(q, k, v, 0.3)
    )


def test_rope_rotation_preserves_norm_and_is_relative():
    D = 16
    pos = torch.arange(32)
    ang = plain_model.rope_angles(D, 10000.0, 1.0, pos).double()
    x = torch.randn(32, 1, D, dtype=torch.float64)
    y = plain_model.rotate_half(x, ang.cos(), ang.sin())
    assert torch.allclose(x.norm(dim=-1), y.norm(dim=-1))
    # dot(rot(a, p), rot(b, p + d)) depends on d only
    a = torch.randn(D, dtype=torch.float64).expand(32, 1, D)
    b = torch.randn(D, dtype=torch.float64).expand(32, 1, D)
    ra = plain_model.rotate_half(a, ang.cos(), ang.sin())
    rb = plain_model.rotate_half(b, ang.cos(), ang.sin())
    d1 = (ra[3, 0] * rb[8, 0]).sum()
    d2 = (ra[13, 0] * rb[18, 0]).sum()
    # angles are built in float32, as the reference builds them
    assert abs(d1 - d2) < 1e-4


def test_greedy_generate_runs(tmp_path):
    cfg = tiny_configs.TINY_A
    write_model(str(tmp_path), cfg, seed=5, dtype="float32")
    tensors = read_tensors(str(tmp_path))
    out = plain_model.greedy_generate(tensors, cfg, [1, 2, 3], 4)
    assert len(out) == 4 and all(0 <= t < cfg["vocab_size"] for t in out)
