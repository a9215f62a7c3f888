"""Plain, slow implementation of the Qwen2.5 dense model, written from the reference's formulas.

Whole sequences, no cache, no batching, one function for each part, plain torch on the CPU (or
wherever the tensors are).  It shares no code with ``velox_b200``: it reads the config.json
dict and the checkpoint tensors by their own names.  Every function cites the file and lines of
the reference (paths inside that project) whose arithmetic it restates.

It was compared once with the reference's own model code, run on the CPU under the Triton
interpreter, on tiny random models: ``tests/golden/make_golden.py`` wrote the small outputs in
``tests/golden/`` and ``tests/test_plain_model.py`` checks this file against them.

The sliding window is the one formula that does not come from the reference, which never reads
``use_sliding_window``: a query at position p sees the keys at positions p-window+1 .. p, in the
layers with index >= ``max_window_layers``.
"""
from __future__ import annotations

import math
from typing import Dict, Mapping, Optional, Sequence

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * w`` (src/rmsnorm.py:20-28)."""
    variance = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(variance + eps) * weight


def rope_angles(head_dim: int, theta: float, factor: float, positions: torch.Tensor) -> torch.Tensor:
    """``angle[p, i] = (p / factor) * theta^(-2i/D)``, built in float32 (src/rope.py:45-56)."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = 1.0 / (theta ** exponent)
    pos = positions.to(torch.float32)
    if factor != 1.0:
        pos = pos / factor
    return torch.outer(pos, inv_freq)


def rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``lo' = lo*cos - hi*sin, hi' = lo*sin + hi*cos`` on the two halves of every head
    (src/rope_inplace.py:25-47; src/rope.py:73-85).  ``x`` is [T, heads, D]; cos, sin [T, D/2]."""
    lo, hi = x.chunk(2, dim=-1)
    c = cos.unsqueeze(1)
    s = sin.unsqueeze(1)
    return torch.cat([lo * c - hi * s, lo * s + hi * c], dim=-1)


def causal_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: float,
    window: Optional[int] = None,
) -> torch.Tensor:
    """Softmax attention of every query over the keys at or before it.

    ``q`` is [T, H, D]; ``k`` and ``v`` are [T, G, D]; query head h uses KV head h // (H/G)
    (src/attention_prefill.py:36).  Scores are ``(q.k) * scale`` with -inf where the key is
    after the query (src/attention_prefill.py:105-117), the softmax is over keys
    (src/attention_prefill.py:119-139).
    """
    T, H, D = q.shape
    G = k.shape[1]
    group = H // G
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("thd,shd->hts", q, k) * scale
    query_pos = torch.arange(T, device=q.device).unsqueeze(1)
    key_pos = torch.arange(T, device=q.device).unsqueeze(0)
    hidden = key_pos > query_pos
    if window is not None:
        hidden = hidden | (key_pos <= query_pos - window)
    scores = scores.masked_fill(hidden.unsqueeze(0), float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hts,shd->thd", probs, v)


def swiglu_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """``down(silu(gate(x)) * up(x))``, no biases (src/mlp.py:9-15)."""
    gate = x @ w_gate.T
    up = x @ w_up.T
    return (torch.nn.functional.silu(gate) * up) @ w_down.T


def attention_block(
    x: torch.Tensor,
    tensors: Mapping[str, torch.Tensor],
    prefix: str,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    cos: torch.Tensor,
    sin: torch.Tensor,
    window: Optional[int],
) -> torch.Tensor:
    """q/k/v projections with bias, RoPE on q and k, attention, bias-free output projection
    (src/self_attention.py:48-90; scale 1/sqrt(D) from src/self_attention.py:35)."""
    T = x.shape[0]
    q = x @ tensors[prefix + "q_proj.weight"].T + tensors[prefix + "q_proj.bias"]
    k = x @ tensors[prefix + "k_proj.weight"].T + tensors[prefix + "k_proj.bias"]
    v = x @ tensors[prefix + "v_proj.weight"].T + tensors[prefix + "v_proj.bias"]
    q = rotate_half(q.view(T, num_heads, head_dim), cos, sin)
    k = rotate_half(k.view(T, num_kv_heads, head_dim), cos, sin)
    v = v.view(T, num_kv_heads, head_dim)
    out = causal_attention(q, k, v, 1.0 / math.sqrt(head_dim), window)
    return out.reshape(T, num_heads * head_dim) @ tensors[prefix + "o_proj.weight"].T


def decoder_layer(
    h: torch.Tensor,
    tensors: Mapping[str, torch.Tensor],
    layer: int,
    cfg: Mapping[str, object],
    cos: torch.Tensor,
    sin: torch.Tensor,
    window: Optional[int],
) -> torch.Tensor:
    """Pre-norm residual block: ``h += attn(norm(h)); h += mlp(norm(h))``
    (src/decoder_layer.py:34-54)."""
    p = f"model.layers.{layer}."
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    heads = int(cfg["num_attention_heads"])
    kv_heads = int(cfg.get("num_key_value_heads", heads))
    head_dim = int(cfg.get("head_dim") or int(cfg["hidden_size"]) // heads)
    x = rms_norm(h, tensors[p + "input_layernorm.weight"], eps)
    h = h + attention_block(x, tensors, p + "self_attn.", heads, kv_heads, head_dim, cos, sin, window)
    x = rms_norm(h, tensors[p + "post_attention_layernorm.weight"], eps)
    return h + swiglu_mlp(
        x,
        tensors[p + "mlp.gate_proj.weight"],
        tensors[p + "mlp.up_proj.weight"],
        tensors[p + "mlp.down_proj.weight"],
    )


def layer_window(cfg: Mapping[str, object], layer: int) -> Optional[int]:
    if not cfg.get("use_sliding_window", False):
        return None
    if layer < int(cfg.get("max_window_layers", cfg["num_hidden_layers"])):
        return None
    return int(cfg["sliding_window"])


def forward_hidden(
    tensors: Mapping[str, torch.Tensor],
    cfg: Mapping[str, object],
    token_ids: Sequence[int],
    dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """Embedding, every layer in order, final norm (src/transformer.py:43-52)."""
    weights: Dict[str, torch.Tensor] = {name: t.to(dtype) for name, t in tensors.items()}
    device = next(iter(weights.values())).device
    ids = torch.as_tensor(list(token_ids), dtype=torch.long, device=device)
    heads = int(cfg["num_attention_heads"])
    head_dim = int(cfg.get("head_dim") or int(cfg["hidden_size"]) // heads)
    scaling = cfg.get("rope_scaling") or {}
    factor = 1.0
    if (scaling.get("type") or scaling.get("rope_type")) == "linear":
        factor = float(scaling.get("factor", 1.0))
    angles = rope_angles(head_dim, float(cfg.get("rope_theta", 10000.0)), factor, torch.arange(len(ids)))
    cos, sin = angles.cos().to(dtype).to(device), angles.sin().to(dtype).to(device)

    h = weights["model.embed_tokens.weight"][ids]
    for layer in range(int(cfg["num_hidden_layers"])):
        h = decoder_layer(h, weights, layer, cfg, cos, sin, layer_window(cfg, layer))
    return rms_norm(h, weights["model.norm.weight"], float(cfg.get("rms_norm_eps", 1e-6)))


def forward_logits(
    tensors: Mapping[str, torch.Tensor],
    cfg: Mapping[str, object],
    token_ids: Sequence[int],
    dtype: torch.dtype = torch.float32,
    rows: Optional[Sequence[int]] = None,
) -> torch.Tensor:
    """Logits at every position (or at ``rows`` only): ``hidden @ lm_head.T``; the head is the
    embedding when ``tie_word_embeddings`` is set (src/transformer.py:60-68)."""
    hidden = forward_hidden(tensors, cfg, token_ids, dtype)
    if rows is not None:
        hidden = hidden[torch.as_tensor(list(rows), dtype=torch.long, device=hidden.device)]
    if cfg.get("tie_word_embeddings", False):
        head = tensors["model.embed_tokens.weight"]
    else:
        head = tensors["lm_head.weight"]
    return hidden @ head.to(dtype).T


def greedy_generate(
    tensors: Mapping[str, torch.Tensor],
    cfg: Mapping[str, object],
    prompt: Sequence[int],
    num_tokens: int,
    dtype: torch.dtype = torch.float32,
) -> list:
    """Argmax decoding by full recompute: the slowest correct generator there is."""
    ids = list(prompt)
    out = []
    for _ in range(num_tokens):
        logits = forward_logits(tensors, cfg, ids, dtype)
        token = int(torch.argmax(logits[-1]).item())
        out.append(token)
        ids.append(token)
    return out
