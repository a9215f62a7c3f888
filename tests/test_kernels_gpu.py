"""Each CUDA kernel alone against a plain float64 torch statement of the same operation, at
sizes other than the engine's test models: widths and vocabularies that are no power of two,
head sizes in steps of 16, every grouping of query heads, windows, split key ranges, pages
in shuffled order."""
import math

import numpy as np
import pytest
import torch

import plain_model

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype):
    # float32: summation-order noise only.  bfloat16: one rounding of the output (2^-9 relative)
    # plus rounding of products inside, a few ulp.
    return (3e-6, 3e-6) if dtype == torch.float32 else (2e-2, 1e-2)


def _close(got, want, dtype, scale=None):
    got = got.double().cpu()
    want = want.double().cpu()
    rtol, atol = _tol(dtype)
    scale = float(want.abs().max()) if scale is None else scale
    err = (got - want).abs().max().item()
    assert err <= atol * max(scale, 1e-6) + 1e-12, f"max abs error {err:.3e} at scale {scale:.3e}"


@pytest.fixture(scope="module")
def k():
    from velox_b200.ops import kernels

    kernels._require_cuda()
    return kernels


@pytest.fixture()
def status():
    return torch.zeros(4, dtype=torch.int32, device="cuda")


# ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab", [(64, 100), (1536, 777), (250, 33)])
def test_embed(k, status, dtype, hidden, vocab):
    gen = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, hidden, generator=gen).to(dtype).cuda()
    ids = torch.randint(0, vocab, (37,), generator=gen, dtype=torch.int32).cuda()
    resid = torch.full((40, hidden), 7.0, device="cuda")
    k.embed(table, ids, resid, status)
    assert torch.equal(resid[:37], table[ids.long()].float())
    assert torch.all(resid[37:] == 7.0)
    assert int(status[0]) == 0
    bad = ids.clone()
    bad[3] = vocab
    k.embed(table, bad, resid, status)
    assert int(status[0]) & 1
    assert torch.all(resid[3] == 0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [64, 240, 1000, 1536, 5120])
@pytest.mark.parametrize("with_delta", [False, True])
def test_add_rmsnorm(k, dtype, hidden, with_delta):
    gen = torch.Generator().manual_seed(hidden)
    T = 19
    resid = (torch.randn(T, hidden, generator=gen) * 3).cuda()
    delta = torch.randn(T, hidden, generator=gen).to(dtype).cuda() if with_delta else None
    weight = (1 + 0.1 * torch.randn(hidden, generator=gen)).cuda()
    eps = 1e-5
    out = torch.empty(T, hidden, dtype=dtype, device="cuda")
    before = resid.clone()
    k.add_rmsnorm(resid, delta, weight, eps, out, T)
    v = before.double() + (delta.double() if with_delta else 0)
    want = plain_model.rms_norm(v, weight.double(), eps)
    _close(out, want, dtype)
    assert torch.allclose(resid.double(), v, atol=1e-6)
    # Selected rows, residual left alone.
    rows = torch.tensor([5, 0, 18], dtype=torch.int32, device="cuda")
    out2 = torch.empty(3, hidden, dtype=dtype, device="cuda")
    resid2 = before.clone()
    k.add_rmsnorm(resid2, delta, weight, eps, out2, 3, rows=rows, write_resid=False)
    _close(out2, want[rows.long().cpu()], dtype)
    assert torch.equal(resid2, before)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,rot", [(4, 2, 16, 16), (5, 5, 48, 48), (6, 2, 80, 80), (12, 2, 128, 128), (3, 1, 64, 32)])
def test_rope_cache_write(k, status, dtype, H, G, D, rot):
    gen = torch.Generator().manual_seed(D)
    T, pages, P = 23, 9, 4
    qkv = torch.randn(T, (H + 2 * G) * D, generator=gen).to(dtype).cuda()
    positions = torch.randint(0, 200, (T,), generator=gen, dtype=torch.int32).cuda()
    angles = plain_model.rope_angles(rot, 10000.0, 1.0, torch.arange(200))
    cos, sin = angles.cos().cuda().contiguous(), angles.sin().cuda().contiguous()
    slots = torch.randperm(pages * P, generator=gen)[:T].to(torch.int32)
    slots[7] = -1
    slots = slots.cuda()
    k_cache = torch.zeros(pages, P, G, D, dtype=dtype, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    original = qkv.clone()
    k.rope_cache_write(qkv, positions, cos, sin, slots, k_cache, v_cache, T, H, G, D, rot, status)
    assert int(status[0]) == 0

    src = original.double().cpu()
    q = src[:, : H * D].view(T, H, D)
    kk = src[:, H * D : (H + G) * D].view(T, G, D)
    vv = src[:, (H + G) * D :].view(T, G, D)
    c = angles.cos().double()[positions.long().cpu()]
    s = angles.sin().double()[positions.long().cpu()]

    def rotate(x):
        rotated = plain_model.rotate_half(x[..., :rot], c, s)
        return torch.cat([rotated, x[..., rot:]], dim=-1)

    _close(qkv[:, : H * D].view(T, H, D), rotate(q), dtype)
    # k and v columns of the qkv buffer are left as they were
    assert torch.equal(qkv[:, H * D :], original[:, H * D :])
    flat_k = k_cache.view(-1, G, D)
    flat_v = v_cache.view(-1, G, D)
    want_k = rotate(kk)
    for t in range(T):
        slot = int(slots[t])
        if slot < 0:
            continue
        _close(flat_k[slot], want_k[t], dtype, scale=float(want_k.abs().max()))
        assert torch.equal(flat_v[slot].double().cpu(), vv[t].to(dtype).double())
    written = set(int(x) for x in slots.tolist() if x >= 0)
    for slot in range(pages * P):
        if slot not in written:
            assert torch.all(flat_k[slot] == 0) and torch.all(flat_v[slot] == 0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,inter", [(1, 128), (17, 704), (5, 8960), (3, 333)])
def test_swiglu(k, dtype, T, inter):
    gen = torch.Generator().manual_seed(inter)
    gate_up = (torch.randn(T + 2, 2 * inter, generator=gen) * 2).to(dtype).cuda()
    out = torch.empty(T + 2, inter, dtype=dtype, device="cuda")
    k.swiglu(gate_up, out, T)
    g = gate_up[:T, :inter].double()
    u = gate_up[:T, inter:].double()
    _close(out[:T], torch.nn.functional.silu(g) * u, dtype)


@pytest.mark.parametrize("M,N,K", [(1, 33, 5), (7, 704, 250), (65, 64, 64), (130, 100, 1536), (3, 1, 17)])
@pytest.mark.parametrize("bias", [False, True])
def test_gemm_f32(k, M, N, K, bias):
    gen = torch.Generator().manual_seed(M * N + K)
    a = torch.randn(M + 3, K, generator=gen).cuda()
    w = torch.randn(N, K, generator=gen).cuda()
    b = torch.randn(N, generator=gen).cuda() if bias else None
    out = torch.full((M + 3, N), 5.0, device="cuda")
    k.gemm_f32(a, w, b, out, M)
    want = a[:M].double() @ w.double().T + (b.double() if bias else 0)
    err = (out[:M].double() - want).abs().max().item()
    # K float32 additions in sequence: rounding errors of 2^-24 relative to the running sum
    # add up like a random walk, sqrt(K) of them
    assert err <= 2 * 2.0 ** -24 * math.sqrt(K) * want.abs().max().item() + 1e-6, err
    assert torch.all(out[M:] == 5.0)


def test_gemm_f32_rows_do_not_depend_on_batch(k):
    gen = torch.Generator().manual_seed(1)
    a = torch.randn(70, 300, generator=gen).cuda()
    w = torch.randn(129, 300, generator=gen).cuda()
    full = torch.empty(70, 129, device="cuda")
    k.gemm_f32(a, w, None, full, 70)
    one = torch.empty(1, 129, device="cuda")
    for row in (0, 33, 69):
        k.gemm_f32(a[row : row + 1].contiguous(), w, None, one, 1)
        assert torch.equal(one[0], full[row])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,T", [(1536, 700), (3584, 300), (240, 513), (4100, 260)])
def test_add_rmsnorm_many_rows(k, dtype, hidden, T):
    """Steps of many rows (a warp per row in bfloat16), with and without rows to add, selected
    rows, and a tail that does not fill the last block."""
    gen = torch.Generator().manual_seed(hidden + T)
    resid = (torch.randn(T + 2, hidden, generator=gen) * 3).cuda()
    delta = torch.randn(T + 2, hidden, generator=gen).to(dtype).cuda()
    weight = (1 + 0.1 * torch.randn(hidden, generator=gen)).cuda()
    before = resid.clone()
    out = torch.full((T + 2, hidden), 5.0, dtype=dtype, device="cuda")
    k.add_rmsnorm(resid, delta, weight, 1e-6, out, T)
    v = before[:T].double() + delta[:T].double()
    want = plain_model.rms_norm(v, weight.double(), 1e-6)
    _close(out[:T], want, dtype)
    assert torch.allclose(resid[:T].double(), v, atol=1e-6)
    assert torch.equal(resid[T:], before[T:]) and bool((out[T:] == 5.0).all())  # rows past the step untouched
    picked = min(300, T)  # as many rows as the index array names, never more
    rows = torch.randperm(T, generator=gen)[:picked].to(torch.int32).cuda()
    out2 = torch.empty(picked, hidden, dtype=dtype, device="cuda")
    resid2 = before.clone()
    k.add_rmsnorm(resid2, None, weight, 1e-6, out2, picked, rows=rows, write_resid=False)
    _close(out2, plain_model.rms_norm(before.double()[rows.long()], weight.double(), 1e-6), dtype)
    assert torch.equal(resid2, before)


# ----------------------------------------------------------------------------------------------
# Attention
# ----------------------------------------------------------------------------------------------
def plain_paged_attention(q, k_all, v_all, ctx, scale, window):
    """q [n, H, D] at positions ctx..ctx+n-1 over keys/values [ctx+n, G, D] (float64)."""
    n, H, D = q.shape
    G = k_all.shape[1]
    group = H // G
    kk = k_all.repeat_interleave(group, dim=1)
    vv = v_all.repeat_interleave(group, dim=1)
    scores = torch.einsum("thd,shd->hts", q, kk) * scale
    qpos = (ctx + torch.arange(n)).unsqueeze(1)
    kpos = torch.arange(k_all.shape[0]).unsqueeze(0)
    hidden = kpos > qpos
    if window:
        hidden = hidden | (kpos <= qpos - window)
    scores = scores.masked_fill(hidden.unsqueeze(0), float("-inf"))
    return torch.einsum("hts,shd->thd", torch.softmax(scores, -1), vv)


def run_attention_case(k, dtype, H, G, D, P, seqs, window=None, seed=0, min_split_keys=256,
                       target_ctas=296, spike=None, fused_merge=True, max_cluster=1, max_splits=64,
                       tensor_memory=False, ramp=None, tc_ctas_per_sm=1, tc_merge_us=30.0):
    """seqs: list of (q_len, ctx_len).  Returns (got, want) as float64 [T, H, D]."""
    from velox_b200.ops import attention_plan as ap

    gen = torch.Generator().manual_seed(seed)
    group = H // G
    total_pages = sum(-(-(q + c) // P) for q, c in seqs) + 3
    order = (torch.randperm(total_pages - 1, generator=gen) + 1).tolist()
    k_cache = torch.randn(total_pages, P, G, D, generator=gen).to(dtype)
    v_cache = torch.randn(total_pages, P, G, D, generator=gen).to(dtype)
    T = sum(q for q, _ in seqs)
    qkv = torch.randn(T, (H + 2 * G) * D, generator=gen).to(dtype)
    width = max(-(-(q + c) // P) for q, c in seqs)
    tables = torch.zeros(len(seqs), width, dtype=torch.int32)
    q_start, q_lens, kv_lens = [], [], []
    want = torch.zeros(T, H, D, dtype=torch.float64)
    row = 0
    for s, (q_len, ctx) in enumerate(seqs):
        n_pages = -(-(q_len + ctx) // P)
        pages = [order.pop() for _ in range(n_pages)]
        tables[s, :n_pages] = torch.tensor(pages, dtype=torch.int32)
        kv_len = q_len + ctx
        if spike is not None and s == spike[0]:
            # One far key stands out for one query: scale them so that their score dominates.
            _, qi, key_index = spike
            page, off = pages[key_index // P], key_index % P
            direction = torch.randn(D, generator=gen)
            direction = direction / direction.norm()
            k_cache[page, off, :, :] = (direction * 12).to(dtype)
            q_view = qkv[row + qi, : H * D].view(H, D)
            q_view[:] = (direction * 12).to(dtype)
        slots = [pages[i // P] * P + i % P for i in range(kv_len)]
        if ramp is not None:
            # Every query looks along one direction and the keys' share of it grows with the
            # position, so the running maximum of a row keeps growing along the key tiles.
            direction = torch.ones(D) / math.sqrt(D)
            qkv[row : row + q_len, : H * D] = (direction * 8).repeat(H).to(dtype)
            for i, slot in enumerate(slots):
                k_cache.view(-1, G, D)[slot] = (direction * ramp * i * math.sqrt(D) / 8
                                                + 0.1 * torch.randn(G, D, generator=gen)).to(dtype)
        k_all = k_cache.view(-1, G, D)[slots].double()
        v_all = v_cache.view(-1, G, D)[slots].double()
        q = qkv[row : row + q_len, : H * D].view(q_len, H, D).double()
        want[row : row + q_len] = plain_paged_attention(q, k_all, v_all, ctx, 1 / math.sqrt(D), window)
        q_start.append(row)
        q_lens.append(q_len)
        kv_lens.append(kv_len)
        row += q_len

    plan = ap.plan_attention(
        q_lens, kv_lens,
        ap.PlanOptions(num_kv_heads=G, group=group, window=window, use_f32=dtype == torch.float32,
                       min_split_keys=min_split_keys, tc_min_split_keys=min_split_keys, tc_merge_us=tc_merge_us,
                       target_ctas=target_ctas,
                       narrow_max_cluster=max_cluster, max_splits=max_splits,
                       narrow_global_split_keys=min_split_keys, wide_on_tensor_memory=tensor_memory),
    )
    dev = lambda x: torch.as_tensor(x, dtype=torch.int32).cuda()
    out = torch.zeros(T, H * D, dtype=dtype, device="cuda")
    partial_o = torch.zeros(max(plan.partial_rows, 1) * D, device="cuda")
    partial_lse = torch.zeros(max(plan.partial_rows, 1), device="cuda")
    args = (qkv.cuda(), out, k_cache.cuda(), v_cache.cuda(), tables.cuda(), dev(q_start), dev(q_lens), dev(kv_lens))
    fused = fused_merge and dtype != torch.float32 and len(plan.merge_items) > 0
    counters = torch.zeros(max(1, len(plan.merge_items) * G), dtype=torch.int32, device="cuda") if fused else None
    merge_dev = dev(plan.merge_items) if fused else None
    for kind, items in plan.items.items():
        k.attention(kind, *args, dev(items), len(items), partial_o, partial_lse, H, G, D, window, 1 / math.sqrt(D),
                    merge_items=merge_dev, split_counters=counters,
                    cluster=(plan.cluster if kind == ap.KIND_BF16_NARROW else
                             tc_ctas_per_sm if kind == ap.KIND_BF16_TC else 1))
    if fused:
        torch.cuda.synchronize()
        assert int(counters.abs().sum()) == 0  # the last split of every item put its counter back
    elif len(plan.merge_items):
        k.attention_merge(out, dev(q_start), dev(plan.merge_items), len(plan.merge_items), partial_o,
                          partial_lse, H, G, D, max_rows=64)
    torch.cuda.synchronize()
    return out.view(T, H, D).double().cpu(), want, plan


ATTN_SHAPES = [
    # H, G, D, P
    (4, 2, 16, 4),
    (8, 1, 32, 8),
    (5, 5, 48, 16),
    (6, 2, 80, 16),
    (12, 2, 128, 16),
    (3, 3, 256, 32),
    (32, 1, 64, 16),  # 32 query heads on one KV head: a group wider than a 16-row tile
]


def _attn_tol(dtype):
    # bfloat16: p is rounded to bf16 before the PV product and the output once more.
    return 2e-5 if dtype == torch.float32 else 2.5e-2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,P", ATTN_SHAPES)
def test_attention_mixed_batch(k, dtype, H, G, D, P):
    # whole prompts, portions with context, single decoded tokens, a first token, a 2-token portion
    seqs = [(70, 0), (1, 0), (1, 130), (2, 61), (33, 100), (1, 63), (1, 64), (17, 15)]
    got, want, _ = run_attention_case(k, dtype, H, G, D, P, seqs, seed=D + H)
    err = (got - want).abs().max().item()
    assert err <= _attn_tol(dtype) * want.abs().max().item(), err


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,P", [(4, 2, 16, 4), (12, 2, 128, 16), (5, 5, 48, 8)])
@pytest.mark.parametrize("window", [1, 24, 100])
def test_attention_window(k, dtype, H, G, D, P, window):
    seqs = [(90, 0), (1, 200), (5, 57), (1, 23), (1, 24), (40, 70)]
    got, want, _ = run_attention_case(k, dtype, H, G, D, P, seqs, window=window, seed=window)
    err = (got - want).abs().max().item()
    assert err <= _attn_tol(dtype) * want.abs().max().item(), err


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,P", [(4, 2, 16, 4), (12, 2, 128, 16), (6, 2, 80, 16)])
@pytest.mark.parametrize("fused_merge", [True, False])
def test_attention_split_key_ranges(k, dtype, H, G, D, P, fused_merge):
    # Long contexts with few rows: the key range is cut into many splits and merged, by the
    # last split to finish (bfloat16) or by the merge kernel.
    seqs = [(1, 1500), (1, 700), (2, 1023), (3, 64), (70, 900)]
    got, want, plan = run_attention_case(k, dtype, H, G, D, P, seqs, seed=5, min_split_keys=64,
                                         target_ctas=10_000, fused_merge=fused_merge)
    assert len(plan.merge_items) > 0 and plan.partial_rows > 0
    err = (got - want).abs().max().item()
    assert err <= _attn_tol(dtype) * want.abs().max().item(), err


@pytest.mark.parametrize("H,G,D,P", [(4, 2, 16, 4), (12, 2, 128, 16), (6, 2, 80, 16), (5, 5, 48, 8),
                                     (3, 3, 256, 32), (32, 1, 64, 16)])
@pytest.mark.parametrize("max_cluster,max_splits", [(2, 1), (4, 1), (8, 1), (8, 64), (2, 64)])
def test_attention_cluster_shares_an_item(k, H, G, D, P, max_cluster, max_splits):
    # The CTAs of a thread-block cluster take runs of an item's key tiles and merge through
    # distributed shared memory; where more splits are allowed the ranges are split through
    # memory as well.  Short ranges leave some CTAs of a cluster without keys; a window cuts
    # others.
    seqs = [(1, 1500), (1, 700), (2, 1023), (1, 0), (1, 63), (3, 64), (1, 129), (70, 900)]
    for window in (None, 300):
        got, want, plan = run_attention_case(k, torch.bfloat16, H, G, D, P, seqs, window=window, seed=7,
                                             min_split_keys=32, target_ctas=10_000,
                                             max_cluster=max_cluster, max_splits=max_splits)
        assert plan.cluster == max_cluster
        assert (len(plan.merge_items) == 0) == (max_splits == 1)
        err = (got - want).abs().max().item()
        assert err <= _attn_tol(torch.bfloat16) * want.abs().max().item(), (window, err)


# One CTA per SM with P in shared memory over the K tile, or two with P in tensor memory.
TC_FORMS = pytest.mark.parametrize("per_sm", [1, 2], ids=["p_in_shared_memory", "p_in_tensor_memory"])


@TC_FORMS
@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("H,G", [(12, 2), (4, 4), (7, 1)])
@pytest.mark.parametrize("window", [None, 100])
def test_attention_on_tensor_memory(k, H, G, window, per_sm, D):
    """Prompt portions of head sizes 128 and 64 on tcgen05 tensor cores with S and O in tensor
    memory: whole prompts, portions with context, a last tile with few rows, page order shuffled."""
    seqs = [(300, 0), (70, 130), (129, 1000), (200, 57), (1, 40), (64, 64)]
    got, want, plan = run_attention_case(k, torch.bfloat16, H, G, D, 16, seqs, window=window, seed=H + G,
                                         tensor_memory=True, tc_ctas_per_sm=per_sm)
    from velox_b200.ops import attention_plan as ap

    assert ap.KIND_BF16_TC in plan.items
    err = (got - want).abs().max().item()
    assert err <= _attn_tol(torch.bfloat16) * want.abs().max().item(), err


@TC_FORMS
@pytest.mark.parametrize("D", [128, 64])
def test_attention_on_tensor_memory_rescales_when_the_maximum_grows(k, per_sm, D):
    """Scores that grow along the keys by far more than 2^8: the reference maximum of the
    exponentials moves several times and O in tensor memory is rescaled each time."""
    H, G, P = 6, 2, 64
    seqs = [(128, 400)]
    got, want, plan = run_attention_case(k, torch.bfloat16, H, G, D, P, seqs, seed=3, tensor_memory=True,
                                         ramp=0.05, tc_ctas_per_sm=per_sm)
    err = (got - want).abs().max().item()
    assert err <= _attn_tol(torch.bfloat16) * want.abs().max().item(), err


@TC_FORMS
@pytest.mark.parametrize("D", [128, 64])
def test_attention_on_tensor_memory_split_key_ranges(k, per_sm, D):
    seqs = [(100, 1500), (130, 700)]
    got, want, plan = run_attention_case(k, torch.bfloat16, 12, 2, D, 16, seqs, seed=9, min_split_keys=64,
                                         target_ctas=10_000, tensor_memory=True, tc_ctas_per_sm=per_sm,
                                         tc_merge_us=0.0)
    assert len(plan.merge_items) > 0
    err = (got - want).abs().max().item()
    assert err <= _attn_tol(torch.bfloat16) * want.abs().max().item(), err


@TC_FORMS
@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("key_index", [0, 63, 64, 1000, 1940])
def test_attention_on_tensor_memory_finds_one_far_key(k, key_index, per_sm, D):
    """One key among 1,950 carries the output of a row of a 200-token portion: its tile's
    probabilities must reach the second product with the right weight, whichever buffer and
    stage they pass through."""
    seqs = [(64, 300), (200, 1800), (130, 40)]
    got, want, plan = run_attention_case(k, torch.bfloat16, 12, 2, D, 16, seqs, seed=key_index,
                                         spike=(1, 150, key_index), tensor_memory=True, tc_ctas_per_sm=per_sm)
    from velox_b200.ops import attention_plan as ap

    assert ap.KIND_BF16_TC in plan.items
    err = (got - want).abs().max().item()
    assert err <= _attn_tol(torch.bfloat16) * want.abs().max().item(), err


@pytest.mark.parametrize("key_index", [0, 63, 64, 500, 1499])
def test_attention_cluster_finds_one_far_key(k, key_index):
    """One key among 1,500 carries the output: whichever CTA of the cluster owns its tile, its
    share must reach the row's owner with the right weight."""
    seqs = [(1, 300), (1, 1500), (1, 40)]
    got, want, plan = run_attention_case(k, torch.bfloat16, 12, 2, 128, 16, seqs, seed=key_index,
                                         spike=(1, 0, key_index), min_split_keys=64, target_ctas=96,
                                         max_cluster=8)
    assert plan.cluster == 8
    err = (got - want).abs().max().item()
    assert err <= _attn_tol(torch.bfloat16) * want.abs().max().item(), err


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key_index", [0, 15, 16, 511, 777])
def test_attention_finds_one_far_key(k, dtype, key_index):
    """One key among a thousand has a score far above the rest: the output must be its value.
    Random keys alone would hide a wrong page or a skipped tile."""
    H, G, D, P = 12, 2, 128, 16
    seqs = [(1, 999), (4, 996)]
    for spike_seq, qi in ((0, 0), (1, 2)):
        got, want, _ = run_attention_case(k, dtype, H, G, D, P, seqs, seed=key_index,
                                          spike=(spike_seq, qi, key_index), min_split_keys=64,
                                          target_ctas=2000)
        err = (got - want).abs().max().item()
        assert err <= _attn_tol(dtype) * want.abs().max().item(), (spike_seq, err)
        # The spiked query really is dominated by that one key.
        row = sum(q for q, _ in seqs[:spike_seq]) + qi
        assert (got[row] - want[row]).abs().max().item() <= _attn_tol(dtype) * want.abs().max().item()


def test_attention_f32_unsplit_rows_do_not_depend_on_portions(k):
    """A row's float32 result is bitwise the same whether its token came in a whole prompt, in
    a portion with context, or alone, as long as its key range is not split."""
    H, G, D, P = 4, 2, 16, 4
    from velox_b200.ops import attention_plan as ap

    gen = torch.Generator().manual_seed(3)
    L = 75
    pages = list(range(1, 1 + -(-L // P)))
    k_cache = torch.randn(len(pages) + 1, P, G, D, generator=gen).cuda()
    v_cache = torch.randn(len(pages) + 1, P, G, D, generator=gen).cuda()
    q_all = torch.randn(L, (H + 2 * G) * D, generator=gen).cuda()
    table = torch.tensor([pages], dtype=torch.int32).cuda()

    def run(start, n):
        plan = ap.plan_attention([n], [start + n], ap.PlanOptions(G, H // G, None, True))
        out = torch.zeros(n, H * D, device="cuda")
        dev = lambda x: torch.as_tensor(x, dtype=torch.int32).cuda()
        for kind, items in plan.items.items():
            k.attention(kind, q_all[start : start + n].contiguous(), out, k_cache, v_cache, table,
                        dev([0]), dev([n]), dev([start + n]), dev(items), len(items), None, None,
                        H, G, D, None, 0.25)
        return out

    whole = run(0, L)
    assert torch.equal(run(40, 35), whole[40:])
    assert torch.equal(run(74, 1), whole[74:])
    assert torch.equal(run(33, 2), whole[33:35])


# ----------------------------------------------------------------------------------------------
# Sampling
# ----------------------------------------------------------------------------------------------
def philox4x32_10(counter, key):
    """Plain restatement of Philox4x32-10 (Salmon et al. 2011) on python ints."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    c = list(counter)
    k0, k1 = key
    for _ in range(10):
        p0 = M0 * c[0]
        p1 = M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k1) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k0 = (k0 + W0) & 0xFFFFFFFF
        k1 = (k1 + W1) & 0xFFFFFFFF
    return c


def plain_race_scores(logits_row, temperature, seed, draw):
    """scaled - log(noise), noise = max(-log(u), 1e-10), u from Philox keyed by the seed."""
    V = logits_row.shape[0]
    key = (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    u = np.empty(V, dtype=np.float32)
    for base in range(0, V, 4):
        bits = philox4x32_10((base >> 2, draw, 0, 0), key)
        for j in range(4):
            if base + j < V:
                u[base + j] = (np.float32(bits[j] >> 8) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    noise = np.maximum(-np.log(u.astype(np.float64)), 1e-10)
    scaled = logits_row.astype(np.float64) / max(temperature, 1e-5)
    return scaled - np.log(noise), scaled


def test_sample_greedy_first_maximum(k):
    logits = torch.randn(5, 1000).cuda()
    logits[0, 700] = 50.0
    logits[0, 30] = 50.0
    logits[1, 999] = 60.0
    logits[2] = 0.0  # all equal: index 0
    out = torch.empty(5, dtype=torch.int32, device="cuda")
    k.sample(logits, 5, None, None, None, None, out)
    assert out.tolist() == torch.argmax(logits, dim=-1).tolist()
    assert out[0] == 30 and out[1] == 999 and out[2] == 0


@pytest.mark.parametrize("vocab,rows", [(20011, 3), (151936, 8), (40960, 70)])
def test_sample_greedy_in_segments(k, vocab, rows):
    """Rows long enough to be cut into segments (20011: rows that do not start on 16 bytes): the
    first maximum wins across segments too, launch after launch (the arrival counters go back
    to zero)."""
    gen = torch.Generator().manual_seed(vocab)
    logits = torch.randn(rows, vocab, generator=gen).cuda()
    logits[0, vocab - 1] = 40.0
    logits[0, 3000] = 40.0
    logits[1, vocab - 2] = 41.0
    logits[2] = -1.0  # all equal: index 0
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    for _ in range(3):
        out.fill_(-1)
        k.sample(logits, rows, None, None, None, None, out)
        assert out.tolist() == torch.argmax(logits, dim=-1).tolist()
    assert out[0] == 3000 and out[1] == vocab - 2 and out[2] == 0


@pytest.mark.parametrize("vocab", [331, 5000, 20011, 40960])
def test_sample_temperature_matches_plain_restatement(k, vocab):
    gen = torch.Generator().manual_seed(vocab)
    R = 6
    logits = (torch.randn(R, vocab, generator=gen) * 2).cuda()
    temps = [0.8, 0.0, 1.5, 0.3, 1.0, 0.7]
    seeds = [7, 8, (1 << 40) + 12345, 3, 99, 2**63 - 5]
    draws = [0, 5, 2, 11, 1, 400]
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    seed_t = torch.tensor(seeds, dtype=torch.int64).cuda()
    k.sample(logits, R, torch.tensor(temps).cuda(), seed_t, torch.tensor(draws, dtype=torch.int32).cuda(), None, out)
    host = logits.cpu().numpy()
    for r in range(R):
        if temps[r] == 0.0:
            assert int(out[r]) == int(np.argmax(host[r]))
            continue
        scores, _ = plain_race_scores(host[r], temps[r], seeds[r], draws[r])
        best = int(np.argmax(scores))
        ranked = np.sort(scores)
        # If the two best scores are within float32 rounding of each other either may win.
        if ranked[-1] - ranked[-2] > 1e-4:
            assert int(out[r]) == best
    # the same seed and draw index give the same token whatever the row or the neighbours
    logits2 = torch.cat([logits[3:4], logits[0:1]]).contiguous()
    out2 = torch.empty(2, dtype=torch.int32, device="cuda")
    k.sample(logits2, 2, torch.tensor([temps[3], temps[0]]).cuda(),
             torch.tensor([seeds[3], seeds[0]], dtype=torch.int64).cuda(),
             torch.tensor([draws[3], draws[0]], dtype=torch.int32).cuda(), None, out2)
    assert out2.tolist() == [int(out[3]), int(out[0])]


def test_sample_distribution(k):
    """Many draws from a small distribution follow softmax(logits / T)."""
    vocab, n = 7, 4000
    base = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5, 1.5, -3.0])
    logits = base.repeat(n, 1).cuda()
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    temps = torch.full((n,), 0.9).cuda()
    seeds = torch.full((n,), 1234, dtype=torch.int64).cuda()
    draws = torch.arange(n, dtype=torch.int32).cuda()
    # the sampler handles at most blockDim rows per launch? no: rows are blocks; any count works
    k.sample(logits, n, temps, seeds, draws, None, out)
    freq = torch.bincount(out.long().cpu(), minlength=vocab).double() / n
    want = torch.softmax(base.double() / 0.9, -1)
    assert (freq - want).abs().max().item() < 4 * math.sqrt(0.25 / n)


def plain_candidates(scaled, top_k, top_p):
    """The reference's candidate set (engine/sampler.py:216-228): ranks < k and exclusive
    cumulative probability < top_p, on values sorted in descending order."""
    probs = torch.softmax(scaled, -1)
    order = torch.argsort(scaled, descending=True, stable=True)
    sorted_probs = probs[order]
    keep = torch.ones_like(sorted_probs, dtype=torch.bool)
    if top_k > 0:
        keep &= torch.arange(len(order)) < top_k
    keep &= (sorted_probs.cumsum(0) - sorted_probs) < top_p
    return set(order[keep].tolist())


@pytest.mark.parametrize("kind", [1, 2], ids=["one_cta", "cluster"])
@pytest.mark.parametrize("vocab", [3001, 50021])
@pytest.mark.parametrize("top_k,top_p", [(5, 1.0), (0, 0.6), (40, 0.9), (1, 1.0), (0, 0.05), (700, 0.999)])
def test_filter_threshold(k, top_k, top_p, vocab, kind):
    gen = torch.Generator().manual_seed(top_k + int(top_p * 100))
    R = 4
    logits = (torch.randn(R, vocab, generator=gen) * 3).cuda()
    temps = torch.tensor([0.7, 1.0, 1.3, 0.0]).cuda()
    thr = torch.empty(R, device="cuda")
    k.filter_threshold(logits, R, temps, torch.full((R,), top_k, dtype=torch.int32).cuda(),
                       torch.full((R,), top_p).cuda(), thr, kind=kind)
    for r in range(3):
        scaled = logits[r].double().cpu() / float(temps[r])
        want = plain_candidates(scaled, top_k, top_p)
        got = set(torch.nonzero(logits[r].cpu() * (1.0 / max(float(temps[r]), 1e-5)) >= thr[r].cpu()).flatten().tolist())
        # The boundary candidate may differ where cumulative masses agree to rounding.
        assert len(got ^ want) <= 1, (len(got), len(want))
        assert max(scaled.argmax().item(), 0) in got
    assert thr[3].item() == float("-inf")


@pytest.mark.parametrize("vocab", [7, 1000, 8191, 151936, 196608])
def test_filter_threshold_kernels_agree(k, vocab):
    """One CTA a row and the cluster of eight add up the same integers: equal thresholds, bit
    for bit, with rows off a 16-byte boundary, mixed options per row, NaN and -inf entries
    and a row whose mass sits in one entry."""
    gen = torch.Generator().manual_seed(vocab)
    R = 9
    # With an odd row length most rows start off a 16-byte boundary.
    store = torch.randn(R, vocab, generator=gen) * torch.tensor([0.1, 0.5, 1, 2, 4, 8, 1, 1, 1]).unsqueeze(1)
    store[6, : vocab // 2] = float("-inf")
    store[7, ::5] = float("nan")
    store[8, vocab // 3] = 60.0
    logits = store.cuda()
    temps = torch.tensor([0.7, 1.0, 1.3, 0.0, 0.3, 2.0, 1.0, 1.0, 1.0]).cuda()
    top_k = torch.tensor([0, 50, 3, 5, 0, vocab + 5, 0, 20, 0], dtype=torch.int32).cuda()
    top_p = torch.tensor([0.9, 1.0, 0.5, 0.9, 0.999, 0.95, 0.8, 0.7, 0.9]).cuda()
    one, cluster, auto = (torch.full((R,), 7.0, device="cuda") for _ in range(3))
    k.filter_threshold(logits, R, temps, top_k, top_p, one, kind=1)
    k.filter_threshold(logits, R, temps, top_k, top_p, cluster, kind=2)
    k.filter_threshold(logits, R, temps, top_k, top_p, auto, kind=0)
    assert torch.equal(one.view(torch.int32), cluster.view(torch.int32)), (one.tolist(), cluster.tolist())
    assert torch.equal(one.view(torch.int32), auto.view(torch.int32))
    assert one[3].item() == float("-inf")
    # The entry that holds the row's mass is the only candidate of the last row.
    assert int((logits[8] >= one[8]).sum()) == 1


def test_filter_threshold_beyond_the_cluster_kernel(k):
    """A row longer than the cluster's registers hold takes the one-CTA kernel; asking for the
    cluster kernel by name is refused."""
    vocab, R = 196608 + 40, 2
    gen = torch.Generator().manual_seed(3)
    logits = (torch.randn(R, vocab, generator=gen) * 2).cuda()
    temps = torch.ones(R).cuda()
    top_k = torch.tensor([10, 0], dtype=torch.int32).cuda()
    top_p = torch.tensor([1.0, 0.5]).cuda()
    thr = torch.empty(R, device="cuda")
    k.filter_threshold(logits, R, temps, top_k, top_p, thr)
    assert int((logits[0] >= thr[0]).sum()) == 10
    want = plain_candidates(logits[1].double().cpu(), 0, 0.5)
    got = set(torch.nonzero(logits[1] >= thr[1]).flatten().tolist())
    assert len(got ^ want) <= 1
    with pytest.raises(RuntimeError):
        k.filter_threshold(logits, R, temps, top_k, top_p, thr, kind=2)


def test_penalties(k):
    gen = torch.Generator().manual_seed(9)
    R, vocab, width = 3, 500, 64
    logits = (torch.randn(R, vocab, generator=gen) * 2).cuda()
    original = logits.clone().cpu().double()
    history = torch.randint(0, vocab, (5, width), generator=gen, dtype=torch.int32)
    history[2, :10] = 7  # a token seen ten times
    slots = torch.tensor([2, 0, 4], dtype=torch.int32)
    lengths = torch.tensor([20, 0, 64], dtype=torch.int32)
    rep = torch.tensor([1.3, 1.0, 0.8])
    pres = torch.tensor([0.5, 0.0, -0.2])
    freq = torch.tensor([0.1, 0.0, 0.3])
    counts = torch.zeros(R, vocab, dtype=torch.int32, device="cuda")
    k.apply_penalties(logits, R, history.cuda(), slots.cuda(), lengths.cuda(), counts,
                      rep.cuda(), pres.cuda(), freq.cuda())
    for r in range(R):
        want = original[r].clone()
        seen = history[slots[r], : lengths[r]].long()
        count = torch.bincount(seen, minlength=vocab).double()
        x = want - freq[r].double() * count
        x = torch.where(x > 0, x / rep[r].double(), x * rep[r].double()) - pres[r].double()
        want = torch.where(count > 0, x, want)
        assert (logits[r].cpu().double() - want).abs().max().item() < 1e-5


# ----------------------------------------------------------------------------------------------
# bf16 GEMM on tcgen05 tensor cores
# ----------------------------------------------------------------------------------------------
GEMM_SHAPES = [
    # T, N, K
    (1, 128, 64), (8, 256, 128), (16, 2048, 1536), (5, 331, 240), (33, 704, 256), (64, 1536, 8960),
    (100, 136, 480), (300, 640, 200), (2, 97, 48), (7, 1000, 72),
]


@pytest.mark.parametrize("T,N,K", GEMM_SHAPES)
def test_gemm_bf16_plain_and_bias(k, status, T, N, K):
    gen = torch.Generator().manual_seed(T * N + K)
    x = torch.randn(T + 5, K, generator=gen).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=gen) / math.sqrt(K)).to(torch.bfloat16).cuda()
    bias = torch.randn(N, generator=gen).cuda()
    want = x[:T].double() @ w.double().T
    out = torch.full((T + 5, N), 9.0, dtype=torch.bfloat16, device="cuda")
    k.gemm_bf16(x, w, None, out, k.GEMM_OUT_BF16, T, status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    scale = want.abs().max().item()
    assert (out[:T].double().cpu() - want.cpu()).abs().max().item() <= 1e-2 * scale
    assert torch.all(out[T:] == 9.0)
    outf = torch.full((T + 5, N), 9.0, dtype=torch.float32, device="cuda")
    k.gemm_bf16(x, w, bias, outf, k.GEMM_OUT_F32, T, status)
    want_b = want + bias.double()
    # float32 accumulation of bf16 products: error ~ sqrt(K) * 2^-24 relative to the terms
    assert (outf[:T].double().cpu() - want_b.cpu()).abs().max().item() <= 2e-5 * max(scale, 1.0)
    assert torch.all(outf[T:] == 9.0)
    assert int(status[0]) == 0


@pytest.mark.parametrize("T,N,K,splits", [(8, 1536, 8960, 8), (3, 256, 704, 4), (64, 2048, 1536, 8),
                                          (17, 136, 480, 100), (1, 1536, 1536, 2), (40, 331, 240, 3),
                                          (8, 1536, 8960, 16), (13, 200, 4104, 5)])
@pytest.mark.parametrize("mode", ["bf16", "f32", "add"])
def test_gemm_bf16_split_over_a_cluster(k, status, T, N, K, splits, mode):
    """K split over a thread-block cluster, reduced through distributed shared memory."""
    gen = torch.Generator().manual_seed(K + splits)
    x = torch.randn(T, K, generator=gen).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=gen) / math.sqrt(K)).to(torch.bfloat16).cuda()
    bias = torch.randn(N, generator=gen).cuda()
    want = x.double() @ w.double().T + bias.double()
    scale = max(want.abs().max().item(), 1.0)
    if mode == "bf16":
        out = torch.zeros(T, N, dtype=torch.bfloat16, device="cuda")
        k.gemm_bf16(x, w, bias, out, k.GEMM_OUT_BF16, T, status, splits=splits)
        tol = 1e-2
    elif mode == "f32":
        out = torch.zeros(T, N, dtype=torch.float32, device="cuda")
        k.gemm_bf16(x, w, bias, out, k.GEMM_OUT_F32, T, status, splits=splits)
        tol = 2e-5
    else:
        start = torch.randn(T, N, generator=gen).cuda()
        out = start.clone()
        k.gemm_bf16(x, w, bias, out, k.GEMM_ADD_F32, T, status, splits=splits)
        want = want + start.double()
        tol = 2e-5
    assert (out.double().cpu() - want.cpu()).abs().max().item() <= tol * scale
    assert int(status[0]) == 0
    # the same call twice gives the same bits: the order of the sums is fixed
    if mode == "f32":
        again = torch.zeros_like(out)
        k.gemm_bf16(x, w, bias, again, k.GEMM_OUT_F32, T, status, splits=splits)
        assert torch.equal(out, again)


@pytest.mark.parametrize("T,N,K", [(4, 1536, 1536), (70, 240, 200), (256, 1536, 8960)])
def test_gemm_bf16_adds_into_residual(k, status, T, N, K):
    gen = torch.Generator().manual_seed(N)
    x = torch.randn(T, K, generator=gen).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=gen) / math.sqrt(K)).to(torch.bfloat16).cuda()
    resid = torch.randn(T, N, generator=gen).cuda()
    want = resid.double() + x.double() @ w.double().T
    k.gemm_bf16(x, w, None, resid, k.GEMM_ADD_F32, T, status)
    assert (resid.double().cpu() - want.cpu()).abs().max().item() <= 2e-5 * want.abs().max().item()
    assert int(status[0]) == 0


@pytest.mark.parametrize("T,I,K", [(8, 8960, 1536), (40, 704, 256), (3, 200, 240), (130, 312, 136)])
def test_gemm_bf16_swiglu(k, status, T, I, K):
    gen = torch.Generator().manual_seed(I)
    x = torch.randn(T, K, generator=gen).to(torch.bfloat16).cuda()
    w = (torch.randn(2 * I, K, generator=gen) * 2 / math.sqrt(K)).to(torch.bfloat16).cuda()
    out = torch.zeros(T, I, dtype=torch.bfloat16, device="cuda")
    k.gemm_bf16(x, w, None, out, k.GEMM_SWIGLU, T, status)
    gu = x.double() @ w.double().T
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    assert (out.double().cpu() - want.cpu()).abs().max().item() <= 1e-2 * want.abs().max().item()
    assert int(status[0]) == 0


@pytest.mark.parametrize("T,N,K,splits", [(8, 2048, 1536, 8), (1, 256, 704, 4), (64, 1536, 1536, 8),
                                          (17, 136, 480, 1), (33, 331, 240, 2), (16, 384, 200, 1),
                                          (5, 256, 4608, 16)])
@pytest.mark.parametrize("mode", ["bf16", "f32"])
def test_gemm_bf16_makes_its_input_norm(k, status, T, N, K, splits, mode):
    """The projection of rmsnorm(resid) * w_norm with the norm made inside the kernel: the X
    tiles come from the float32 rows, 1 / rms is applied to the accumulator, and with split K
    the sums of squares are added up across the cluster."""
    gen = torch.Generator().manual_seed(N + K + T)
    rows = T + 3
    resid = (torch.randn(rows, K + 4, generator=gen) * 3).cuda()[:, :K]  # a row pitch that is not K
    resid[:, 5] *= 20  # one dimension dominates the mean square, as in real residual streams
    w_norm = (torch.rand(K, generator=gen) + 0.5).cuda()
    eps = 1e-6
    w = (torch.randn(N, K, generator=gen) / math.sqrt(K)).to(torch.bfloat16).cuda()
    bias = torch.randn(N, generator=gen).cuda()
    r64 = resid[:T].double()
    normed = r64 * torch.rsqrt((r64 * r64).mean(-1, keepdim=True) + eps) * w_norm.double()
    want = normed @ w.double().T + bias.double()
    scale = max(want.abs().max().item(), 1.0)
    if mode == "bf16":
        out = torch.full((rows, N), 9.0, dtype=torch.bfloat16, device="cuda")
        k.gemm_bf16_normed(resid, w_norm, eps, w, bias, out, k.GEMM_OUT_BF16, T, status, splits=splits)
    else:
        out = torch.full((rows, N), 9.0, dtype=torch.float32, device="cuda")
        k.gemm_bf16_normed(resid, w_norm, eps, w, bias, out, k.GEMM_OUT_F32, T, status, splits=splits)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    # The inputs are rounded to bfloat16 once (2^-9 relative each), as the norm kernel's output is.
    assert (out[:T].double().cpu() - want.cpu()).abs().max().item() <= 1e-2 * scale
    assert torch.all(out[T:] == 9.0)
    # It agrees with the two-kernel route to within the rounding of the normalised input.
    x = torch.zeros(rows, K, dtype=torch.bfloat16, device="cuda")
    k.add_rmsnorm(resid.contiguous(), None, w_norm, eps, x, T, None, False)
    two = torch.zeros_like(out)
    k.gemm_bf16(x, w, bias, two, k.GEMM_OUT_BF16 if mode == "bf16" else k.GEMM_OUT_F32, T, status, splits=splits)
    assert (out[:T].double() - two[:T].double()).abs().max().item() <= 1e-2 * scale


@pytest.mark.parametrize("T,E,I", [(8, 1536, 8960), (16, 256, 704), (1, 128, 64), (5, 640, 1344), (13, 3584, 1024),
                                   (32, 1536, 8960), (17, 256, 704), (25, 1792, 320)])
def test_mlp_fused_is_the_feed_forward(k, status, T, E, I):
    """The gated feed-forward in one kernel: norm, gate|up, SiLU * up, down and the add into the
    residual rows, against the formulas in float64 and against the separate projections."""
    gen = torch.Generator().manual_seed(E + I + T)
    rows = T + 2
    resid_in = (torch.randn(rows, E + 4, generator=gen) * 2).cuda()[:, :E]  # a row pitch that is not E
    resid_in[:, 3] *= 15
    w_norm = (torch.rand(E, generator=gen) + 0.5).cuda()
    eps = 1e-6
    w_gu = (torch.randn(2 * I, E, generator=gen) * 2 / math.sqrt(E)).to(torch.bfloat16).cuda()
    w_down = (torch.randn(E, I, generator=gen) / math.sqrt(I)).to(torch.bfloat16).cuda()
    # A far column of W_down that matters: a fault in the tile coordinates of the second part shows.
    w_down[:, I - 1] *= 8
    before = torch.randn(rows, E, generator=gen).cuda()
    resid_out = before.clone()
    assert k.mlp_fused(resid_in, w_norm, eps, w_gu, w_down, resid_out, T, status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    r64 = resid_in[:T].double()
    normed = (r64 * torch.rsqrt((r64 * r64).mean(-1, keepdim=True) + eps) * w_norm.double()).to(torch.bfloat16).double()
    gu = normed @ w_gu.double().T
    act = (torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]).to(torch.bfloat16).double()
    want = act @ w_down.double().T
    got = (resid_out[:T] - before[:T]).double()
    scale = max(want.abs().max().item(), 1.0)
    assert (got.cpu() - want.cpu()).abs().max().item() <= 1e-2 * scale
    assert torch.equal(resid_out[T:], before[T:])
    # The separate kernels of the same step agree to the rounding of the activations.
    act2 = torch.zeros(rows, I, dtype=torch.bfloat16, device="cuda")
    assert k.gemm_bf16_normed(resid_in, w_norm, eps, w_gu, None, act2, k.GEMM_SWIGLU, T, status)
    two = before.clone()
    k.gemm_bf16(act2, w_down, None, two, k.GEMM_ADD_F32, T, status, splits=4)
    assert (resid_out[:T].double() - two[:T].double()).abs().max().item() <= 1e-2 * scale


@pytest.mark.parametrize("T,N,K,splits", [(8, 1536, 1536, 8), (16, 256, 704, 4), (3, 136, 480, 2), (40, 384, 512, 8)])
def test_gemm_bf16_add_mirrored(k, status, T, N, K, splits):
    """out += x w^T with the sums written to a second buffer as well."""
    gen = torch.Generator().manual_seed(N + K)
    rows = T + 1
    x = torch.randn(rows, K, generator=gen).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=gen) / math.sqrt(K)).to(torch.bfloat16).cuda()
    before = torch.randn(rows, N, generator=gen).cuda()
    out = before.clone()
    mirror = torch.full((rows, N + 4), 7.0, device="cuda")[:, :N]  # a row pitch of its own
    assert k.gemm_bf16_add_mirrored(x, w, out, mirror, T, status, splits)
    want = before[:T].double() + x[:T].double() @ w.double().T
    assert (out[:T].double() - want).abs().max().item() <= 2e-5 * max(want.abs().max().item(), 1.0)
    assert torch.equal(mirror[:T], out[:T])
    assert torch.equal(out[T:], before[T:]) and torch.all(mirror[T:] == 7.0)
    # the plain accumulate gives the same sums
    plain = before.clone()
    k.gemm_bf16(x, w, None, plain, k.GEMM_ADD_F32, T, status, splits=splits)
    assert torch.equal(plain[:T], out[:T])
    assert int(status[0]) == 0
    # no split along K: refused, nothing written
    assert not k.gemm_bf16_add_mirrored(x, w, out, mirror, T, status, 1)


def test_mlp_fused_refuses_what_it_cannot_do(k, status):
    E, I = 256, 128
    resid = torch.zeros(40, E, device="cuda")
    out = torch.zeros(40, E, device="cuda")
    w_norm = torch.ones(E, device="cuda")
    w_gu = torch.zeros(2 * I, E, dtype=torch.bfloat16, device="cuda")
    w_down = torch.zeros(E, I, dtype=torch.bfloat16, device="cuda")
    assert not k.mlp_fused(resid, w_norm, 1e-6, w_gu, w_down, out, 33, status)  # too many rows
    with pytest.raises(ValueError):
        k.mlp_fused(resid, w_norm, 1e-6, w_gu, w_down, resid, 4, status)  # in place
    odd = torch.zeros(2 * 96, E, dtype=torch.bfloat16, device="cuda")
    assert not k.mlp_fused(resid, w_norm, 1e-6, odd, torch.zeros(E, 96, dtype=torch.bfloat16, device="cuda"), out, 4, status)


@pytest.mark.parametrize("T,I,K", [(8, 8960, 1536), (40, 704, 256), (3, 200, 240)])
def test_gemm_bf16_swiglu_makes_its_input_norm(k, status, T, I, K):
    gen = torch.Generator().manual_seed(I + T)
    resid = (torch.randn(T, K, generator=gen) * 2).cuda()
    w_norm = (torch.rand(K, generator=gen) + 0.5).cuda()
    eps = 1e-5
    w = (torch.randn(2 * I, K, generator=gen) * 2 / math.sqrt(K)).to(torch.bfloat16).cuda()
    out = torch.zeros(T, I, dtype=torch.bfloat16, device="cuda")
    k.gemm_bf16_normed(resid, w_norm, eps, w, None, out, k.GEMM_SWIGLU, T, status)
    r64 = resid.double()
    normed = r64 * torch.rsqrt((r64 * r64).mean(-1, keepdim=True) + eps) * w_norm.double()
    gu = normed @ w.double().T
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    assert (out.double().cpu() - want.cpu()).abs().max().item() <= 1e-2 * want.abs().max().item()
    assert int(status[0]) == 0


@pytest.mark.parametrize("T,H,G,K", [(8, 12, 2, 1536), (1, 2, 1, 256), (37, 3, 3, 704), (64, 4, 2, 512)])
@pytest.mark.parametrize("normed", [False, True])
def test_gemm_bf16_qkv_rotates_and_writes_the_cache(k, status, T, H, G, K, normed):
    """Heads of 128 dims: the QKV projection rotates q and k by the tokens' positions and writes
    k and v into the paged cache in its epilogue (and makes its input norm, if asked)."""
    D, P = 128, 16
    gen = torch.Generator().manual_seed(T + H + K)
    N = (H + 2 * G) * D
    w = (torch.randn(N, K, generator=gen) / math.sqrt(K)).to(torch.bfloat16).cuda()
    bias = torch.randn(N, generator=gen).cuda()
    max_pos = 300
    positions = torch.randint(0, max_pos, (T,), generator=gen, dtype=torch.int32)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    angles = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv_freq)
    cos, sin = angles.cos().cuda(), angles.sin().cuda()
    pages = 6
    slots = torch.randperm(pages * P, generator=gen)[:T].to(torch.int32)
    if T > 2:
        slots[1] = -1  # a row without a cache slot (padding)
    k_cache = torch.full((pages, P, G, D), 7.0, dtype=torch.bfloat16, device="cuda")
    v_cache = torch.full((pages, P, G, D), 7.0, dtype=torch.bfloat16, device="cuda")
    out = torch.full((T + 2, N), 9.0, dtype=torch.bfloat16, device="cuda")
    if normed:
        resid = (torch.randn(T + 2, K, generator=gen) * 2).cuda()
        w_norm = (torch.rand(K, generator=gen) + 0.5).cuda()
        r64 = resid[:T].double()
        x64 = r64 * torch.rsqrt((r64 * r64).mean(-1, keepdim=True) + 1e-6) * w_norm.double()
        ok = k.gemm_bf16_qkv_rope(None, resid, w_norm, 1e-6, w, bias, out, T, positions.cuda(), cos, sin,
                                  slots.cuda(), k_cache, v_cache, H, G, status, splits=8)
    else:
        x = torch.randn(T + 2, K, generator=gen).to(torch.bfloat16).cuda()
        x64 = x[:T].double()
        ok = k.gemm_bf16_qkv_rope(x, None, None, 0.0, w, bias, out, T, positions.cuda(), cos, sin,
                                  slots.cuda(), k_cache, v_cache, H, G, status, splits=8)
    assert ok
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    y = (x64 @ w.double().T + bias.double()).cpu().view(T, H + 2 * G, D)
    c64, s64 = angles.cos().double()[positions.long()], angles.sin().double()[positions.long()]  # [T, 64]
    lo, hi = y[..., :64], y[..., 64:]
    rot = torch.cat([lo * c64[:, None] - hi * s64[:, None], lo * s64[:, None] + hi * c64[:, None]], dim=-1)
    want_q, want_k, want_v = rot[:, :H], rot[:, H:H + G], y[:, H + G:]
    scale = max(y.abs().max().item(), 1.0)
    got_q = out[:T, : H * D].double().cpu().view(T, H, D)
    assert (got_q - want_q).abs().max().item() <= 1e-2 * scale
    assert torch.all(out[T:] == 9.0)
    kc, vc = k_cache.double().cpu().view(-1, G, D), v_cache.double().cpu().view(-1, G, D)
    written = torch.zeros(pages * P, dtype=torch.bool)
    for t in range(T):
        slot = int(slots[t])
        if slot < 0:
            continue
        written[slot] = True
        assert (kc[slot] - want_k[t]).abs().max().item() <= 1e-2 * scale
        assert (vc[slot] - want_v[t]).abs().max().item() <= 1e-2 * scale
    assert torch.all(kc[~written] == 7.0) and torch.all(vc[~written] == 7.0)


def test_bounded_wait_runs_out_and_reports(k, tmp_path):
    """A wait on a barrier that nobody arrives at: the kernel returns by itself after its limit
    (a few milliseconds here, about two seconds in the engine's kernels), the status word gets
    its bit, and the runner turns the word into an error that names the wait."""
    import time

    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    start = time.perf_counter()
    assert k.selftest_bounded_wait(status, 5_000_000) == 1  # about 3 ms of SM clock
    assert time.perf_counter() - start < 1.0
    assert int(status[0].item()) == 16
    # the context is still good: another kernel runs and gives the right answer
    x = torch.arange(8, dtype=torch.float32, device="cuda")
    assert float((x * 2).sum()) == 56.0

    from velox_b200.engine.runner import ModelRunner

    runner = ModelRunner.__new__(ModelRunner)
    runner.status = status
    with pytest.raises(RuntimeError, match="a bounded wait ran out"):
        runner.check_status()
    assert int(status[0].item()) == 0


@pytest.mark.parametrize("T,N,K,chunks", [(8, 1536, 8960, 24), (64, 5120, 1600, 3), (3, 331, 240, 2), (130, 136, 1352, 5),
                                          (200, 640, 4096, 9), (17, 384, 200, 50), (1, 128, 64, 4)])
def test_gemm_bf16_add_chunked(k, status, T, N, K, chunks):
    """out += x w^T with the inner dimension in chunks of independent CTAs that meet in the
    output by reductions at the L2: any number of chunks (more than there are K blocks is cut
    down), widths and rows that are no multiple of a tile, what was in the output kept."""
    gen = torch.Generator().manual_seed(N + K + T)
    x = torch.randn(T + 3, K, generator=gen).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=gen) / math.sqrt(K)).to(torch.bfloat16).cuda()
    start = torch.randn(T + 2, N, generator=gen).cuda()
    out = start.clone()
    k.gemm_bf16_add_chunked(x, w, out, T, status, chunks)
    want = start[:T].double() + x[:T].double() @ w.double().T
    torch.cuda.synchronize()
    assert (out[:T].double() - want).abs().max().item() <= 2e-5 * want.abs().max().item()
    assert torch.equal(out[T:], start[T:])  # rows past the step are not touched
    assert int(status[0]) == 0


@pytest.mark.parametrize("T,N,K,mode", [(16, 1792, 5120, "swiglu"), (8, 1024, 5120, "swiglu"), (3, 640, 8960, "swiglu"),
                                        (11, 384, 7168, "f32"), (16, 256, 14336, "bf16")])
def test_gemm_bf16_norm_with_a_ring_of_x_tiles(k, status, T, N, K, mode):
    """The norm made inside the projection when the X tiles of all K blocks do not fit in shared
    memory at once: their places are a ring, written again when the products that read them
    have finished."""
    gen = torch.Generator().manual_seed(N + K + T)
    resid = (torch.randn(T + 1, K, generator=gen) * 1.5).cuda()
    w_norm = (torch.rand(K, generator=gen) + 0.5).cuda()
    r64 = resid[:T].double()
    x64 = r64 * torch.rsqrt((r64 * r64).mean(-1, keepdim=True) + 1e-5) * w_norm.double()
    rows = 2 * N if mode == "swiglu" else N
    w = (torch.randn(rows, K, generator=gen) * 2 / math.sqrt(K)).to(torch.bfloat16).cuda()
    if mode == "swiglu":
        out = torch.zeros(T, N, dtype=torch.bfloat16, device="cuda")
        assert k.gemm_bf16_normed(resid, w_norm, 1e-5, w, None, out, k.GEMM_SWIGLU, T, status)
        # wider token tiles are refused (the norm then runs as a kernel of its own)
        if K >= 5120:
            wide = torch.zeros(64, N, dtype=torch.bfloat16, device="cuda")
            rows64 = torch.randn(64, K, device="cuda")
            assert not k.gemm_bf16_normed(rows64, w_norm, 1e-5, w, None, wide, k.GEMM_SWIGLU, 64, status)
        gu = x64 @ w.double().T
        want = torch.nn.functional.silu(gu[:, :N]) * gu[:, N:]
    else:
        out = torch.zeros(T, N, dtype=torch.float32 if mode == "f32" else torch.bfloat16, device="cuda")
        assert k.gemm_bf16_normed(resid, w_norm, 1e-5, w, None, out, k.GEMM_OUT_F32 if mode == "f32" else k.GEMM_OUT_BF16,
                                  T, status, splits=1)
        want = x64 @ w.double().T
    torch.cuda.synchronize()
    assert (out.double() - want).abs().max().item() <= 1.2e-2 * want.abs().max().item()
    assert int(status[0]) == 0
