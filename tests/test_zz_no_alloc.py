"""The attention entry point that allocates nothing (``vx_attention_decode_static``, declared in
``velox_b200/csrc/attention_static.h``): called through the exported C symbol and compared with
the ordinary launcher, which gets its scratch from the caller.

The file sorts last on purpose: the entry point keeps its scratch in one array inside the
library, and the test has to pass alone as well as after every other test has used the same
library.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_PARTIAL_ROWS = 8192  # VX_ATTENTION_STATIC_MAX_PARTIAL_ROWS
TOO_LARGE = -2  # VX_ATTENTION_STATIC_TOO_LARGE


def _static_entry(head_dim):
    from velox_b200.ops import kernels

    kernels._require_cuda()
    lib = kernels.attention_lib(head_dim)
    fn = lib.vx_attention_decode_static
    p, i = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [p, p, p, p, p, p, p, p, p, i, p, i, i, p, i, i, i, i, i, i, ctypes.c_longlong, i,
                   ctypes.c_float, p, ctypes.c_char_p, i]
    fn.restype = i
    return kernels, fn


def _plain(case, qkv):
    """The same attention in float64, sequence by sequence, from the cache's pages."""
    from test_kernels_gpu import plain_paged_attention

    H, G, D, P = case["H"], case["G"], case["D"], case["P"]
    k_flat = case["k_cache"].cpu().view(-1, G, D)
    v_flat = case["v_cache"].cpu().view(-1, G, D)
    tables = case["tables"].cpu()
    rows = []
    for s, kv_len in enumerate(case["kv_len"].cpu().tolist()):
        slots = [int(tables[s, i // P]) * P + i % P for i in range(kv_len)]
        q = qkv[s : s + 1, : H * D].cpu().view(1, H, D).double()
        rows.append(plain_paged_attention(q, k_flat[slots].double(), v_flat[slots].double(), kv_len - 1,
                                          1 / math.sqrt(D), None))
    return torch.cat(rows).view(len(rows), H * D)


def _decode_case(H, G, D, P, contexts, seed, split=True):
    """Single decoded tokens over contexts of the given lengths, pages in shuffled order."""
    from velox_b200.ops import attention_plan as ap

    gen = torch.Generator().manual_seed(seed)
    pages_of = [-(-(c + 1) // P) for c in contexts]
    total_pages = sum(pages_of) + 2
    order = (torch.randperm(total_pages - 1, generator=gen) + 1).tolist()
    tables = torch.zeros(len(contexts), max(pages_of), dtype=torch.int32)
    for s, n in enumerate(pages_of):
        tables[s, :n] = torch.tensor([order.pop() for _ in range(n)], dtype=torch.int32)
    kv_lens = [c + 1 for c in contexts]
    plan = ap.plan_attention(
        [1] * len(contexts), kv_lens,
        ap.PlanOptions(num_kv_heads=G, group=H // G, window=None, use_f32=False,
                       min_split_keys=64, target_ctas=10_000 if split else 1),
    )
    assert set(plan.items) == {ap.KIND_BF16_NARROW} and (len(plan.merge_items) > 0) == split
    dev = lambda x: torch.as_tensor(x, dtype=torch.int32).cuda()
    return dict(
        k_cache=torch.randn(total_pages, P, G, D, generator=gen).bfloat16().cuda(),
        v_cache=torch.randn(total_pages, P, G, D, generator=gen).bfloat16().cuda(),
        tables=tables.cuda(), q_start=dev(list(range(len(contexts)))), q_len=dev([1] * len(contexts)),
        kv_len=dev(kv_lens), items=dev(plan.items[ap.KIND_BF16_NARROW]),
        merges=dev(plan.merge_items) if split else torch.zeros(1, 8, dtype=torch.int32, device="cuda"),
        plan=plan, gen=gen, H=H, G=G, D=D, P=P, T=len(contexts),
    )


def _ordinary(kernels, case, qkv):
    """The existing launcher, with scratch from torch."""
    from velox_b200.ops import attention_plan as ap

    H, G, D = case["H"], case["G"], case["D"]
    out = torch.zeros(case["T"], H * D, dtype=torch.bfloat16, device="cuda")
    partial_o = torch.zeros(case["plan"].partial_rows * D, device="cuda")
    partial_lse = torch.zeros(case["plan"].partial_rows, device="cuda")
    counters = torch.zeros(len(case["merges"]) * G, dtype=torch.int32, device="cuda")
    kernels.attention(ap.KIND_BF16_NARROW, qkv, out, case["k_cache"], case["v_cache"], case["tables"],
                      case["q_start"], case["q_len"], case["kv_len"], case["items"], len(case["items"]),
                      partial_o, partial_lse, H, G, D, None, 1 / math.sqrt(D),
                      merge_items=case["merges"], split_counters=counters)
    torch.cuda.synchronize()
    return out


def _static(fn, case, qkv, status, partial_rows=None):
    H, G, D = case["H"], case["G"], case["D"]
    out = torch.zeros(case["T"], H * D, dtype=torch.bfloat16, device="cuda")
    message = ctypes.create_string_buffer(512)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    code = fn(ptr(qkv), ptr(out), ptr(case["k_cache"]), ptr(case["v_cache"]), ptr(case["tables"]),
              ptr(case["q_start"]), ptr(case["q_len"]), ptr(case["kv_len"]), ptr(case["items"]),
              len(case["items"]), ptr(case["merges"]), len(case["plan"].merge_items),
              case["plan"].partial_rows if partial_rows is None else partial_rows, ptr(status),
              qkv.shape[1], out.shape[1], case["tables"].shape[1], G, H // G, case["P"],
              case["k_cache"].shape[0], 0, 1 / math.sqrt(D),
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), message, len(message))
    torch.cuda.synchronize()
    taken = free_before - torch.cuda.mem_get_info()[0]
    return code, message.value.decode(), out, taken


@pytest.mark.parametrize("H,G,D,P", [(12, 2, 128, 16), (6, 3, 48, 8)])
def test_static_scratch_entry_matches_the_ordinary_launcher(H, G, D, P):
    kernels, fn = _static_entry(D)
    case = _decode_case(H, G, D, P, contexts=[1500, 63, 700, 1023, 64, 300], seed=D)
    assert 0 < case["plan"].partial_rows <= MAX_PARTIAL_ROWS
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tol = 2.5e-2  # the attention kernel tests' bfloat16 bound, relative to the largest output
    for call in range(2):  # two calls in a row share the library's scratch
        qkv = torch.randn(case["T"], (H + 2 * G) * D, generator=case["gen"]).bfloat16().cuda()
        want = _ordinary(kernels, case, qkv).double()
        code, message, got, taken = _static(fn, case, qkv, status)
        assert code == 0, message
        if call == 1:  # the first call of a process may load the kernel's module
            assert taken == 0  # nothing was taken from the device
        err = (got.double() - want).abs().max().item()
        assert err <= tol * want.abs().max().item(), (call, err)
        assert want.abs().max().item() > 0.1
        # and against the plain statement of the operation, not only another path of the engine
        plain = _plain(case, qkv)
        err = (got.double().cpu() - plain).abs().max().item()
        assert err <= tol * plain.abs().max().item(), (call, err)
    assert int(status.item()) == 0


def test_static_scratch_entry_without_split_key_ranges():
    """Contexts so short that no key range is split: no merge items, no partial rows."""
    kernels, fn = _static_entry(128)
    case = _decode_case(12, 2, 128, 16, contexts=[40, 7, 100, 63], seed=9, split=False)
    assert case["plan"].partial_rows == 0
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    qkv = torch.randn(case["T"], 16 * 128, generator=case["gen"]).bfloat16().cuda()
    code, message, got, _ = _static(fn, case, qkv, status)
    assert code == 0, message
    plain = _plain(case, qkv)
    err = (got.double().cpu() - plain).abs().max().item()
    assert err <= 2.5e-2 * plain.abs().max().item()
    assert int(status.item()) == 0


def test_static_scratch_entry_flags_rows_beyond_its_scratch():
    """A caller that under-reports its partial rows: the kernel writes nothing beyond the
    array and says so in the status word."""
    kernels, fn = _static_entry(128)
    case = _decode_case(12, 2, 128, 16, contexts=[600, 300], seed=5)
    items = case["items"].clone()
    split = items[:, 5] >= 0
    assert bool(split.any())
    items[:, 5] = torch.where(split, items[:, 5] + MAX_PARTIAL_ROWS, items[:, 5])  # every partial row lies beyond
    case = dict(case, items=items)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    qkv = torch.randn(case["T"], 16 * 128, generator=case["gen"]).bfloat16().cuda()
    code, message, _, _ = _static(fn, case, qkv, status)
    assert code == 0, message
    assert int(status.item()) & 32


def test_static_scratch_entry_refuses_what_does_not_fit():
    kernels, fn = _static_entry(128)
    case = _decode_case(12, 2, 128, 16, contexts=[200, 100], seed=3)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    qkv = torch.zeros(case["T"], 16 * 128, dtype=torch.bfloat16, device="cuda")
    code, message, out, _ = _static(fn, case, qkv, status, partial_rows=MAX_PARTIAL_ROWS + 1)
    assert code == TOO_LARGE
    assert str(MAX_PARTIAL_ROWS) in message and "partial rows" in message
    assert float(out.abs().max()) == 0.0  # nothing was launched
