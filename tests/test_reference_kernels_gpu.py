"""This library's kernels against the reference project's OWN CUDA kernels on the same inputs.

The reference's engine is Rust and cannot be built here, but its kernels are plain `.cu` files;
`x0ne_engine_b200.reference_kernels` compiles them unchanged (the reference's build flags) and
launches them at their documented grids.  Where the sources are not present (an unmodified copy of
x0ne-core/kernels/cuda under baseline/_ref, or X0NE_REFERENCE_KERNELS) these tests are skipped.
Sizes are the reference's: head size 128, one sequence, a contiguous cache [positions][kv heads][128].
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BF16_EPS = 2.0 ** -7


@pytest.fixture(scope="module")
def ref():
    from x0ne_engine_b200 import reference_kernels as R
    try:
        return R, R.load()
    except R.ReferenceUnavailable as e:
        pytest.skip(str(e).splitlines()[0])


def rnd(shape, seed, scale=1.0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def paged_from(k_cache, v_cache):
    """This library's paged cache holding the same keys and values, pages in a scattered order."""
    from x0ne_engine_b200.csrc import ops
    ctx, kvh, hd = k_cache.shape
    pages = (ctx + 63) // 64
    storage = torch.zeros((pages, 2, kvh, 64, hd), dtype=torch.bfloat16, device=DEV)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(3))
    table = torch.empty((1, pages), dtype=torch.int32)
    for lp in range(pages):
        n = min(64, ctx - 64 * lp)
        storage[order[lp], 0, :, :n] = k_cache[64 * lp:64 * lp + n].transpose(0, 1)
        storage[order[lp], 1, :, :n] = v_cache[64 * lp:64 * lp + n].transpose(0, 1)
        table[0, lp] = order[lp]
    table = table.to(DEV)
    view = ops.PagedCacheArg(storage.data_ptr(), table.data_ptr(), 2 * kvh * 64 * hd, pages, pages, 64, kvh, hd, pages)
    return storage, table, view


@pytest.mark.parametrize("rows,hidden", [(1, 4096), (7, 1000)])
def test_add_rmsnorm_against_the_reference_kernel(ref, rows, hidden):
    R, k = ref
    from x0ne_engine_b200.csrc import ops
    resid0, delta = rnd((rows, hidden), 1, 2.0, torch.float32), rnd((rows, hidden), 2)
    w = (1 + 0.1 * torch.randn(hidden, generator=torch.Generator().manual_seed(3))).bfloat16().to(DEV)   # the reference keeps norm weights in bfloat16
    r_ref, out_ref = resid0.clone(), torch.empty_like(delta)
    R.add_rmsnorm(k, r_ref, delta, w, out_ref, rows, hidden, 1e-6)
    r_own, out_own = resid0.clone(), torch.empty_like(delta)
    ops.add_rmsnorm(r_own, delta, w.float(), out_own, rows, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(r_ref, r_own)                                    # one IEEE add per value, the same bits
    assert (out_ref.float() - out_own.float()).abs().max() <= BF16_EPS * out_ref.float().abs().max()   # sums in another order


@pytest.mark.parametrize("rows,pos0", [(1, 77), (5, 0), (40, 130)])
def test_qk_norm_rope_and_cache_write_against_the_reference_kernel(ref, rows, pos0):
    R, k = ref
    from x0ne_engine_b200.csrc import ops
    qh, kvh, hd, theta, max_ctx = 8, 2, 128, 1e6, 256
    qkv = rnd((rows, (qh + 2 * kvh) * hd), 4)
    qn = (1 + 0.1 * torch.randn(hd, generator=torch.Generator().manual_seed(5))).bfloat16().to(DEV)
    kn = (1 + 0.1 * torch.randn(hd, generator=torch.Generator().manual_seed(6))).bfloat16().to(DEV)
    inv_freq = (theta ** (-torch.arange(0, hd, 2, dtype=torch.float32) / hd)).to(DEV)
    q_ref = torch.empty((rows, qh * hd), dtype=torch.bfloat16, device=DEV)
    kc, vc = torch.zeros((max_ctx, kvh, hd), dtype=torch.bfloat16, device=DEV), torch.zeros((max_ctx, kvh, hd), dtype=torch.bfloat16, device=DEV)
    R.qk_norm_rope_kv_write(k, qkv, qn, kn, inv_freq, q_ref, kc, vc, torch.tensor([pos0], dtype=torch.int32, device=DEV), rows, qh,
                            kvh, max_ctx, 1e-6)
    storage, table, view = paged_from(torch.zeros_like(kc), torch.zeros_like(vc))
    q_own = torch.empty_like(q_ref)
    slots = torch.zeros(rows, dtype=torch.int32, device=DEV)
    pos = torch.arange(pos0, pos0 + rows, dtype=torch.int32, device=DEV)
    ops.qk_norm_rope_kv_write(qkv, qn.float(), kn.float(), inv_freq, hd, q_own, view, slots, pos, rows, qh, 1e-6)
    torch.cuda.synchronize()
    tol = BF16_EPS * float(qkv.float().abs().max())
    assert (q_ref.float() - q_own.float()).abs().max() <= tol
    for r in range(rows):
        p = pos0 + r
        page = int(table[0, p // 64])
        assert (storage[page, 0, :, p % 64].float() - kc[p].float()).abs().max() <= tol
        assert torch.equal(storage[page, 1, :, p % 64], vc[p])              # V is copied bit for bit by both


@pytest.mark.parametrize("ctx", [1, 100, 129, 1000])
def test_decode_attention_against_the_reference_kernel(ref, ctx):
    R, k = ref
    from x0ne_engine_b200.csrc import ops
    qh, kvh, hd = 8, 2, 128
    kc, vc, q = rnd((ctx, kvh, hd), 7), rnd((ctx, kvh, hd), 8), rnd((1, qh * hd), 9)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    plan = R.split_plan(k, qh, kvh, sms)
    state = torch.zeros(qh * plan[2] * R.SPLIT_STATE, device=DEV)
    counter = torch.zeros(max(qh, kvh), dtype=torch.int32, device=DEV)
    out_ref = torch.empty_like(q)
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device=DEV)
    R.attention_decode(k, q, kc, vc, state, counter, out_ref, pos, qh, kvh, ctx, 1 / math.sqrt(hd), plan)
    storage, table, view = paged_from(kc, vc)
    slots = torch.zeros(1, dtype=torch.int32, device=DEV)
    for splits in (1, 3):
        out_own = torch.empty_like(q)
        ops.attention_decode_bf16(q, out_own, view, slots, pos, 1, qh, 1 / math.sqrt(hd), 0, splits, None)
        torch.cuda.synchronize()
        assert (out_ref.float() - out_own.float()).abs().max() <= BF16_EPS * float(vc.float().abs().max()), f"{splits} splits"
    assert int(counter.abs().sum()) == 0


@pytest.mark.parametrize("rows,pos0", [(9, 0), (130, 0), (70, 200)])
def test_prefill_attention_against_the_reference_kernel(ref, rows, pos0):
    R, k = ref
    from x0ne_engine_b200.csrc import ops
    qh, kvh, hd = 8, 2, 128
    ctx = pos0 + rows
    kc, vc, q = rnd((ctx, kvh, hd), 10), rnd((ctx, kvh, hd), 11), rnd((rows, qh * hd), 12)
    out_ref = torch.empty_like(q)
    R.attention_prefill(k, q, kc, vc, out_ref, torch.tensor([pos0], dtype=torch.int32, device=DEV), rows, qh, kvh, ctx,
                        1 / math.sqrt(hd))
    storage, table, view = paged_from(kc, vc)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)   # noqa: E731
    tr = ops.attention_prefill_tile_rows()
    tiles = list(range(0, rows, tr))
    out_own = torch.full_like(q, 55.0)
    ops.attention_prefill_tcgen05(q, out_own, view, mk([0] * len(tiles)), mk(tiles), len(tiles), mk([0, rows]), mk([0]), mk([pos0]), qh,
                                  1 / math.sqrt(hd), 0)
    ops.check_tc_status(q.device)
    torch.cuda.synchronize()
    assert (out_ref.float() - out_own.float()).abs().max() <= 2 * BF16_EPS * float(vc.float().abs().max())


def test_swiglu_against_the_reference_kernel(ref):
    R, k = ref
    from x0ne_engine_b200.csrc import ops
    rows, inter = 5, 1000
    gu = rnd((rows, 2 * inter), 13, 3.0)
    out_ref, out_own = torch.empty((rows, inter), dtype=torch.bfloat16, device=DEV), torch.empty((rows, inter), dtype=torch.bfloat16, device=DEV)
    R.swiglu(k, gu, out_ref, rows, inter)
    ops.swiglu(gu, out_own, rows)
    torch.cuda.synchronize()
    assert torch.equal(out_ref, out_own)               # the same formula in float32, rounded once
