"""Each CUDA kernel alone against a plain float32/float64 PyTorch restatement of its formula, at
sizes other than the engine's (no powers of two, edges of every tile), in float32 and bfloat16."""
import math

import numpy as np
import pytest
import torch

import plain_impl as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
BF16_EPS = 2.0 ** -7        # x0ne-core/oracle/tests/common/mod.rs:98-107


def ops():
    from x0ne_engine_b200.csrc import ops as o
    return o


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else BF16_EPS


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


# ------------------------------------------------------------------------------------------ embedding
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_rows_and_out_of_range_ids(dtype):
    table = rnd((37, 24), dtype, 0)
    toks = torch.tensor([0, 36, 5, 37, -1, 12], dtype=torch.int32, device=DEV)
    resid = torch.full((6, 24), 7.0, device=DEV)
    ops().embedding(table, toks, resid, 6)
    want = torch.zeros(6, 24, device=DEV)
    for r, t in enumerate(toks.tolist()):
        if 0 <= t < 37:
            want[r] = table[t].float()
    assert torch.equal(resid, want)


# ------------------------------------------------------------------------------------------ norm
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [24, 100, 120, 4096, 5000, 8200])
def test_add_rmsnorm(dtype, hidden):
    n, eps = 5, 3e-6
    resid = rnd((n, hidden), torch.float32, 1)
    delta = rnd((n, hidden), dtype, 2)
    w = 1 + 0.1 * rnd((hidden,), torch.float32, 3)
    out = torch.empty((n, hidden), dtype=dtype, device=DEV)
    r64 = resid.double() + delta.double()
    want = r64 * torch.rsqrt((r64 * r64).mean(-1, keepdim=True) + eps) * w.double()
    r_before = resid.clone()
    ops().add_rmsnorm(resid, delta, w, out, n, eps)
    assert torch.equal(resid, r_before + delta.float())          # one IEEE add, stored back
    err = (out.double() - want).abs().max() / want.abs().max()
    assert err < tol(dtype)
    # no delta, gathered rows
    rows = torch.tensor([3, 0], dtype=torch.int32, device=DEV)
    out2 = torch.zeros((2, hidden), dtype=dtype, device=DEV)
    before = resid.clone()
    ops().add_rmsnorm(resid, None, w, out2, 2, eps, rows)
    assert torch.equal(resid, before)
    assert torch.equal(out2, out[[3, 0]])


# ------------------------------------------------------------------------------------------ swiglu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(dtype):
    n, inter = 3, 203
    gu = rnd((n, 2 * inter), dtype, 4, 3.0)
    gu[0, 0] = -200.0                                           # e^200 overflows: silu is -0
    out = torch.empty((n, inter), dtype=dtype, device=DEV)
    ops().swiglu(gu, out, n)
    g, u = gu[:, :inter].double(), gu[:, inter:].double()
    want = g / (1 + torch.exp(-g)) * u
    assert (out.double() - want).abs().max() / want.abs().max() < tol(dtype)
    assert out[0, 0] == 0


# ------------------------------------------------------------------------------------------ float32 product
@pytest.mark.parametrize("m,n,k", [(1, 7, 5), (3, 130, 33), (129, 65, 100), (64, 384, 96), (200, 70, 257)])
def test_gemm_f32_matches_and_rows_do_not_depend_on_the_batch(m, n, k):
    a, w = rnd((m, k), torch.float32, 5), rnd((n, k), torch.float32, 6)
    c = torch.zeros((m, n), device=DEV)
    ops().gemm_f32_nt(a, w, c, m)
    want = a.double() @ w.double().T
    assert (c.double() - want).abs().max() / want.abs().max() < 1e-5
    # a row alone gives the same bits as the row in the batch
    c1 = torch.zeros((1, n), device=DEV)
    for r in (0, m - 1):
        ops().gemm_f32_nt(a[r:r + 1].contiguous(), w, c1, 1)
        assert torch.equal(c1[0], c[r])


# ------------------------------------------------------------------------------------------ small-M bf16 product
@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(16, 32), (100, 120), (333, 200), (4096, 1024)])
def test_gemm_bf16_smallm(m, n, k):
    x, w = rnd((m, k), torch.bfloat16, 7), rnd((n, k), torch.bfloat16, 8, 0.05)
    want = x.double() @ w.double().T
    for out_dtype in (torch.bfloat16, torch.float32):
        y = torch.full((m, n), 9.0, dtype=out_dtype, device=DEV)
        ops().gemm_bf16_smallm(x, w, y, m)
        bound = BF16_EPS if out_dtype == torch.bfloat16 else 1e-5
        mag = (x.double().abs() @ w.double().abs().T).max()    # error is a share of sum |terms|
        assert (y.double() - want).abs().max() / mag < bound


@pytest.mark.parametrize("m,inter,k", [(1, 48, 24), (5, 200, 120), (16, 1000, 512)])
def test_gemm_bf16_smallm_with_swiglu_epilogue(m, inter, k):
    x, w = rnd((m, k), torch.bfloat16, 9), rnd((2 * inter, k), torch.bfloat16, 10, 0.2)
    y = torch.zeros((m, inter), dtype=torch.bfloat16, device=DEV)
    ops().gemm_bf16_smallm(x, w, y, m, swiglu=True)
    gu = x.double() @ w.double().T
    g, u = gu[:, :inter], gu[:, inter:]
    want = g / (1 + torch.exp(-g)) * u
    assert (y.double() - want).abs().max() / want.abs().max() < 2 * BF16_EPS


# ------------------------------------------------------------------------------------------ tcgen05 product
@pytest.mark.parametrize("pair", [True, False])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (100, 300, 200), (1000, 520, 328), (2048, 1024, 512)])
def test_gemm_bf16_tcgen05(m, n, k, pair):
    """TMA + tcgen05.mma + tensor memory, single blocks and pairs; rows, columns and k past the tiles."""
    o = ops()
    x, w = rnd((m, k), torch.bfloat16, 90), rnd((n, k), torch.bfloat16, 91, 0.05)
    want = x.double() @ w.double().T
    mag = (x.double().abs() @ w.double().abs().T).max()
    for out_dtype, bound in ((torch.bfloat16, BF16_EPS), (torch.float32, 1e-5)):
        y = torch.full((m, n), 9.0, dtype=out_dtype, device=DEV)
        o.gemm_bf16_tcgen05(x, w, y, m, pair=pair)
        assert int(o.gemm_tc_status(x.device)[0]) == 0
        assert (y.double() - want).abs().max() / mag < bound
    o.check_tc_status(x.device)


@pytest.mark.parametrize("pair", [True, False])
@pytest.mark.parametrize("m,inter,k", [(128, 128, 64), (300, 200, 136), (1024, 1000, 512)])
def test_gemm_bf16_tcgen05_with_swiglu_epilogue(m, inter, k, pair):
    o = ops()
    x, w = rnd((m, k), torch.bfloat16, 92), rnd((2 * inter, k), torch.bfloat16, 93, 0.2)
    y = torch.zeros((m, inter), dtype=torch.bfloat16, device=DEV)
    o.gemm_bf16_tcgen05(x, w, y, m, swiglu=True, pair=pair)
    assert int(o.gemm_tc_status(x.device)[0]) == 0
    gu = x.double() @ w.double().T
    g, u = gu[:, :inter], gu[:, inter:]
    want = g / (1 + torch.exp(-g)) * u
    assert (y.double() - want).abs().max() / want.abs().max() < 2 * BF16_EPS


# ------------------------------------------------------------------------------------------ rope + cache write
def make_cache(kv_heads, head_dim, n_pages, n_slots, dtype, pages_per_slot):
    """A one-entry paged cache with a page table that scatters each slot's pages."""
    o = ops()
    storage = torch.zeros((n_pages, 2, kv_heads, 64, head_dim), dtype=dtype, device=DEV)
    table = torch.full((n_slots, pages_per_slot), -1, dtype=torch.int32, device=DEV)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(11)).tolist()
    for s in range(n_slots):
        for p in range(pages_per_slot):
            table[s, p] = perm[s * pages_per_slot + p]
    view = o.PagedCacheArg(storage.data_ptr(), table.data_ptr(), 2 * kv_heads * 64 * head_dim, pages_per_slot,
                           pages_per_slot, 64, kv_heads, head_dim, n_pages)
    return storage, table, view


def dense_slot(storage, table, slot):
    """K and V of one slot as [2, kv_heads, positions, head_dim] (positions in order)."""
    pages = table[slot].long().clamp(min=0)
    t = storage[pages]                                   # [pages, 2, kv_heads, 64, hd]
    return t.permute(1, 2, 0, 3, 4).reshape(2, t.shape[2], -1, t.shape[4])


def cache_rows(storage, table, slot, which, kv_head, n):
    """Rows 0..n-1 of K (which=0) or V (which=1) of one slot and head, as [n, head_dim]."""
    return dense_slot(storage, table, slot)[which, kv_head, :n]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_heads,kv_heads,hd,rot", [(4, 2, 16, 16), (6, 2, 32, 32), (5, 1, 48, 48), (3, 3, 24, 12),
                                                       (2, 1, 128, 128), (5, 3, 64, 64), (3, 1, 256, 256)])
@pytest.mark.parametrize("table_rows", [0, 100, 200])      # no table; one that ends before position 130; a full one
def test_qk_norm_rope_kv_write(dtype, q_heads, kv_heads, hd, rot, table_rows):
    o = ops()
    n, eps, theta = 7, 1e-5, 50000.0
    storage, table, view = make_cache(kv_heads, hd, 8, 2, dtype, 3)
    storage.fill_(-77.0)                                         # sentinel: only written rows may change
    qkv = rnd((n, (q_heads + 2 * kv_heads) * hd), dtype, 12)
    qn, kn = 1 + 0.1 * rnd((hd,), torch.float32, 13), 1 + 0.1 * rnd((hd,), torch.float32, 14)
    inv = torch.from_numpy(P.inv_freq(rot, theta)).to(DEV)
    slots = torch.tensor([0, 0, 0, 1, 1, 1, 1], dtype=torch.int32, device=DEV)
    pos = torch.tensor([63, 64, 65, 0, 1, 130, 5], dtype=torch.int32, device=DEV)
    q_out = torch.empty((n, q_heads * hd), dtype=dtype, device=DEV)
    rope_tab = None
    if table_rows:
        ang = (np.arange(table_rows, dtype=np.float32)[:, None] * P.inv_freq(rot, theta)[None, :]).astype(np.float64)
        rope_tab = torch.from_numpy(np.concatenate([np.cos(ang), np.sin(ang)], 1).astype(np.float32)).to(DEV)
    o.qk_norm_rope_kv_write(qkv, qn, kn, inv, rot, q_out, view, slots, pos, n, q_heads, eps, rope_table=rope_tab)

    x = qkv.double().cpu().numpy()
    qd, kvd = q_heads * hd, kv_heads * hd

    def rope_part(v, w):
        v = P.rmsnorm(v, w.double().cpu().numpy(), eps)
        rotated = P.rope(v[..., :rot], pos.cpu().numpy(), P.inv_freq(rot, theta))
        return np.concatenate([rotated, v[..., rot:]], axis=-1)
    want_q = rope_part(x[:, :qd].reshape(n, q_heads, hd), qn).reshape(n, qd)
    want_k = rope_part(x[:, qd:qd + kvd].reshape(n, kv_heads, hd), kn)
    want_v = x[:, qd + kvd:].reshape(n, kv_heads, hd)
    t = 1e-3 if dtype == torch.float32 else BF16_EPS            # rope tolerance 1e-3 * max|x| (same source)
    assert np.abs(q_out.double().cpu().numpy() - want_q).max() / np.abs(want_q).max() < t
    written = set()
    for r in range(n):
        s, p = int(slots[r]), int(pos[r])
        page = int(table[s, p // 64])
        for h in range(kv_heads):
            got_k = storage[page, 0, h, p % 64].double().cpu().numpy()
            got_v = storage[page, 1, h, p % 64]
            assert np.abs(got_k - want_k[r, h]).max() / np.abs(want_k).max() < t
            assert torch.equal(got_v, qkv[r, qd + kvd + h * hd: qd + kvd + (h + 1) * hd])    # V is copied bit for bit
            written.add((page, h, p % 64))
    untouched = torch.ones_like(storage, dtype=torch.bool)
    for page, h, off in written:
        untouched[page, :, h, off] = False
    assert torch.all(storage[untouched] == -77.0)


# ------------------------------------------------------------------------------------------ attention
def plain_attention_over_cache(q, storage, table, slots, pos, q_heads, kv_heads, hd, window):
    """float64: each row attends keys max(0, p-w+1)..p of its slot."""
    n = q.shape[0]
    out = torch.zeros((n, q_heads, hd), dtype=torch.float64)
    group = q_heads // kv_heads
    dense = {}
    for r in range(n):
        s, p = int(slots[r]), int(pos[r])
        if s not in dense:
            dense[s] = dense_slot(storage, table, s).double().cpu()
        lo = max(0, p - window + 1) if window else 0
        for h in range(q_heads):
            kh = h // group
            k, v = dense[s][0, kh, lo:p + 1], dense[s][1, kh, lo:p + 1]
            sc = (k @ q[r, h].double().cpu()) / math.sqrt(hd)
            out[r, h] = torch.softmax(sc, 0) @ v
    return out.reshape(n, q_heads * hd)


def fill_cache(storage, dtype, seed, scale=1.0):
    storage.copy_(rnd(tuple(storage.shape), dtype, seed, scale))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_heads,kv_heads,hd", [(4, 2, 16), (6, 2, 32), (5, 1, 48), (3, 1, 8), (2, 2, 130)])
@pytest.mark.parametrize("window", [0, 5, 70])
def test_plain_attention_kernel(dtype, q_heads, kv_heads, hd, window):
    o = ops()
    storage, table, view = make_cache(kv_heads, hd, 8, 2, dtype, 3)
    fill_cache(storage, dtype, 20)
    slots = torch.tensor([0, 0, 1, 1, 1, 0], dtype=torch.int32, device=DEV)
    pos = torch.tensor([0, 63, 64, 129, 1, 31], dtype=torch.int32, device=DEV)
    n = 6
    q = rnd((n, q_heads * hd), dtype, 21)
    out = torch.empty_like(q)
    o.attention_rows(q, out, view, slots, pos, n, q_heads, 1 / math.sqrt(hd), window)
    want = plain_attention_over_cache(q.reshape(n, q_heads, hd), storage, table, slots, pos, q_heads, kv_heads, hd, window)
    t = 1e-5 if dtype == torch.float32 else BF16_EPS
    assert (out.double().cpu() - want).abs().max() / storage.double().abs().max().cpu() < t


def test_plain_attention_finds_one_far_key_among_hundreds():
    """One key at a far position carries a score that dwarfs the rest: the output must be its value."""
    o = ops()
    kv_heads, hd, q_heads = 1, 16, 2
    storage, table, view = make_cache(kv_heads, hd, 8, 1, torch.float32, 8)
    fill_cache(storage, torch.float32, 30, 0.05)
    q = torch.zeros((1, q_heads * hd), device=DEV)
    q[0, :] = 1.0
    far = 77
    page = int(table[0, far // 64])
    storage[page, 0, 0, far % 64] = 40.0                         # its score is 16 * 40 / 4 = 160
    slots = torch.zeros(1, dtype=torch.int32, device=DEV)
    pos = torch.tensor([500], dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    o.attention_rows(q, out, view, slots, pos, 1, q_heads, 0.25, 0)
    want = storage[page, 1, 0, far % 64]
    assert torch.allclose(out[0, :hd], want, atol=1e-6) and torch.allclose(out[0, hd:], want, atol=1e-6)
    # with a window that ends just after the far key, it is gone
    o.attention_rows(q, out, view, slots, pos, 1, q_heads, 0.25, 500 - far)
    assert not torch.allclose(out[0, :hd], want, atol=1e-3)
    o.attention_rows(q, out, view, slots, pos, 1, q_heads, 0.25, 500 - far + 1)
    assert torch.allclose(out[0, :hd], want, atol=1e-6)


def tiles_for(first_rows):
    """Host tables of the prefill kernel for sequences whose rows start at first_rows (last = end)."""
    tile_seq, tile_row0 = [], []
    tr = ops().attention_prefill_tile_rows()
    for s in range(len(first_rows) - 1):
        for r0 in range(first_rows[s], first_rows[s + 1], tr):
            tile_seq.append(s)
            tile_row0.append(r0)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)   # noqa: E731
    return mk(tile_seq), mk(tile_row0), len(tile_seq)


@pytest.mark.parametrize("q_heads,kv_heads,hd", [(4, 2, 16), (6, 2, 32), (5, 1, 48), (8, 2, 64), (4, 1, 128), (3, 3, 112)])
@pytest.mark.parametrize("window", [0, 3, 64, 100])
def test_prefill_attention_bf16_equals_plain_kernel(q_heads, kv_heads, hd, window):
    """Several sequences of unequal length, one of them continuing from position 70, tile edges at
    63/64/65 rows: the tensor-core kernel against the float64 restatement."""
    o = ops()
    storage, table, view = make_cache(kv_heads, hd, 16, 3, torch.bfloat16, 5)
    fill_cache(storage, torch.bfloat16, 40)
    lens, pos0, seq_slots = [65, 1, 130], [0, 7, 70], [2, 0, 1]     # 130 rows: a full tile and a short one
    first = [0, 65, 66, 196]
    n = first[-1]
    slots = torch.tensor(sum(([s] * l for s, l in zip(seq_slots, lens)), []), dtype=torch.int32, device=DEV)
    pos = torch.tensor(sum((list(range(p, p + l)) for p, l in zip(pos0, lens)), []), dtype=torch.int32, device=DEV)
    q = rnd((n, q_heads * hd), torch.bfloat16, 41)
    out = torch.full_like(q, 55.0)
    tile_seq, tile_row0, n_tiles = tiles_for(first)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)   # noqa: E731
    o.attention_prefill_bf16(q, out, view, tile_seq, tile_row0, n_tiles, mk(first), mk(seq_slots), mk(pos0), q_heads,
                             1 / math.sqrt(hd), window)
    ref = torch.empty_like(q)
    o.attention_rows(q, ref, view, slots, pos, n, q_heads, 1 / math.sqrt(hd), window)
    vmax = float(storage.float().abs().max())
    assert (out.float() - ref.float()).abs().max() / vmax < 2 * BF16_EPS
    rows = [0, 63, 64, 65, 66, 130, 195]
    want = plain_attention_over_cache(q.reshape(n, q_heads, hd)[rows], storage, table, slots[rows], pos[rows], q_heads,
                                      kv_heads, hd, window)
    assert (out[rows].double().cpu() - want).abs().max() / vmax < BF16_EPS


def run_tc_attention(q_heads, kv_heads, hd, window, lens, pos0, seq_slots, seed=40, edit=None, q_edit=None):
    """The tcgen05 prefill kernel and the plain kernel on the same cache and queries; returns
    (out, ref, largest cached magnitude, q, storage, table, slots, pos)."""
    o = ops()
    n_slots = len(lens)
    pages_per = max((p + l + 63) // 64 for p, l in zip(pos0, lens)) + 1
    storage, table, view = make_cache(kv_heads, hd, n_slots * pages_per, n_slots, torch.bfloat16, pages_per)
    fill_cache(storage, torch.bfloat16, seed)
    if edit is not None:
        edit(storage, table)
    first = [0]
    for l in lens:
        first.append(first[-1] + l)
    n = first[-1]
    slots = torch.tensor(sum(([s] * l for s, l in zip(seq_slots, lens)), []), dtype=torch.int32, device=DEV)
    pos = torch.tensor(sum((list(range(p, p + l)) for p, l in zip(pos0, lens)), []), dtype=torch.int32, device=DEV)
    q = rnd((n, q_heads * hd), torch.bfloat16, seed + 1)
    if q_edit is not None:
        q_edit(q)
    out = torch.full_like(q, 55.0)
    tile_seq, tile_row0, n_tiles = tiles_for(first)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)   # noqa: E731
    assert o.attention_tc_takes(view, torch.bfloat16)
    o.attention_prefill_tcgen05(q, out, view, tile_seq, tile_row0, n_tiles, mk(first), mk(seq_slots), mk(pos0), q_heads,
                                1 / math.sqrt(hd), window)
    o.check_tc_status(q.device)
    ref = torch.empty_like(q)
    o.attention_rows(q, ref, view, slots, pos, n, q_heads, 1 / math.sqrt(hd), window)
    return out, ref, float(storage.float().abs().max()), q, storage, table, slots, pos


@pytest.mark.parametrize("m", [9, 16, 17, 33, 64])
@pytest.mark.parametrize("n,k", [(128, 256), (200, 264), (1024, 4096), (6144, 512), (4096, 12288)])
@pytest.mark.parametrize("out", ["bf16", "f32", "swiglu"])
def test_skinny_tcgen05_product(m, n, k, out):
    """The tcgen05 product for 9 to 64 rows (K cut over a cluster, partial sums added through shared
    memory) against float64: widths that are no multiples of the tiles, every output kind, and the
    same bits on a second call."""
    o = ops()
    swiglu = out == "swiglu"
    x = rnd((m, k), torch.bfloat16, 90)
    w = rnd(((2 if swiglu else 1) * n, k), torch.bfloat16, 91, 1.0 / math.sqrt(k))
    y = torch.full((m, n), 7.0, dtype=torch.float32 if out == "f32" else torch.bfloat16, device=DEV)
    assert o.gemm_skinny_tc_takes(w, m)
    o.gemm_bf16_skinny_tcgen05(x, w, y, m, swiglu=swiglu)
    o.check_tc_status(x.device)
    ref = x.double() @ w.double().T
    if swiglu:
        g, u = ref[:, :n], ref[:, n:]
        ref = g / (1 + torch.exp(-g)) * u
    tol = 1e-5 if out == "f32" else BF16_EPS
    assert float((y.double() - ref).abs().max() / ref.abs().max()) < tol
    y2 = torch.empty_like(y)
    o.gemm_bf16_skinny_tcgen05(x, w, y2, m, swiglu=swiglu)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("q_heads,kv_heads,hd", [(8, 2, 64), (4, 1, 128), (3, 3, 64), (10, 5, 128)])
@pytest.mark.parametrize("window", [0, 3, 64, 100])
def test_prefill_attention_tcgen05_equals_plain_kernel(q_heads, kv_heads, hd, window):
    """Unequal sequences, one continuing from position 70 and one of four tiles, slots in another
    order than the rows: the tcgen05 kernel against the plain kernel and the float64 restatement."""
    out, ref, vmax, q, storage, table, slots, pos = run_tc_attention(
        q_heads, kv_heads, hd, window, [65, 1, 130, 500], [0, 7, 70, 3], [2, 0, 1, 3])
    assert (out.float() - ref.float()).abs().max() / vmax < 2 * BF16_EPS
    rows = [0, 63, 64, 65, 66, 130, 195, 196, 323, 324, 695]
    n = q.shape[0]
    want = plain_attention_over_cache(q.reshape(n, q_heads, hd)[rows], storage, table, slots[rows], pos[rows], q_heads,
                                      kv_heads, hd, window)
    assert (out[rows].double().cpu() - want).abs().max() / vmax < BF16_EPS


@pytest.mark.parametrize("gain", [0.7, 40.0])
def test_prefill_attention_tcgen05_late_large_key(gain):
    """A key at position 300 scores far above everything before it for every later query.  With
    the small gain the rows keep their reference maximum (the kernel raises it only past a
    threshold); with the large one the output accumulated so far is rescaled in tensor memory.
    Rows before 300 never see the key."""
    hd, far = 128, 300

    def edit(storage, table):
        page = int(table[0, far // 64])
        storage[page, 0, 0, far % 64] = gain                       # key: all components equal

    def q_edit(q):
        q[:, :hd] = q[:, :hd].abs()                                # head 0: positive queries, so the score is large

    out, ref, vmax, q, storage, table, slots, pos = run_tc_attention(2, 1, hd, 0, [450], [0], [0], seed=70, edit=edit,
                                                                     q_edit=q_edit)
    assert (out.float() - ref.float()).abs().max() / vmax < 2 * BF16_EPS
    if gain > 10:
        page = int(table[0, far // 64])
        value = storage[page, 1, 0, far % 64].float()
        assert (out[far + 5, :hd].float() - value).abs().max() < 2 * BF16_EPS * vmax     # that key alone
    assert torch.isfinite(out.float()).all()


@pytest.mark.parametrize("q_heads,kv_heads,hd", [(4, 2, 16), (6, 2, 32), (5, 1, 48), (32, 8, 128), (20, 1, 64), (3, 3, 96)])
@pytest.mark.parametrize("window", [0, 9, 200])
@pytest.mark.parametrize("splits", [1, 2, 5, 13])
def test_decode_attention_bf16(q_heads, kv_heads, hd, window, splits):
    """One row per sequence at contexts around every tile edge, any number of splits (also more
    splits than pages); the arrival counters must be back at zero afterwards."""
    o = ops()
    ctxs = [1, 2, 16, 17, 63, 64, 65, 127, 128, 129, 300, 513]
    n = len(ctxs)
    storage, table, view = make_cache(kv_heads, hd, n * 9, n, torch.bfloat16, 9)
    fill_cache(storage, torch.bfloat16, 50)
    slots = torch.arange(n, dtype=torch.int32, device=DEV)
    pos = torch.tensor([c - 1 for c in ctxs], dtype=torch.int32, device=DEV)
    q = rnd((n, q_heads * hd), torch.bfloat16, 51)
    out = torch.full_like(q, 55.0)
    nbytes = o.attention_decode_scratch_bytes(n, q_heads, kv_heads, hd, splits)
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    for _ in range(2):                                            # twice: the counters were reset
        o.attention_decode_bf16(q, out, view, slots, pos, n, q_heads, 1 / math.sqrt(hd), window, splits, scratch)
    want = plain_attention_over_cache(q.reshape(n, q_heads, hd), storage, table, slots, pos, q_heads, kv_heads, hd, window)
    vmax = float(storage.float().abs().max())
    assert (out.double().cpu() - want).abs().max() / vmax < BF16_EPS
    if 1 < splits <= 8:      # without scratch the splits merge inside a thread-block cluster
        out2 = torch.full_like(q, 55.0)
        o.attention_decode_bf16(q, out2, view, slots, pos, n, q_heads, 1 / math.sqrt(hd), window, splits, None)
        # (the same sums in the same order, unless the launch is small enough for blocks of 8 warps,
        # which add their warps' partial sums in another grouping)
        assert (out2.double().cpu() - want).abs().max() / vmax < BF16_EPS
        assert (out2.float() - out.float()).abs().max() / vmax < BF16_EPS
        out3 = torch.full_like(q, 55.0)
        o.attention_decode_bf16(q, out3, view, slots, pos, n, q_heads, 1 / math.sqrt(hd), window, splits, None)
        assert torch.equal(out3, out2)
    group_chunks = (q_heads // kv_heads + 15) // 16
    counters = scratch[: n * kv_heads * group_chunks * 4].view(torch.int32)
    assert int(counters.abs().sum()) == 0


@pytest.mark.parametrize("q_heads,kv_heads,hd", [(4, 2, 16), (5, 1, 48), (32, 8, 128), (3, 3, 96)])
@pytest.mark.parametrize("window", [0, 200])
@pytest.mark.parametrize("cluster,groups", [(2, 2), (8, 4), (3, 5), (5, 7), (8, 8)])
def test_decode_attention_bf16_in_several_clusters(q_heads, kv_heads, hd, window, cluster, groups):
    """The splits of a (sequence, kv head) as several thread-block clusters: each cluster merges in
    shared memory, the clusters' results meet in scratch.  Contexts around every tile edge, also
    fewer pages than splits (clusters with nothing to read); the arrival counters must be back at
    zero afterwards, and the second call must give the same bits."""
    o = ops()
    ctxs = [1, 2, 17, 64, 65, 129, 300, 513, 1100]
    n = len(ctxs)
    storage, table, view = make_cache(kv_heads, hd, n * 18, n, torch.bfloat16, 18)
    fill_cache(storage, torch.bfloat16, 54)
    slots = torch.arange(n, dtype=torch.int32, device=DEV)
    pos = torch.tensor([c - 1 for c in ctxs], dtype=torch.int32, device=DEV)
    q = rnd((n, q_heads * hd), torch.bfloat16, 55)
    scratch = torch.zeros(o.attention_decode_scratch_bytes(n, q_heads, kv_heads, hd, groups), dtype=torch.uint8, device=DEV)
    outs = []
    for _ in range(2):
        out = torch.full_like(q, 55.0)
        o.attention_decode_bf16(q, out, view, slots, pos, n, q_heads, 1 / math.sqrt(hd), window, cluster * groups, scratch,
                                groups=groups)
        outs.append(out)
    want = plain_attention_over_cache(q.reshape(n, q_heads, hd), storage, table, slots, pos, q_heads, kv_heads, hd, window)
    vmax = float(storage.float().abs().max())
    assert (outs[0].double().cpu() - want).abs().max() / vmax < BF16_EPS
    assert torch.equal(outs[0], outs[1])
    group_chunks = (q_heads // kv_heads + 15) // 16
    assert int(scratch[: n * kv_heads * group_chunks * 4].view(torch.int32).abs().sum()) == 0
    with pytest.raises(o.KernelError):      # clusters of 2 to 8 blocks; a scratch is needed
        o.attention_decode_bf16(q, out, view, slots, pos, n, q_heads, 1 / math.sqrt(hd), window, 9 * 2, scratch, groups=2)
    with pytest.raises(o.KernelError):
        o.attention_decode_bf16(q, out, view, slots, pos, n, q_heads, 1 / math.sqrt(hd), window, cluster * groups, None,
                                groups=groups)


@pytest.mark.parametrize("splits", [1, 3])
def test_decode_attention_bf16_long_contexts(splits):
    """Contexts past 128 pages per block (the page numbers a block keeps in shared memory) and a
    far key that decides the output: position 8200 of 9000 carries a score far above the rest."""
    o = ops()
    q_heads, kv_heads, hd = 4, 2, 64
    ctxs = [8191, 8193, 9000]
    n = len(ctxs)
    pages = 141
    storage, table, view = make_cache(kv_heads, hd, n * pages, n, torch.bfloat16, pages)
    fill_cache(storage, torch.bfloat16, 52, 0.3)
    far = 8200
    page = int(table[2, far // 64])
    storage[page, 0, :, far % 64] = 6.0                          # key of both kv heads at the far position
    slots = torch.arange(n, dtype=torch.int32, device=DEV)
    pos = torch.tensor([c - 1 for c in ctxs], dtype=torch.int32, device=DEV)
    q = rnd((n, q_heads * hd), torch.bfloat16, 53)
    q[2] = q[2].abs() + 1.0                                      # score of the far key: about 64 * 6 * 1.8 / 8
    out = torch.full_like(q, 55.0)
    scratch = torch.zeros(o.attention_decode_scratch_bytes(n, q_heads, kv_heads, hd, splits), dtype=torch.uint8, device=DEV)
    o.attention_decode_bf16(q, out, view, slots, pos, n, q_heads, 1 / math.sqrt(hd), 0, splits, scratch)
    ref = torch.empty_like(q)
    o.attention_rows(q, ref, view, slots, pos, n, q_heads, 1 / math.sqrt(hd), 0)
    vmax = float(storage.float().abs().max())
    assert (out.float() - ref.float()).abs().max() / vmax < 2 * BF16_EPS
    want = storage[page, 1, :, far % 64].float()                 # [kv_heads, hd]: the far position's values
    got = out[2].float().reshape(kv_heads, q_heads // kv_heads, hd)
    assert (got - want[:, None, :]).abs().max() < 2 * BF16_EPS * vmax


# ------------------------------------------------------------------------------------------ sampler
@pytest.mark.parametrize("v", [5, 1000, 4099, 151936])
@pytest.mark.parametrize("rows", [1, 8, 200])
def test_sampler_with_the_many_block_search_for_the_largest_logit(v, rows):
    """With a word of scratch per row the rows' largest logits are found by many blocks per row
    first.  Same picks, greedy and sampled, with ties, a NaN row, a finished row and a row whose
    start is not 16-byte aligned; the scratch is zero again afterwards."""
    o = ops()
    logits = rnd((rows, v), torch.float32, 61)                    # (5 and 4,099 logits: rows that start off 16-byte boundaries)
    logits[0, v // 2] = logits[0, v - 1] = 40.0                   # tie: lowest index
    if rows > 1:
        logits[1, v // 3] = float("nan")
    temp = torch.zeros(rows, dtype=torch.float32, device=DEV)
    temp[2::3] = 0.8                                              # every third row is sampled
    top_p = torch.full((rows,), 0.9, dtype=torch.float32, device=DEV)
    seed = torch.arange(rows, dtype=torch.int64, device=DEV) + 5
    results = []
    for scratch in (None, torch.zeros(rows, dtype=torch.int64, device=DEV)):
        out = torch.full((rows,), -9, dtype=torch.int32, device=DEV)
        fin = torch.zeros(rows, dtype=torch.int32, device=DEV)
        fin[rows - 1] = 1 if rows > 2 else 0
        cnt = torch.zeros(rows, dtype=torch.int32, device=DEV)
        nxt = torch.full((rows,), 7, dtype=torch.int32, device=DEV)
        o.sample(logits, rows, out, temperature=temp, top_p=top_p, seed=seed, draw_counter=cnt, finished=fin,
                 next_token=nxt, row_best=scratch)
        results.append((out.clone(), fin.clone(), cnt.clone(), nxt.clone()))
        if scratch is not None:
            assert int(scratch.abs().sum()) == 0
            o.sample(logits, rows, out, temperature=temp, top_p=top_p, seed=seed, draw_counter=cnt * 0, finished=fin * 0 + fin,
                     next_token=nxt, row_best=scratch)          # a second step on the same scratch
            assert int(scratch.abs().sum()) == 0
    for a, b in zip(*results):
        assert torch.equal(a, b)
    out = results[0][0]
    assert out[0] == v // 2
    if rows > 1:
        assert out[1] == -1
    if rows > 2:
        assert out[rows - 1] == -2


def test_sampler_argmax_ties_nan_and_feedback():
    o = ops()
    v = 1000
    logits = rnd((4, v), torch.float32, 60)
    logits[0, 17] = logits[0, 900] = 50.0                         # tie: lowest index
    logits[1, 5] = float("nan")
    logits[2, 999] = 60.0
    out = torch.zeros(4, dtype=torch.int32, device=DEV)
    nxt = torch.full((4,), 7, dtype=torch.int32, device=DEV)
    posn = torch.tensor([10, 20, 30, 40], dtype=torch.int32, device=DEV)
    fin = torch.tensor([0, 0, 0, 1], dtype=torch.int32, device=DEV)
    budget = torch.tensor([5, 5, 1, 5], dtype=torch.int32, device=DEV)
    cnt = torch.zeros(4, dtype=torch.int32, device=DEV)
    o.sample(logits, 4, out, finished=fin, budget=budget, next_token=nxt, next_pos=posn, draw_counter=cnt)
    assert out.tolist() == [17, -1, 999, -2]
    assert nxt.tolist() == [17, 7, 7, 7]                          # NaN row, spent budget, finished row: not fed
    assert posn.tolist() == [11, 20, 30, 40]
    assert fin.tolist() == [0, 1, 1, 1] and budget.tolist() == [4, 5, 0, 5] and cnt.tolist() == [1, 0, 1, 0]
    stop = torch.tensor([17], dtype=torch.int32, device=DEV)
    fin.zero_()
    o.sample(logits, 1, out, finished=fin, stop_ids=stop, next_token=nxt, next_pos=posn)
    assert out[0] == 17 and fin[0] == 1 and posn[0] == 11         # a stop token is reported but not fed


@pytest.mark.parametrize("vocab", [2, 331, 1024, 151936])
@pytest.mark.parametrize("top_p", [1.0, 0.9, 0.3])
def test_sampler_draws_by_inverse_cdf_with_the_documented_stream(vocab, top_p):
    """The device's pick must be the token whose interval of the index-ordered CDF over the kept
    tokens holds the uniform that (seed, draw counter) give, up to float32 rounding at the edges."""
    o = ops()
    rows, temp = 6, 0.7
    logits = rnd((rows, vocab), torch.float32, 70, 3.0)
    seeds = torch.tensor([1, 2, 3, 2 ** 40 + 5, 7, 7], dtype=torch.int64, device=DEV)
    cnt = torch.tensor([0, 1, 2, 3, 4, 5], dtype=torch.int32, device=DEV)
    out = torch.zeros(rows, dtype=torch.int32, device=DEV)
    t = torch.full((rows,), temp, device=DEV)
    p = torch.full((rows,), top_p, device=DEV)
    cnt0 = cnt.clone()
    o.sample(logits, rows, out, temperature=t, top_p=p, seed=seeds, draw_counter=cnt)
    assert cnt.tolist() == [c + 1 for c in cnt0.tolist()]
    lg = logits.cpu().numpy()
    for r in range(rows):
        u = P.uniform_of(int(seeds[r]), int(cnt0[r]))
        lo, hi = P.draw_interval(lg[r], temp, top_p, int(out[r]))
        assert hi > lo, f"row {r}: token {int(out[r])} is outside the nucleus"
        assert lo - 1e-5 <= u <= hi + 1e-5, (r, int(out[r]), lo, u, hi)


def test_sampler_rows_do_not_depend_on_batch_mates():
    o = ops()
    logits = rnd((5, 4000), torch.float32, 80, 2.0)
    seeds = torch.arange(5, dtype=torch.int64, device=DEV) + 11
    t = torch.full((5,), 0.9, device=DEV)
    p = torch.full((5,), 0.95, device=DEV)
    out = torch.zeros(5, dtype=torch.int32, device=DEV)
    o.sample(logits, 5, out, temperature=t, top_p=p, seed=seeds)
    for r in range(5):
        one = torch.zeros(1, dtype=torch.int32, device=DEV)
        o.sample(logits[r:r + 1].contiguous(), 1, one, temperature=t[r:r + 1].contiguous(),
                 top_p=p[r:r + 1].contiguous(), seed=seeds[r:r + 1].contiguous())
        assert int(one[0]) == int(out[r])


@pytest.mark.parametrize("hd,dtype", [(64, torch.bfloat16), (128, torch.bfloat16), (48, torch.bfloat16), (32, torch.float32)])
def test_attention_kernels_on_a_ring_that_has_lapped(hd, dtype):
    """A windowed cache keeps a ring of 3 pages: logical page (pos / 64) % 3.  A sequence is at
    position 400, so the ring has lapped twice; the places of its newest page past position 400
    still hold keys of positions 208..255 (made huge here: a read past the causal bound would
    show), and key 330 scores far above everything: with a window of 70 the rows at 380..399 see
    it and give its value, the row at 400 must not (it lies just outside, in a page that is still
    in the ring).  Every attention kernel that takes the shape: a chunk of 21 rows through the
    prefill kernels, the last row through the decode kernel, all rows through the plain kernel,
    against float64 on the positions in order."""
    o = ops()
    q_heads, kv_heads, window, last, ring = 4, 2, 70, 400, 3
    n_pages, table_stride = 7, 4
    g = torch.Generator().manual_seed(61)
    K = (torch.randn((last + 1, kv_heads, hd), generator=g) * 0.3).to(dtype)
    V = torch.randn((last + 1, kv_heads, hd), generator=g).to(dtype)
    far = 330
    K[far] = 6.0                                            # against positive queries: the largest score by far
    storage = torch.zeros((n_pages, 2, kv_heads, 64, hd), dtype=dtype, device=DEV)
    table = torch.full((2, table_stride), -1, dtype=torch.int32, device=DEV)
    table[1, :ring] = torch.tensor([5, 2, 6], dtype=torch.int32)
    table[0, :ring] = torch.tensor([0, 1, 3], dtype=torch.int32)
    newest = last // 64
    for pos in range((newest - ring + 1) * 64, (newest + 1) * 64):
        page = int(table[1, (pos // 64) % ring])
        if pos <= last:
            storage[page, 0, :, pos % 64] = K[pos].to(DEV)
            storage[page, 1, :, pos % 64] = V[pos].to(DEV)
        else:                                               # what the lap before left there
            storage[page, 0, :, pos % 64] = 50.0
            storage[page, 1, :, pos % 64] = -99.0
    view = o.PagedCacheArg(storage.data_ptr(), table.data_ptr(), 2 * kv_heads * 64 * hd, table_stride, ring, 64, kv_heads,
                           hd, n_pages)
    first_pos = 380
    n = last - first_pos + 1
    q = (torch.rand((n, q_heads * hd), generator=g) * 0.5 + 0.25).to(dtype).to(DEV)
    slots = torch.full((n,), 1, dtype=torch.int32, device=DEV)
    pos = torch.arange(first_pos, last + 1, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(hd)

    want = torch.zeros((n, q_heads, hd), dtype=torch.float64)
    for r in range(n):
        p = first_pos + r
        lo = p - window + 1
        for h in range(q_heads):
            kh = h // (q_heads // kv_heads)
            sc = (K[lo:p + 1, kh].double() @ q[r].reshape(q_heads, hd)[h].double().cpu()) * scale
            want[r, h] = torch.softmax(sc, 0) @ V[lo:p + 1, kh].double()
    want = want.reshape(n, q_heads * hd)
    assert (want[:-1].reshape(n - 1, q_heads, hd) - V[far].double().repeat_interleave(2, 0)).abs().max() < 0.05   # they see key 330
    assert (want[-1].reshape(q_heads, hd) - V[far].double().repeat_interleave(2, 0)).abs().max() > 0.5            # row 400 does not
    tol = (1e-5 if dtype == torch.float32 else BF16_EPS) * float(V.float().abs().max())

    out = torch.full_like(q, 55.0)
    o.attention_rows(q, out, view, slots, pos, n, q_heads, scale, window)
    assert (out.double().cpu() - want).abs().max() < tol, "plain kernel"
    if dtype != torch.bfloat16:
        return
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)   # noqa: E731
    tile_seq, tile_row0, n_tiles = tiles_for([0, n])
    kernels = [("mma.sync prefill", o.attention_prefill_bf16)]
    if o.attention_tc_takes(view, dtype):
        kernels.append(("tcgen05 prefill", o.attention_prefill_tcgen05))
    for name, kernel in kernels:
        out = torch.full_like(q, 55.0)
        kernel(q, out, view, tile_seq, tile_row0, n_tiles, mk([0, n]), mk([1]), mk([first_pos]), q_heads, scale, window)
        o.check_tc_status(q.device)
        assert (out.double().cpu() - want).abs().max() < tol, name
    for splits in (1, 2):
        for k in (n - 1, n - 2):                            # the row that must not see key 330, and one that does
            out1 = torch.full((1, q_heads * hd), 55.0, dtype=dtype, device=DEV)
            o.attention_decode_bf16(q[k:k + 1].contiguous(), out1, view, slots[k:k + 1].contiguous(),
                                    pos[k:k + 1].contiguous(), 1, q_heads, scale, window, splits, None)
            assert (out1.double().cpu() - want[k:k + 1]).abs().max() < tol, f"decode kernel, {splits} splits, row {k}"
