"""The entry point that allocates nothing (x0ne_attention_decode_bf16_noalloc), called through its
exported C symbol as a caller without an allocator would call it, and compared with the ordinary
decode-attention entry point on two calls in a row.

It is for callers that cannot allocate device memory when they need attention: a runtime that has
frozen its one device arena, code inside another process's memory budget, a serving loop that must
not take cudaMalloc's device-wide synchronisation.  The library carries the scratch for the split
partial results itself (4 MiB per GPU, held until exit), so the second call finds what the first one
left there; both calls must still give the ordinary entry point's result.  This file is collected last
so that a run which stops at the first failure has run every other test before it.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BF16_EPS = 2.0 ** -7      # the tolerance the kernel tests use for bfloat16 attention


def _setup(n, q_heads, kv_heads, hd, ctxs, seed):
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(seed)
    pages_per = (max(ctxs) + 63) // 64
    n_pages = n * pages_per
    storage = torch.randn((n_pages, 2, kv_heads, 64, hd), generator=g).bfloat16().to(DEV)
    perm = torch.randperm(n_pages, generator=g).to(torch.int32).reshape(n, pages_per).contiguous().to(DEV)
    view = ops.PagedCacheArg(storage.data_ptr(), perm.data_ptr(), 2 * kv_heads * 64 * hd, pages_per, pages_per, 64,
                             kv_heads, hd, n_pages)
    q = torch.randn((n, q_heads * hd), generator=g).bfloat16().to(DEV)
    slots = torch.arange(n, dtype=torch.int32, device=DEV)
    pos = torch.tensor([c - 1 for c in ctxs], dtype=torch.int32, device=DEV)
    return ops, storage, perm, view, q, slots, pos


def test_noalloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from x0ne_engine_b200.csrc import build
    lib = ctypes.CDLL(build.build("noalloc"))
    lib.x0ne_last_error.restype = ctypes.c_char_p
    lib.x0ne_noalloc_scratch_capacity.restype = ctypes.c_int64
    assert lib.x0ne_noalloc_scratch_capacity() == 4 << 20
    fn = lib.x0ne_attention_decode_bf16_noalloc
    torch.cuda.set_device(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    # two different problems, so the second call meets the first one's leftovers in the scratch
    cases = [dict(n=5, q_heads=8, kv_heads=2, hd=64, ctxs=[300, 64, 1, 129, 513], splits=4, seed=1),
             dict(n=3, q_heads=6, kv_heads=2, hd=32, ctxs=[700, 65, 200], splits=7, seed=2)]
    # The first call on a device loads the library's code and its scratch array onto the GPU (the
    # driver does that at a kernel's first use) and looks the array's address up.  The third call
    # repeats the first problem, so nothing is left to load: the device's free memory must not move.
    for call, c in enumerate(cases + cases[:1]):
        ops, storage, table, view, q, slots, pos = _setup(c["n"], c["q_heads"], c["kv_heads"], c["hd"], c["ctxs"], c["seed"])
        scale = 1 / math.sqrt(c["hd"])
        want = torch.empty_like(q)
        scratch = torch.zeros(ops.attention_decode_scratch_bytes(c["n"], c["q_heads"], c["kv_heads"], c["hd"], c["splits"]),
                              dtype=torch.uint8, device=DEV)
        ops.attention_decode_bf16(q, want, view, slots, pos, c["n"], c["q_heads"], scale, 0, c["splits"], scratch)
        got = torch.full_like(q, 55.0)
        torch.cuda.synchronize()
        # Free device memory as the driver counts it: an allocation by anyone in this process, through
        # torch's allocator or past it, would lower it.
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        rc = fn(ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(got.data_ptr()), view,
                ctypes.c_void_p(slots.data_ptr()), ctypes.c_void_p(pos.data_ptr()), ctypes.c_int(c["n"]),
                ctypes.c_int(c["q_heads"]), ctypes.c_float(scale), ctypes.c_int(0), ctypes.c_int(c["splits"]), stream)
        assert rc == 0, lib.x0ne_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if call == 2:
            assert torch.cuda.mem_get_info()[0] >= free_before, "the entry point took device memory"
        vmax = float(storage.float().abs().max())
        assert (got.float() - want.float()).abs().max() / vmax < BF16_EPS
        assert torch.equal(got, want)            # same kernel, same order of the splits: the same bits


def test_noalloc_entry_point_refuses_what_does_not_fit():
    from x0ne_engine_b200.csrc import build
    lib = ctypes.CDLL(build.build("noalloc"))
    lib.x0ne_last_error.restype = ctypes.c_char_p
    ops, storage, table, view, q, slots, pos = _setup(64, 32, 8, 128, [100] * 64, 3)
    out = torch.zeros_like(q)
    rc = lib.x0ne_attention_decode_bf16_noalloc(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(out.data_ptr()), view, ctypes.c_void_p(slots.data_ptr()),
        ctypes.c_void_p(pos.data_ptr()), ctypes.c_int(64), ctypes.c_int(32), ctypes.c_float(0.1), ctypes.c_int(0),
        ctypes.c_int(16), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0 and b"scratch" in lib.x0ne_last_error()
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0
