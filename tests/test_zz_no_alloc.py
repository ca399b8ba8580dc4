"""GPU: the allocation-free decode entry point (wr_cuda_attn_decode_static).

Some callers of this library may not allocate once they are serving: their
device memory is fully committed to the KV pool, or the step runs on a thread
that must stay out of the CUDA allocator.  For them the library carries its
split-KV scratch inside its own image.  This test drives that entry point
through the C-ABI twice in a row on the same inputs and checks each result
against the regular entry point (wr_cuda_attn_decode) within the tolerance the
other decode tests use; the second call proves that what the first call left
in the shared scratch array does no harm.  It also checks that a call too large
for the fixed array is refused with WR_ERR_LIMIT instead of overrunning it.

Collected last on purpose (file name): a run that stops at the first failure
has then already run every other test.
"""
import numpy as np
import pytest

import _gen
from _cuda_util import TOL, make_cache, port

pytestmark = pytest.mark.gpu


def test_static_scratch_decode_matches_regular_entry_point_twice():
    import torch
    import wayruntime_b200 as wr
    ctx = wr.Context(0, attn_max_seq=32768)
    P = port()
    hq, hkv, hd = 32, 8, 128
    lens = [1500, 64, 4096, 333, 1, 2049]
    ks = [P.f32_to_f16(_gen.normal(3000 + 2 * i, (n, hkv, hd))) for i, n in enumerate(lens)]
    vs = [P.f32_to_f16(_gen.normal(3001 + 2 * i, (n, hkv, hd))) for i, n in enumerate(lens)]
    kvs = [make_cache(ctx, k, v) for k, v in zip(ks, vs)]
    q = torch.from_numpy(_gen.normal(3999, (len(lens), hq, hd))).cuda()
    want = torch.empty_like(q)
    ctx.attn_decode(kvs, 0, lens, q, want, hq)
    ctx.sync()
    want = want.cpu().numpy()
    rc, ref = P.decode_batch(q.cpu().numpy(), ks, vs, threads=6)
    assert rc == 0 and np.abs(want - ref).max() <= TOL          # the yardstick itself is sound
    for call in range(2):
        got = torch.full_like(q, float("nan"))
        ctx.attn_decode_static(kvs, 0, lens, q, got, hq)
        ctx.sync()
        got = got.cpu().numpy()
        assert np.isfinite(got).all(), f"call {call}"
        assert np.abs(got - want).max() <= TOL, f"call {call}"
    # windowed and scale-override variants go through the same scratch
    for window, scale in ((100, 0.0), (0, 0.05)):
        a = torch.empty_like(q)
        b = torch.empty_like(q)
        ctx.attn_decode(kvs, 0, lens, q, a, hq, scale=scale, window=window)
        ctx.attn_decode_static(kvs, 0, lens, q, b, hq, scale=scale, window=window)
        ctx.sync()
        assert np.abs(a.cpu().numpy() - b.cpu().numpy()).max() <= TOL
    for kv in kvs:
        kv.close()
    ctx.close()


def test_static_scratch_decode_refuses_what_does_not_fit():
    import torch
    import wayruntime_b200 as wr
    ctx = wr.Context(0, attn_max_seq=32768)
    # 16 sessions x 32 kv heads x 16 chunks = 8192 work items > WR_CUDA_STATIC_MAX_ITEMS (4096)
    kvs = [ctx.kv_create(1, 32, 128, 4096) for _ in range(16)]
    q = torch.zeros((16, 32, 128), device="cuda")
    out = torch.zeros_like(q)
    with pytest.raises(wr.WrCudaError) as e:
        ctx.attn_decode_static(kvs, 0, [4096] * 16, q, out, 32)
    assert e.value.status == -8
    ctx.attn_decode_static(kvs, 0, [1024] * 16, q, out, 32)       # 16*32*8 = 4096 items: fits
    ctx.sync()
    kv64 = ctx.kv_create(1, 2, 64, 64)
    q64 = torch.zeros((1, 2, 64), device="cuda")
    with pytest.raises(wr.WrCudaError) as e:
        ctx.attn_decode_static([kv64], 0, [10], q64, torch.zeros_like(q64), 2)
    assert e.value.status == -3                                   # head_dim 128 only
    with pytest.raises(ValueError):
        ctx.attn_decode_static(kvs[:1], 0, [10], np.zeros((1, 32, 128), np.float32),
                               np.zeros((1, 32, 128), np.float32), 32)   # host buffers not accepted
    # straight through the C-ABI: a pageable host pointer is refused by the library
    # itself (pointer-attribute query, no launch), not only by the Python mirror
    import ctypes as C
    host_q = np.zeros((1, 32, 128), np.float32)
    host_o = np.zeros((1, 32, 128), np.float32)
    handles = (C.c_void_p * 1)(kvs[0]._h)
    lens = (C.c_uint32 * 1)(10)
    rc = ctx._lib.wr_cuda_attn_decode_static(ctx._h, 1, handles, 0, lens, host_q.ctypes.data,
                                             host_o.ctypes.data, 32, 0.0, 0)
    assert rc == -4
    kv64.close()
    for kv in kvs:
        kv.close()
    ctx.close()


def test_static_scratch_is_resident_after_context_creation():
    """The scratch array is instantiated when the context is created, so the
    first call of the entry point takes no device memory: a caller may size its
    KV pool from the free memory it sees after wr_cuda_ctx_create."""
    import torch
    import wayruntime_b200 as wr
    ctx = wr.Context(0)
    kv = ctx.kv_create(1, 8, 128, 256)
    q = torch.zeros((1, 32, 128), device="cuda")
    out = torch.zeros_like(q)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    ctx.attn_decode_static([kv], 0, [200], q, out, 32)
    ctx.sync()
    free_after, _ = torch.cuda.mem_get_info()
    # (the 17 MB array would show; a first launch may still grow the driver's small per-kernel state)
    assert free_before - free_after < 8 * 1024 * 1024
    kv.close()
    ctx.close()
