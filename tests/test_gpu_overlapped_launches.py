"""GPU: steps enqueued back to back give the bits they give one at a time.

The append and decode kernels are launched so that each may be scheduled, run
its prologue and even request its first K/V tiles while the kernel before it is
still finishing (programmatic dependent launch); everything that could race is
ordered by a wait inside the kernel.  The reference has no such overlap — its
ops run one after another on the calling thread (src/core/session.c:441-496) —
so the contract to keep is simply that a step's result does not depend on what
else is in flight: 24 layer-steps of a 16-session batch (a grid that covers the
whole device, which is what enables the early tile requests) are enqueued
without any synchronisation between them, on rotating layers, and every step's
attention rows and appended cache rows must equal, bit for bit, those of the
same step enqueued alone with a synchronisation before and after.  A second
pass does the same for back-to-back plain decode launches.
"""
import numpy as np
import pytest

import _gen
from _cuda_util import TOL, port

pytestmark = pytest.mark.gpu

HQ, HKV, HD, LAYERS, THETA = 32, 8, 128, 3, 5e5
LENS = [700, 64, 1, 2049, 333, 129, 1500, 65, 1024, 2, 900, 127, 128, 640, 1999, 77]


def _setup(ctx, torch):
    P = port()
    kvs = [ctx.kv_create(LAYERS, HKV, HD, 2304) for _ in LENS]
    for i, (kv, n) in enumerate(zip(kvs, LENS)):
        for layer in range(LAYERS):
            if n > 1:
                kv.write_rows(layer, 0, 0, P.f32_to_f16(_gen.normal(7000 + 10 * i + layer, (n - 1, HKV, HD))))
                kv.write_rows(layer, 1, 0, P.f32_to_f16(_gen.normal(8000 + 10 * i + layer, (n - 1, HKV, HD))))
    return kvs


def _inputs(torch, step):
    n = len(LENS)
    q = torch.from_numpy(_gen.normal(9000 + step, (n, HQ, HD))).cuda()
    k = torch.from_numpy(_gen.normal(9100 + step, (n, HKV, HD))).cuda()
    v = torch.from_numpy(_gen.normal(9200 + step, (n, HKV, HD))).cuda()
    return q, k, v


def test_steps_in_flight_together_match_steps_run_alone():
    import torch
    import wayruntime_b200 as wr
    ctx = wr.Context(0)
    steps = 24
    # the position of a session advances every time its layer comes round again
    pos_of = lambda step: [n - 1 + step // LAYERS for n in LENS]
    results = {}
    for mode in ("alone", "together"):
        kvs = _setup(ctx, torch)
        outs, ins = [], []
        for step in range(steps):
            q, k, v = _inputs(torch, step)
            out = torch.full((len(LENS), HQ, HD), float("nan"), device="cuda")
            ins.append((q, k, v))
            outs.append(out)
        torch.cuda.synchronize()
        for step in range(steps):
            q, k, v = ins[step]
            if mode == "alone":
                ctx.sync()
            ctx.decode_step(kvs, step % LAYERS, pos_of(step), q, k, v, outs[step], HQ, theta=THETA)
            if mode == "alone":
                ctx.sync()
        ctx.sync()
        rows = [[(kv.read_rows(layer, 0, n - 1, steps // LAYERS), kv.read_rows(layer, 1, n - 1, steps // LAYERS))
                 for layer in range(LAYERS)] for kv, n in zip(kvs, LENS)]
        results[mode] = ([o.cpu().numpy() for o in outs], rows, [q.cpu().numpy() for q, _, _ in ins])
        for kv in kvs:
            kv.close()
    a, b = results["alone"], results["together"]
    for step in range(steps):
        assert np.isfinite(b[0][step]).all(), step
        assert np.array_equal(a[0][step].view(np.uint32), b[0][step].view(np.uint32)), step
        assert np.array_equal(a[2][step].view(np.uint32), b[2][step].view(np.uint32)), step     # rotated q rows
    for ra, rb in zip(a[1], b[1]):
        for (ka, va), (kb, vb) in zip(ra, rb):
            assert np.array_equal(ka, kb) and np.array_equal(va, vb)
    # and the steps are right, not only equal: the last one against the CPU reference
    P = port()
    kvs = _setup(ctx, torch)
    for step in range(steps):
        q, k, v = _inputs(torch, step)
        out = torch.empty((len(LENS), HQ, HD), device="cuda")
        ctx.decode_step(kvs, step % LAYERS, pos_of(step), q, k, v, out, HQ, theta=THETA)
    ctx.sync()
    layer, lens = (steps - 1) % LAYERS, [p + 1 for p in pos_of(steps - 1)]
    ks = [kv.read_rows(layer, 0, 0, n) for kv, n in zip(kvs, lens)]
    vs = [kv.read_rows(layer, 1, 0, n) for kv, n in zip(kvs, lens)]
    rc, ref = P.decode_batch(q.cpu().numpy(), ks, vs, threads=8)
    assert rc == 0 and np.abs(out.cpu().numpy() - ref).max() <= TOL
    for kv in kvs:
        kv.close()
    ctx.close()


def test_back_to_back_decode_launches_match_single_launches():
    import torch
    import wayruntime_b200 as wr
    ctx = wr.Context(0)
    kvs = _setup(ctx, torch)
    q = torch.from_numpy(_gen.normal(9999, (len(LENS), HQ, HD))).cuda()
    alone = []
    for layer in range(LAYERS):
        out = torch.empty_like(q)
        ctx.sync()
        ctx.attn_decode(kvs, layer, LENS, q, out, HQ)
        ctx.sync()
        alone.append(out.cpu().numpy())
    outs = [torch.full_like(q, float("nan")) for _ in range(4 * LAYERS)]
    for i, out in enumerate(outs):
        ctx.attn_decode(kvs, i % LAYERS, LENS, q, out, HQ)       # no synchronisation in between
    ctx.sync()
    for i, out in enumerate(outs):
        assert np.array_equal(out.cpu().numpy().view(np.uint32), alone[i % LAYERS].view(np.uint32)), i
    for kv in kvs:
        kv.close()
    ctx.close()


def test_back_to_back_prefill_launches_match_single_launches():
    """Prefill launches given F16 queries, one after another with nothing in between: the
    later one starts its first tiles while the earlier one drains.  Same bits as alone."""
    import torch
    import wayruntime_b200 as wr
    ctx = wr.Context(0)
    P = port()
    n, hq, hkv = 2048 + 77, 32, 8                        # 17 row tiles x 16 head pairs: more tiles than SMs
    kvs = []
    for i in range(2):
        kv = ctx.kv_create(1, hkv, HD, n)
        kv.write_rows(0, 0, 0, P.f32_to_f16(_gen.normal(7700 + i, (n, hkv, HD))))
        kv.write_rows(0, 1, 0, P.f32_to_f16(_gen.normal(7800 + i, (n, hkv, HD))))
        kvs.append(kv)
    qs = [torch.from_numpy(P.f32_to_f16(_gen.normal(7900 + i, (n, hq, HD))).view(np.int16)).cuda() for i in range(2)]
    alone = []
    for kv, q in zip(kvs, qs):
        out = torch.empty((n, hq, HD), device="cuda")
        ctx.sync()
        ctx.attn_prefill(kv, 0, 0, n, q.view(torch.float16), out, hq)
        ctx.sync()
        alone.append(out.cpu().numpy())
    outs = [torch.full((n, hq, HD), float("nan"), device="cuda") for _ in range(6)]
    for i, out in enumerate(outs):
        ctx.attn_prefill(kvs[i % 2], 0, 0, n, qs[i % 2].view(torch.float16), out, hq)
    ctx.sync()
    for i, out in enumerate(outs):
        got = out.cpu().numpy()
        assert np.isfinite(got).all(), i
        assert np.array_equal(got.view(np.uint32), alone[i % 2].view(np.uint32)), i
    for kv in kvs:
        kv.close()
    ctx.close()
