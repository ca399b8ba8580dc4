"""GPU: a device-side wait that runs out is reported, once, by the next call
that synchronises, and the context stays usable.

The wait is made to run out without any fault: a two-rank exchange whose two
objects live in this process on one device; only rank 0 ever runs its step, so
rank 1's flag is never set and rank 0's kernel gives up after the context's
(shortened) wait limit, records its error word and returns.  What must hold
afterwards is the reference's "a failed step is reported and consumes nothing"
(src/core/session.c:160-168, :589-592): wr_cuda_ctx_sync — and equally the next
call with host buffers — returns WR_ERR_INTERNAL exactly once, and the next
ordinary call gives the right answer.
"""
import numpy as np
import pytest

import _gen
from _cuda_util import TOL, decode, make_cache, port

pytestmark = pytest.mark.gpu

SHORT = 200_000          # cycles: about 0.1 ms
HQ, HKV, HD = 8, 2, 128


def _setup():
    import torch
    import wayruntime_b200 as wr
    ctx = wr.Context(0)
    P = port()
    n = 300
    k = P.f32_to_f16(_gen.normal(501, (n, HKV, HD)))
    v = P.f32_to_f16(_gen.normal(502, (n, HKV, HD)))
    q = _gen.normal(503, (1, HQ, HD))
    kv = make_cache(ctx, k, v)
    rc, want = P.attention(q, k, v)
    assert rc == 0
    rows = HQ
    xs = [wr.Exchange(ctx, 2, r, rows, HD) for r in range(2)]
    wr.Exchange.connect_local(xs)
    triples = torch.zeros((rows, 4 + HD), dtype=torch.float32, device="cuda")
    out = torch.zeros((rows, HD), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    return wr, ctx, kv, q, want, xs, triples, out, n


def _time_out_one_step(ctx, xs, triples, out):
    ctx.set_wait_limit(SHORT)
    xs[0].combine(triples.shape[0], triples, out)      # rank 1 never answers
    ctx.set_wait_limit(4_000_000_000)                   # later kernels get the default again


def _teardown(ctx, kv, xs):
    for x in xs:
        x.close()
    kv.close()
    ctx.close()


def test_ctx_sync_reports_the_give_up_once_and_the_context_survives():
    wr, ctx, kv, q, want, xs, triples, out, n = _setup()
    _time_out_one_step(ctx, xs, triples, out)
    with pytest.raises(wr.WrCudaError) as e:
        ctx.sync()
    assert e.value.status == -10
    ctx.sync()                                          # reported once, then clear
    got = decode(ctx, [kv], [n], q, HQ)
    assert np.abs(got - want).max() <= TOL
    _teardown(ctx, kv, xs)


def test_host_buffer_call_reports_the_give_up():
    wr, ctx, kv, q, want, xs, triples, out, n = _setup()
    _time_out_one_step(ctx, xs, triples, out)
    with pytest.raises(wr.WrCudaError) as e:
        decode(ctx, [kv], [n], q, HQ)                   # host buffers: the call synchronises
    assert e.value.status == -10
    got = decode(ctx, [kv], [n], q, HQ)                 # the next one is an ordinary success
    assert np.abs(got - want).max() <= TOL
    ctx.sync()
    _teardown(ctx, kv, xs)


def test_both_ranks_in_one_process_still_merge():
    """The in-process connection itself: with both ranks stepping, the merge of
    the two ranks' triples is the reference merge."""
    import torch
    from wayruntime_b200 import splitkv
    wr, ctx, kv, q, want, xs, triples, out, n = _setup()
    rng = np.random.default_rng(5)
    t = [rng.standard_normal((HQ, 4 + HD)).astype(np.float32) for _ in range(2)]
    for a in t:
        a[:, 1] = np.abs(a[:, 1]) + 0.5
        a[:, 2:4] = 0
    outs = [torch.zeros((HQ, HD), dtype=torch.float32, device="cuda") for _ in range(2)]
    devs = [torch.from_numpy(a).cuda() for a in t]
    # rank 1 first: its kernel stores, flags and then waits for rank 0, whose kernel is
    # next in the same stream — so rank 1 gives up and only rank 0 sees both flags
    ctx.set_wait_limit(SHORT)
    xs[1].combine(HQ, devs[1], outs[1])
    ctx.set_wait_limit(4_000_000_000)
    xs[0].combine(HQ, devs[0], outs[0])
    with pytest.raises(wr.WrCudaError):
        ctx.sync()                                      # rank 1's give-up
    ref = splitkv.merge_triples_reference(np.stack(t))
    assert np.abs(outs[0].cpu().numpy() - ref).max() <= 1e-5
    _teardown(ctx, kv, xs)


def test_wait_limit_argument_is_checked():
    import wayruntime_b200 as wr
    ctx = wr.Context(0)
    with pytest.raises(wr.WrCudaError) as e:
        ctx.set_wait_limit(0)
    assert e.value.status == -4
    ctx.close()


@pytest.mark.parametrize("world", [4, 8])
def test_in_kernel_receive_over_a_world_of_local_ranks(world):
    """Key-sharded decode with the receive fused into the decode kernel, for 4 and 8
    ranks whose exchange objects live in this process on one device.  Ranks cannot
    wait for each other here (their kernels run one after another), so ranks
    1 .. world-1 step first with a short wait limit: each delivers its rows and flags
    to every rank's buffer, then gives up waiting for the ranks that have not run yet —
    reported as WR_ERR_INTERNAL, nothing faults.  Rank 0 steps last, finds every
    rank's rows, and must produce the bits of wr_cuda_attn_decode_partial per shard +
    wr_cuda_attn_combine."""
    import torch
    import wayruntime_b200 as wr
    ctx = wr.Context(0, attn_max_seq=65536)
    P = port()
    hq, hkv, hd, n_sess, shard = 8, 2, HD, 3, 640            # 10 tiles per shard: several chunks, so merge warps carry the rows
    rows = n_sess * hq
    q = torch.from_numpy(_gen.normal(4000, (n_sess, hq, hd))).cuda()
    shards, triples = [], []
    for r in range(world):
        kvs = []
        for s in range(n_sess):
            k = P.f32_to_f16(_gen.normal(4100 + 10 * r + s, (shard, hkv, hd)))
            v = P.f32_to_f16(_gen.normal(4500 + 10 * r + s, (shard, hkv, hd)))
            kvs.append(make_cache(ctx, k, v))
        t = torch.empty((rows, wr.TRIPLE_PAD + hd), dtype=torch.float32, device="cuda")
        ctx.attn_decode_partial(kvs, 0, [shard] * n_sess, q, t, hq)
        shards.append(kvs)
        triples.append(t)
    want = torch.empty((rows, hd), dtype=torch.float32, device="cuda")
    ctx.attn_combine(world, rows, hd, torch.stack(triples).contiguous(), want)
    ctx.sync()
    xs = [wr.Exchange(ctx, world, r, rows, hd) for r in range(world)]
    wr.Exchange.connect_local(xs)
    for r in range(1, world):
        out = torch.empty((n_sess, hq, hd), dtype=torch.float32, device="cuda")
        ctx.set_wait_limit(SHORT)
        xs[r].decode(shards[r], 0, [shard] * n_sess, q, out, hq)
        ctx.set_wait_limit(4_000_000_000)
        with pytest.raises(wr.WrCudaError) as e:
            ctx.sync()                                          # the ranks it waited for have not run
        assert e.value.status == -10
    got = torch.full((n_sess, hq, hd), float("nan"), dtype=torch.float32, device="cuda")
    xs[0].decode(shards[0], 0, [shard] * n_sess, q, got, hq)
    ctx.sync()
    assert torch.equal(got.view(rows, hd), want)
    for x in xs:
        x.close()
    for kvs in shards:
        for kv in kvs:
            kv.close()
    ctx.close()
