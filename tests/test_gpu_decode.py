"""GPU parity: batched split-KV decode attention (wr_cuda_attn_decode).

Bar: max-abs error <= 2e-3 against the reference CPU attention
(src/core/kernels.c:1414-1527) on the same seeded inputs; bit-identical
between a batched call and per-session calls.
"""
import os
import sys

import numpy as np
import pytest

import _gen
from _cuda_util import TOL, decode, make_cache, port

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import cases  # noqa: E402

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden",
                            "reference_outputs.npz"))


@pytest.fixture(scope="module")
def ctx():
    import wayruntime_b200 as wr
    c = wr.Context(0, attn_max_seq=32768)
    yield c
    c.close()


@pytest.mark.parametrize("c", cases.ATTN_CASES, ids=lambda c: c["name"])
def test_decode_matches_reference_fixture(ctx, c):
    """Every golden attention case; seq_q > 1 rows run as separate sessions
    over identical caches.  F32-K/V cases are stored through the truncating
    convert (the device cache is F16 by design) and compared with the oracle
    on those same F16 rows; F16 cases compare with the committed reference
    output directly."""
    P = port()
    q, k, v = cases.attn_inputs(c, cases.case_seed(c["name"]))
    k16, v16 = P.f32_to_f16(k), P.f32_to_f16(v)
    if c["kv"] == "f16":
        want = GOLD[f"attn/{c['name']}"]
    else:
        rc, want = P.attention(q, k16, v16, seq_k=c["ctx"], scale=c.get("scale", 0.0),
                               window=c.get("window", 0))
        assert rc == 0
        # sanity: the F16 rounding of these small fixtures stays near the F32 golden
        assert np.abs(want - GOLD[f"attn/{c['name']}"]).max() < 5e-3
    kvs = [make_cache(ctx, k16, v16) for _ in range(c["sq"])]
    out = decode(ctx, kvs, [c["ctx"]] * c["sq"], q, c["hq"], scale=c.get("scale", 0.0),
                 window=c.get("window", 0))
    assert np.abs(out - want).max() <= TOL
    for kv in kvs:
        kv.close()


def _ragged_batch(ctx, lens, hq, hkv, hd, seed):
    P = port()
    ks = [P.f32_to_f16(_gen.normal(seed + 2 * i, (n, hkv, hd))) for i, n in enumerate(lens)]
    vs = [P.f32_to_f16(_gen.normal(seed + 2 * i + 1, (n, hkv, hd))) for i, n in enumerate(lens)]
    kvs = [make_cache(ctx, k, v) for k, v in zip(ks, vs)]
    q = _gen.normal(seed + 999, (len(lens), hq, hd))
    return q, ks, vs, kvs


@pytest.mark.parametrize("hq,hkv", [(32, 8), (16, 8), (40, 8), (8, 8), (16, 1), (12, 1)])
def test_decode_ragged_batch_group_sizes(ctx, hq, hkv):
    """Group sizes 1, 2, 4, 5, 12 and 16 (the last two need two q-head subgroups)."""
    lens = [1, 2, 15, 16, 17, 63, 64, 65, 127, 255, 256, 257, 300, 511, 1024, 1500]
    q, ks, vs, kvs = _ragged_batch(ctx, lens, hq, hkv, 128, 40)
    out = decode(ctx, kvs, lens, q, hq)
    rc, want = port().decode_batch(q, ks, vs, threads=8)
    assert rc == 0
    assert np.abs(out - want).max() <= TOL
    for kv in kvs:
        kv.close()


def test_decode_more_merge_jobs_than_merge_warps(ctx):
    """16 sessions x 32 KV heads, every one split into chunks: 512 groups, i.e.
    more (group, head pair) merge jobs than the grid has merge warps, so that
    each merge warp has to work through several of them in turn."""
    lens = [600 + 37 * i for i in range(16)]
    q, ks, vs, kvs = _ragged_batch(ctx, lens, 64, 32, 128, 333)
    out = decode(ctx, kvs, lens, q, 64)
    rc, want = port().decode_batch(q, ks, vs, threads=8)
    assert rc == 0
    assert np.abs(out - want).max() <= TOL
    again = decode(ctx, kvs, lens, q, 64)                   # counters were left ready for the next launch
    assert np.array_equal(again.view(np.uint32), out.view(np.uint32))
    for kv in kvs:
        kv.close()


def test_decode_full_length_sessions(ctx):
    """Llama-3-8B geometry at the config's longest context (4096) and the
    seed-uniform lengths in between; 16 sessions in one grid."""
    lens = [int(x) for x in _gen.randint(7, 1024, 4096, (16,))]
    lens[0], lens[1] = 4096, 1024
    q, ks, vs, kvs = _ragged_batch(ctx, lens, 32, 8, 128, 80)
    out = decode(ctx, kvs, lens, q, 32)
    rc, want = port().decode_batch(q, ks, vs, threads=8)
    assert rc == 0
    err = np.abs(out - want).max()
    assert err <= TOL
    # batched == per-session, bit for bit (src/core/batch.c:257-390 contract)
    for i in (0, 1, 5, 15):
        solo = decode(ctx, [kvs[i]], [lens[i]], q[i:i + 1], 32)
        assert np.array_equal(solo[0].view(np.uint32), out[i].view(np.uint32))
    # ...and independent of batch order / composition
    perm = [3, 0, 9]
    sub = decode(ctx, [kvs[i] for i in perm], [lens[i] for i in perm], q[perm], 32)
    for j, i in enumerate(perm):
        assert np.array_equal(sub[j].view(np.uint32), out[i].view(np.uint32))
    for kv in kvs:
        kv.close()


def test_decode_long_context(ctx):
    """32768 keys (needs the raised cap): chunks of more than four tiles."""
    P = port()
    n = 32768
    k = P.f32_to_f16(_gen.normal(301, (n, 2, 128)))
    v = P.f32_to_f16(_gen.normal(302, (n, 2, 128)))
    kv = make_cache(ctx, k, v)
    q = _gen.normal(303, (1, 8, 128))
    for ln in (n, n - 37, 20000):
        out = decode(ctx, [kv], [ln], q, 8)
        rc, want = P.attention(q, k, v, seq_k=ln, max_seq=32768)
        assert rc == 0
        assert np.abs(out - want).max() <= TOL
    kv.close()


def test_decode_window_and_scale(ctx):
    lens = [300, 64, 129, 1000]
    q, ks, vs, kvs = _ragged_batch(ctx, lens, 32, 8, 128, 120)
    P = port()
    for window, scale in ((100, 0.0), (64, 0.0), (1, 0.0), (5000, 0.0), (0, 0.05), (77, 0.125)):
        out = decode(ctx, kvs, lens, q, 32, scale=scale, window=window)
        rc, want = P.decode_batch(q, ks, vs, scale=scale, window=window, threads=4)
        assert rc == 0
        assert np.abs(out - want).max() <= TOL, (window, scale)
    for kv in kvs:
        kv.close()


def test_decode_other_head_dims(ctx):
    """head_dim 64, 8 and 256 go through the generic kernel."""
    P = port()
    for hd, hq, hkv in ((64, 8, 4), (8, 2, 1), (256, 4, 2), (2, 4, 2)):
        lens = [1, 70, 200]
        q, ks, vs, kvs = _ragged_batch(ctx, lens, hq, hkv, hd, 160 + hd)
        out = decode(ctx, kvs, lens, q, hq)
        rc, want = P.decode_batch(q, ks, vs, threads=3)
        assert rc == 0
        assert np.abs(out - want).max() <= TOL, hd
        out = decode(ctx, kvs, lens, q, hq, window=50)
        rc, want = P.decode_batch(q, ks, vs, window=50, threads=3)
        assert np.abs(out - want).max() <= TOL, hd
        for kv in kvs:
            kv.close()


def test_decode_ignores_uncommitted_rows(ctx):
    """Rollback (src/core/session.c:160-168) = the host not advancing seq_len:
    a row appended past seq_len — even one holding inf — must not change or
    poison the result."""
    P = port()
    n = 100
    k = P.f32_to_f16(_gen.normal(201, (n, 8, 128)))
    v = P.f32_to_f16(_gen.normal(202, (n, 8, 128)))
    kv = make_cache(ctx, k, v, max_ctx=256)
    q = _gen.normal(203, (1, 32, 128))
    before = decode(ctx, [kv], [n], q, 32)
    bad = np.full((1, 8, 128), 1e9, np.float32)     # truncates to +inf
    ctx.kv_append([kv], 0, [n], bad, bad, rope=False)
    after = decode(ctx, [kv], [n], q, 32)
    assert np.isfinite(after).all()
    assert np.array_equal(before.view(np.uint32), after.view(np.uint32))
    kv.close()


def test_decode_refusals(ctx):
    """kernels.c:1418-1454 and batch.c:128-137."""
    import wayruntime_b200 as wr
    kv = ctx.kv_create(1, 8, 128, 128)
    q = np.zeros((1, 32, 128), np.float32)
    out = np.zeros_like(q)

    def status(fn):
        with pytest.raises(wr.WrCudaError) as e:
            fn()
        return e.value.status

    assert status(lambda: ctx.attn_decode([kv], 0, [0], q, out, 32)) == -4      # seq_k == 0
    assert status(lambda: ctx.attn_decode([kv], 0, [129], q, out, 32)) == -4    # beyond capacity
    assert status(lambda: ctx.attn_decode([kv], 0, [64], q, out, 12)) == -4     # 12 % 8 != 0
    assert status(lambda: ctx.attn_decode([kv], 1, [64], q, out, 32)) == -4     # layer
    c2 = wr.Context(0)   # default cap 4096 (internal.h:186)
    c2.set_attn_max_seq(8192)
    big = c2.kv_create(1, 1, 128, 8192)
    c2.set_attn_max_seq(4096)
    q1 = np.zeros((1, 1, 128), np.float32)
    o1 = np.zeros_like(q1)
    assert status(lambda: c2.attn_decode([big], 0, [4097], q1, o1, 1)) == -8    # over the cap
    c2.attn_decode([big], 0, [4096], q1, o1, 1)
    big.close()
    many = [c2.kv_create(1, 1, 128, 64) for _ in range(17)]
    q17 = np.zeros((17, 1, 128), np.float32)
    assert status(lambda: c2.attn_decode(many, 0, [1] * 17, q17, np.zeros_like(q17), 1)) == -8
    for m in many:
        m.close()
    c2.close()
    kv.close()


def test_split_kv_partials_and_combine(ctx):
    """Keys sharded over G caches (stand-ins for G devices): per-shard triples
    merged by wr_cuda_attn_combine equal the unsharded attention."""
    import wayruntime_b200 as wr
    P = port()
    hq, hkv, hd = 32, 8, 128
    lens = [2048, 777, 5]      # the 5-key session leaves shards empty at G = 8
    q, ks, vs, kvs_full = _ragged_batch(ctx, lens, hq, hkv, hd, 500)
    rc, want = P.decode_batch(q, ks, vs, threads=3)
    for G in (1, 2, 4, 8):
        shard_kvs, shard_lens = [], []
        for g in range(G):
            row, ln = [], []
            for k, v, n in zip(ks, vs, lens):
                per = (n + G - 1) // G
                lo, hi = min(g * per, n), min((g + 1) * per, n)
                row.append(make_cache(ctx, k[lo:hi], v[lo:hi], max_ctx=max(hi - lo, 1)))
                ln.append(hi - lo)
            shard_kvs.append(row), shard_lens.append(ln)
        triples = np.zeros((G, len(lens), hq, wr.TRIPLE_PAD + hd), np.float32)
        for g in range(G):
            ctx.attn_decode_partial(shard_kvs[g], 0, shard_lens[g], q, triples[g], hq)
        out = np.zeros((len(lens) * hq, hd), np.float32)
        ctx.attn_combine(G, len(lens) * hq, hd, triples, out)
        assert np.abs(out.reshape(want.shape) - want).max() <= TOL, G
        if G == 2:   # the triple itself matches the oracle's shard state
            per = (lens[0] + 1) // 2
            rc, m, l, o = P.partial(q[0], ks[0], vs[0], 0, per)
            t = triples[0, 0]
            w = np.exp(m - t[:, 0])
            assert np.abs(t[:, 1] - w * l).max() <= 1e-3 * np.abs(l).max()
            assert np.abs(t[:, wr.TRIPLE_PAD:] - w[:, None] * o).max() <= TOL
        for row in shard_kvs:
            for kv in row:
                kv.close()
    for kv in kvs_full:
        kv.close()


def test_exchange_single_rank_and_refusals(ctx):
    """The fused exchange + merge kernel with a world of one is the merge of one
    shard: it must reproduce wr_cuda_attn_combine bit for bit, on both buffer
    parities.  (Two ranks over NVLink: tests/test_gpu_multi.py.)"""
    import torch
    import wayruntime_b200 as wr
    hq, hkv, hd = 8, 2, 128
    lens = [300, 64, 1]
    q, ks, vs, kvs = _ragged_batch(ctx, lens, hq, hkv, hd, 900)
    rows = len(lens) * hq
    qd = torch.from_numpy(q).cuda()
    triples = torch.empty((rows, wr.TRIPLE_PAD + hd), dtype=torch.float32, device="cuda")
    ctx.attn_decode_partial(kvs, 0, lens, qd, triples, hq)
    want = torch.empty((rows, hd), dtype=torch.float32, device="cuda")
    ctx.attn_combine(1, rows, hd, triples, want)
    x = wr.Exchange(ctx, 1, 0, rows, hd)
    for _ in range(3):
        got = torch.full((rows, hd), float("nan"), dtype=torch.float32, device="cuda")
        x.combine(rows, triples, got)
        ctx.sync()
        assert torch.equal(got, want)
    # the decode kernel delivering its triples itself (exchange fused in): same bits again,
    # with multi-chunk sessions (merge warps), a one-chunk session (engine) and an empty shard
    out3 = torch.full((len(lens), hq, hd), float("nan"), dtype=torch.float32, device="cuda")
    for _ in range(3):
        x.decode(kvs, 0, lens, qd, out3, hq)
        ctx.sync()
        assert torch.equal(out3.view(rows, hd), want)
    lens0 = [300, 0, 1]
    ctx.attn_decode_partial(kvs, 0, lens0, qd, triples, hq)
    ctx.attn_combine(1, rows, hd, triples, want)
    x.decode(kvs, 0, lens0, qd, out3, hq)
    ctx.sync()
    assert torch.equal(out3.view(rows, hd), want)
    with pytest.raises(wr.WrCudaError) as e:
        x.combine(rows + 1, triples, got)                       # more rows than the buffers hold
    assert e.value.status == -4
    x.close()
    with pytest.raises(wr.WrCudaError) as e:
        wr.Exchange(ctx, 9, 0, rows, hd)                        # world beyond WR_CUDA_XCHG_MAX_WORLD
    assert e.value.status == -4
    two = wr.Exchange(ctx, 2, 1, rows, hd)
    with pytest.raises(wr.WrCudaError) as e:
        two.combine(rows, triples, got)                         # peers not connected yet
    assert e.value.status == -7
    assert len(two.handle) == 64
    two.close()
    for kv in kvs:
        kv.close()
