"""GPU parity: causal prefill attention (wr_cuda_attn_prefill, tcgen05/TMEM).

Bar: max-abs error <= 2e-3 against the reference's prefill, which is a loop of
single-token attention calls (src/core/session.c:599-630): row i attends cache
rows [0, p0+i].  Q reaches the tensor cores as F16 (F32 queries are rounded to
F16 first); P is F16; accumulation is F32.
"""
import os
import sys

import numpy as np
import pytest

import _gen
from _cuda_util import TOL, make_cache, port

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


def run_prefill(ctx, q, k16, v16, p0, hq, scale=0.0, window=0, max_ctx=None):
    kv = make_cache(ctx, k16, v16, max_ctx=max_ctx)
    n = q.shape[0]
    out = np.full((n, hq, q.shape[2]), np.nan, np.float32)
    ctx.attn_prefill(kv, 0, p0, n, np.ascontiguousarray(q), out, hq, scale=scale, window=window)
    kv.close()
    return out


@pytest.mark.parametrize("c", cases.PREFILL_CASES, ids=lambda c: c["name"])
def test_prefill_matches_reference_fixture(ctx, c):
    P = port()
    q, k, v = cases.prefill_inputs(c, cases.case_seed(c["name"]))
    k16, v16 = P.f32_to_f16(k), P.f32_to_f16(v)
    if c["q"] == "f16":
        q = P.f32_to_f16(q)
    out = run_prefill(ctx, q, k16, v16, c["p0"], c["hq"], window=c.get("window", 0))
    rows = cases.prefill_rows(c)
    want = GOLD[f"prefill/{c['name']}"]
    assert np.isfinite(out).all()
    assert np.abs(out[rows] - want).max() <= TOL


@pytest.mark.parametrize("n,p0,hq,hkv", [(1, 0, 8, 2), (127, 0, 8, 2), (128, 0, 4, 4), (129, 0, 8, 8),
                                         (300, 0, 32, 8), (200, 333, 32, 8), (260, 60, 40, 8),
                                         (64, 4000, 16, 8)])
def test_prefill_shapes_vs_oracle(ctx, n, p0, hq, hkv):
    """Ragged tile edges, a non-empty cache before the chunk, group sizes 1-5."""
    P = port()
    tot = p0 + n
    q = P.f32_to_f16(_gen.normal(600 + n, (n, hq, 128)))
    k16 = P.f32_to_f16(_gen.normal(601 + n, (tot, hkv, 128)))
    v16 = P.f32_to_f16(_gen.normal(602 + n, (tot, hkv, 128)))
    out = run_prefill(ctx, q, k16, v16, p0, hq, max_ctx=tot + 70)
    rows = np.unique(np.clip(np.array([0, 1, 62, 63, 64, 65, 126, 127, 128, 129, n - 2, n - 1] +
                                      list(range(0, n, 37))), 0, n - 1)).astype(np.uint32)
    rc, want = P.causal_prefill_rows(q, k16, v16, rows, p0=p0, threads=8, max_seq=32768)
    assert rc == 0
    assert np.isfinite(out).all()
    assert np.abs(out[rows] - want).max() <= TOL


def test_prefill_f32_queries_scale_and_window(ctx):
    P = port()
    n, p0, hq, hkv = 150, 40, 8, 2
    q = _gen.normal(700, (n, hq, 128))
    k16 = P.f32_to_f16(_gen.normal(701, (p0 + n, hkv, 128)))
    v16 = P.f32_to_f16(_gen.normal(702, (p0 + n, hkv, 128)))
    rows = np.arange(0, n, 7, dtype=np.uint32)
    for scale, window in ((0.0, 0), (0.05, 0), (0.0, 50), (0.0, 64), (0.0, 1)):
        out = run_prefill(ctx, q, k16, v16, p0, hq, scale=scale, window=window)
        rc, want = P.causal_prefill_rows(q, k16, v16, rows, p0=p0, scale=scale, window=window,
                                         threads=8)
        assert rc == 0
        assert np.abs(out[rows] - want).max() <= TOL, (scale, window)


def test_prefill_llama3_2048(ctx):
    """benchmark config 3: 2048-token prompt, 32 Q / 8 KV heads, head_dim 128,
    RoPE theta 5e5 applied to Q and K with the reference's rotation before
    attention.  All heads on a deterministic row subset."""
    P = port()
    n, hq, hkv = 2048, 32, 8
    _, q = P.rope(_gen.normal(800, (n, hq, 128)), 0, 500000.0)
    _, k = P.rope(_gen.normal(801, (n, hkv, 128)), 0, 500000.0)
    q16 = P.f32_to_f16(q)
    k16 = P.f32_to_f16(k)
    v16 = P.f32_to_f16(_gen.normal(802, (n, hkv, 128)))
    out = run_prefill(ctx, q16, k16, v16, 0, hq)
    rows = np.unique(np.array([0, 1, 63, 64, 127, 128, 1023, 1024, 2046, 2047] +
                              list(range(5, n, 97)))).astype(np.uint32)
    rc, want = P.causal_prefill_rows(q16, k16, v16, rows, threads=8)
    assert rc == 0
    assert np.isfinite(out).all()
    assert np.abs(out[rows] - want).max() <= TOL


def test_prefill_config5_8192_then_decode(ctx):
    """benchmark config 5 geometry: 40 Q / 8 KV heads (group of five: one lone
    head per pair split), one session's 8192-token prompt, then a decode step
    over the 8193 cached keys.  Prefill rows: all heads on a deterministic row
    subset (first/last rows, 64-boundaries +-1, a stride); the decode row in full."""
    P = port()
    n, hq, hkv = 8192, 40, 8
    q16 = P.f32_to_f16(_gen.normal(810, (n, hq, 128)))
    k16 = P.f32_to_f16(_gen.normal(811, (n + 1, hkv, 128)))
    v16 = P.f32_to_f16(_gen.normal(812, (n + 1, hkv, 128)))
    kv = make_cache(ctx, k16, v16, max_ctx=n + 64)
    out = np.full((n, hq, 128), np.nan, np.float32)
    ctx.attn_prefill(kv, 0, 0, n, np.ascontiguousarray(q16), out, hq)
    rows = np.unique(np.array([0, 1, 63, 64, 65, 127, 128, 4095, 4096, 4097, 8126, 8127, 8128, 8190, 8191] +
                              list(range(31, n, 1021)))).astype(np.uint32)
    rc, want = P.causal_prefill_rows(q16, k16[:n], v16[:n], rows, threads=8, max_seq=32768)
    assert rc == 0
    assert np.isfinite(out).all()
    assert np.abs(out[rows] - want).max() <= TOL
    qd = _gen.normal(813, (1, hq, 128))
    got = np.full((1, hq, 128), np.nan, np.float32)
    ctx.attn_decode([kv], 0, [n + 1], qd, got, hq)
    rc, want_d = P.attention(qd, k16, v16, seq_k=n + 1, max_seq=32768)
    assert rc == 0
    assert np.abs(got - want_d).max() <= TOL
    kv.close()


def test_prefill_then_decode_consistency(ctx):
    """The last row of a prefill equals a decode step over the same cache."""
    P = port()
    n, hq, hkv = 200, 32, 8
    q = _gen.normal(900, (n, hq, 128))
    k16 = P.f32_to_f16(_gen.normal(901, (n, hkv, 128)))
    v16 = P.f32_to_f16(_gen.normal(902, (n, hkv, 128)))
    kv = make_cache(ctx, k16, v16)
    out = np.zeros((n, hq, 128), np.float32)
    ctx.attn_prefill(kv, 0, 0, n, q, out, hq)
    dec = np.zeros((1, hq, 128), np.float32)
    ctx.attn_decode([kv], 0, [n], np.ascontiguousarray(q[n - 1:n]), dec, hq)
    assert np.abs(out[n - 1] - dec[0]).max() <= TOL
    kv.close()


def test_prefill_refusals(ctx):
    import wayruntime_b200 as wr
    kv = ctx.kv_create(1, 2, 128, 256)
    q = np.zeros((10, 8, 128), np.float32)
    out = np.zeros_like(q)

    def status(fn):
        with pytest.raises(wr.WrCudaError) as e:
            fn()
        return e.value.status

    assert status(lambda: ctx.attn_prefill(kv, 0, 250, 10, q, out, 8)) == -4     # past capacity
    assert status(lambda: ctx.attn_prefill(kv, 0, 0, 10, q, out, 7)) == -4       # 7 % 2 != 0
    assert status(lambda: ctx.attn_prefill(kv, 1, 0, 10, q, out, 8)) == -4       # layer
    kv64 = ctx.kv_create(1, 2, 64, 256)
    q64 = np.zeros((10, 8, 64), np.float32)
    assert status(lambda: ctx.attn_prefill(kv64, 0, 0, 10, q64, np.zeros_like(q64), 8)) == -3
    kv.close(), kv64.close()


def test_prefill_row_maximum_grows_for_some_rows_only(ctx):
    """Scores that keep growing along the keys for some query rows and stay flat
    for their neighbours: the accumulator is rescaled again and again, and within
    one warp only some rows need it (the reference rescales per row,
    src/core/kernels.c:1496-1510)."""
    P = port()
    n, hq, hkv = 640, 4, 2
    u = _gen.normal(711, (128,))
    u /= np.linalg.norm(u)
    k = 0.3 * _gen.normal(712, (n, hkv, 128))
    k += (np.arange(n, dtype=np.float32)[:, None, None] / 8.0) * u          # component along u grows with the key index
    q = 0.3 * _gen.normal(713, (n, hq, 128))
    gain = np.where(np.arange(n) % 3 == 0, 6.0, 0.0).astype(np.float32)     # every third row looks along u
    q += gain[:, None, None] * u
    q16, k16 = P.f32_to_f16(q.astype(np.float32)), P.f32_to_f16(k.astype(np.float32))
    v16 = P.f32_to_f16(_gen.normal(714, (n, hkv, 128)))
    out = run_prefill(ctx, q16, k16, v16, 0, hq)
    rows = np.arange(0, n, 5, dtype=np.uint32)
    rc, want = P.causal_prefill_rows(q16, k16, v16, rows, p0=0, threads=8, max_seq=32768)
    assert rc == 0
    assert np.isfinite(out).all()
    assert np.abs(out[rows] - want).max() <= TOL


@pytest.mark.parametrize("n", [1, 33, 70, 128 + 31])
def test_prefill_writes_every_row_of_the_prompt_and_nothing_after_it(ctx, n):
    """The output leaves the kernel in pieces of 32 rows x 32 values; pieces that straddle the
    prompt's last row are cut there and pieces wholly past it are not sent.  Device buffers:
    rows [0, n) are all written, the rows behind them keep what they held."""
    import torch
    P = port()
    hq, hkv, tail = 8, 2, 40
    k16 = P.f32_to_f16(_gen.normal(901 + n, (n, hkv, 128)))
    v16 = P.f32_to_f16(_gen.normal(902 + n, (n, hkv, 128)))
    q16 = P.f32_to_f16(_gen.normal(903 + n, (n, hq, 128)))
    kv = make_cache(ctx, k16, v16, max_ctx=n + 70)
    q = torch.from_numpy(q16.view(np.int16)).cuda().view(torch.float16)
    buf = torch.full((n + tail, hq, 128), float("nan"), device="cuda")
    buf[n:] = 7.0
    torch.cuda.synchronize()
    ctx.attn_prefill(kv, 0, 0, n, q, buf[:n], hq)
    ctx.sync()
    got = buf.cpu().numpy()
    kv.close()
    assert np.isfinite(got[:n]).all()
    assert (got[n:] == 7.0).all()
    rows = np.arange(n, dtype=np.uint32)
    rc, want = P.causal_prefill_rows(q16, k16, v16, rows, p0=0, threads=8, max_seq=32768)
    assert rc == 0
    assert np.abs(got[:n] - want).max() <= TOL
