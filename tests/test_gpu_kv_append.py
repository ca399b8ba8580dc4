"""GPU parity: fused RoPE + KV append (wr_cuda_kv_append) against the oracle.

Bar: BIT-EXACT.  Cache bytes must equal kv_append_row(wri_op_rope(x))
(src/core/session.c:139-154, src/core/kernels.c:1356-1412) and the rotated Q
must equal wri_op_rope(q) bit for bit.
"""
import numpy as np
import pytest

import _gen
from _cuda_util import port

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import wayruntime_b200 as wr
    c = wr.Context(0, attn_max_seq=32768)
    yield c
    c.close()


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("theta", [1e4, 5e5, 1e6])
@pytest.mark.parametrize("hq,hkv,hd", [(32, 8, 128), (16, 8, 128), (40, 8, 128), (4, 4, 64), (2, 1, 8)])
def test_append_single_token_bit_exact(ctx, theta, hq, hkv, hd):
    P = port()
    positions = [0, 1, 63, 64, 65, 511, 1000, 4095]
    kvs = [ctx.kv_create(1, hkv, hd, 4096) for _ in positions]
    n = len(positions)
    q = _gen.normal(1, (n, hq, hd))
    k = _gen.normal(2, (n, hkv, hd)) * np.float32(3.0)
    v = _gen.normal(3, (n, hkv, hd)) * np.float32(3.0)
    q_rot = q.copy()
    ctx.kv_append(kvs, 0, positions, k, v, q_rot, hq, theta=theta)
    for i, pos in enumerate(positions):
        _, kr = P.rope(k[i:i + 1], pos, theta)
        _, qr = P.rope(q[i:i + 1], pos, theta)
        assert np.array_equal(kvs[i].read_rows(0, 0, pos, 1), P.f32_to_f16(kr)), (pos, "K")
        assert np.array_equal(kvs[i].read_rows(0, 1, pos, 1), P.f32_to_f16(v[i:i + 1])), (pos, "V")
        assert np.array_equal(bits(q_rot[i]), bits(qr[0])), (pos, "Q")
    for kv in kvs:
        kv.close()


def test_append_many_tokens_and_long_positions(ctx):
    """A prefill-sized append (n_tokens > 1) and positions up to 32767, where
    the reference's repeated-subtraction range reduction runs thousands of steps."""
    P = port()
    hq, hkv, hd, theta = 8, 2, 128, 1e6
    for p0, n in ((0, 200), (4000, 96), (32768 - 40, 40)):
        kv = ctx.kv_create(1, hkv, hd, 32768)
        q = _gen.normal(5, (n, hq, hd))
        k = _gen.normal(6, (n, hkv, hd))
        v = _gen.normal(7, (n, hkv, hd))
        q_rot = q.copy()
        ctx.kv_append([kv], 0, [p0], k, v, q_rot, hq, theta=theta, n_tokens=n)
        _, kr = P.rope(k, p0, theta)
        _, qr = P.rope(q, p0, theta)
        assert np.array_equal(kv.read_rows(0, 0, p0, n), P.f32_to_f16(kr))
        assert np.array_equal(kv.read_rows(0, 1, p0, n), P.f32_to_f16(v))
        assert np.array_equal(bits(q_rot), bits(qr))
        kv.close()


def test_append_truncation_and_specials(ctx):
    """test/unit_tests.c:105-107 witness plus subnormal flush, overflow and NaN."""
    P = port()
    hkv, hd = 1, 8
    kv = ctx.kv_create(1, hkv, hd, 64)
    row = np.array([1.0, 1.000732421875, -2.0, 6.0e-5, 5e-8, 1e9, -1e9, np.nan], np.float32)
    row = row.reshape(1, 1, 8)
    ctx.kv_append([kv], 0, [0], row, row, rope=False)
    got_k = kv.read_rows(0, 0, 0, 1)
    got_v = kv.read_rows(0, 1, 0, 1)
    want = P.f32_to_f16(row)
    assert np.array_equal(got_k, want) and np.array_equal(got_v, want)
    assert list(want.ravel()[:3]) == [0x3C00, 0x3C00, 0xC000]
    kv.close()


def test_append_partial_rotary_and_default_theta(ctx):
    P = port()
    hq, hkv, hd = 4, 2, 128
    kv = ctx.kv_create(1, hkv, hd, 1024)
    q = _gen.normal(8, (1, hq, hd))
    k = _gen.normal(9, (1, hkv, hd))
    v = _gen.normal(10, (1, hkv, hd))
    for theta, n_rot in ((1e4, 16), (0.5, 0), (1e6, 64), (1e6, 200)):
        q_rot = q.copy()
        ctx.kv_append([kv], 0, [777], k, v, q_rot, hq, theta=theta, n_rot_pairs=n_rot)
        _, kr = P.rope(k, 777, theta, n_rot)
        _, qr = P.rope(q, 777, theta, n_rot)
        assert np.array_equal(kv.read_rows(0, 0, 777, 1), P.f32_to_f16(kr)), (theta, n_rot)
        assert np.array_equal(bits(q_rot), bits(qr)), (theta, n_rot)
    kv.close()


def test_append_refusals(ctx):
    """session.c:144: a row at max_ctx is CTX_FULL and nothing is written."""
    import wayruntime_b200 as wr
    kv = ctx.kv_create(2, 2, 128, 100)
    row = _gen.normal(11, (1, 2, 128))
    with pytest.raises(wr.WrCudaError) as e:
        ctx.kv_append([kv], 0, [100], row, row, rope=False)
    assert e.value.status == -6
    with pytest.raises(wr.WrCudaError) as e:
        ctx.kv_append([kv], 0, [90], np.zeros((11, 2, 128), np.float32),
                      np.zeros((11, 2, 128), np.float32), rope=False, n_tokens=11)
    assert e.value.status == -6
    with pytest.raises(wr.WrCudaError) as e:
        ctx.kv_append([kv], 2, [0], row, row, rope=False)       # layer out of range
    assert e.value.status == -4
    with pytest.raises(wr.WrCudaError) as e:
        ctx.kv_append([kv, kv], 0, [0, 1], np.zeros((2, 2, 128), np.float32),
                      np.zeros((2, 2, 128), np.float32), rope=False)   # same session twice
    assert e.value.status == -4
    assert not kv.read_rows(0, 0, 0, 100).any()
    kv.close()


def test_session_create_limits(ctx):
    """session.c:755: max_ctx above the cap is WR_ERR_LIMIT; odd head_dim is INVAL."""
    import wayruntime_b200 as wr
    c2 = wr.Context(0)          # default cap 4096
    with pytest.raises(wr.WrCudaError) as e:
        c2.kv_create(1, 8, 128, 4097)
    assert e.value.status == -8
    c2.kv_create(1, 8, 128, 4096).close()
    with pytest.raises(wr.WrCudaError) as e:
        c2.kv_create(1, 8, 127, 64)
    assert e.value.status == -4
    with pytest.raises(wr.WrCudaError) as e:
        c2.kv_create(1, 8, 2048, 64)
    assert e.value.status == -8
    c2.close()


def test_rows_round_trip_all_layers(ctx):
    """write_rows/read_rows are inverse on every layer and both layouts."""
    for hd in (128, 64, 24):
        kv = ctx.kv_create(3, 3, hd, 200)
        for layer in range(3):
            for which in (0, 1):
                rows = _gen.uniform_u32(100 + layer * 2 + which, (150, 3, hd)).astype(np.uint16)
                kv.write_rows(layer, which, 25, rows)
                assert np.array_equal(kv.read_rows(layer, which, 25, 150), rows)
        kv.close()


@pytest.mark.parametrize("n_rot", [0, 20])
def test_decode_step_host_buffer_paths_agree(ctx, n_rot):
    """wr_cuda_decode_step with host buffers: pageable arrays are staged through
    copies, page-locked ones are read and written by the kernels directly.  Both
    must leave the same cache bytes and attention rows as the device-buffer
    sequence append -> decode, and must leave the host's Q rows untouched."""
    import torch
    P = port()
    hq, hkv, hd, theta = 32, 8, 128, 5e5
    lens = [130, 1, 700, 64]
    n = len(lens)
    q = _gen.normal(41, (n, hq, hd))
    k_new = _gen.normal(42, (n, hkv, hd))
    v_new = _gen.normal(43, (n, hkv, hd))
    hist_k = [P.f32_to_f16(_gen.normal(50 + i, (ln - 1, hkv, hd))) for i, ln in enumerate(lens)]
    hist_v = [P.f32_to_f16(_gen.normal(60 + i, (ln - 1, hkv, hd))) for i, ln in enumerate(lens)]

    def fresh():
        kvs = [ctx.kv_create(1, hkv, hd, 1024) for _ in lens]
        for kv, hk, hv in zip(kvs, hist_k, hist_v):
            if hk.shape[0]:
                kv.write_rows(0, 0, 0, hk)
                kv.write_rows(0, 1, 0, hv)
        return kvs

    pos = [ln - 1 for ln in lens]
    # device buffers: append (rotates q in place), then decode
    kvs = fresh()
    qd = torch.from_numpy(q.copy()).cuda()
    outd = torch.empty_like(qd)
    ctx.kv_append(kvs, 0, pos, torch.from_numpy(k_new).cuda(), torch.from_numpy(v_new).cuda(), qd, hq,
                  theta=theta, n_rot_pairs=n_rot)
    ctx.attn_decode(kvs, 0, lens, qd, outd, hq)
    ctx.sync()
    want = outd.cpu().numpy()
    want_rows = [(kv.read_rows(0, 0, ln - 1, 1), kv.read_rows(0, 1, ln - 1, 1)) for kv, ln in zip(kvs, lens)]
    for kv in kvs:
        kv.close()
    # pageable host arrays, then page-locked host tensors
    for pinned in (False, True):
        kvs = fresh()
        if pinned:
            hq_, hk_, hv_ = (torch.from_numpy(a.copy()).pin_memory() for a in (q, k_new, v_new))
            hout = torch.full((n, hq, hd), float("nan")).pin_memory()
        else:
            hq_, hk_, hv_ = q.copy(), k_new.copy(), v_new.copy()
            hout = np.full((n, hq, hd), np.nan, np.float32)
        ctx.decode_step(kvs, 0, pos, hq_, hk_, hv_, hout, hq, theta=theta, n_rot_pairs=n_rot)
        got = hout.numpy() if pinned else hout
        assert np.array_equal(bits(got), bits(want)), f"pinned={pinned}"
        q_after = hq_.numpy() if pinned else hq_
        assert np.array_equal(bits(q_after), bits(q)), "host Q rows must stay as given"
        for kv, ln, (wk, wv) in zip(kvs, lens, want_rows):
            assert np.array_equal(kv.read_rows(0, 0, ln - 1, 1), wk)
            assert np.array_equal(kv.read_rows(0, 1, ln - 1, 1), wv)
        for kv in kvs:
            kv.close()


def test_decode_step_page_locked_views_at_odd_offsets_are_staged(ctx):
    """Rows move as 16-byte vectors, so the kernels may touch a page-locked host
    buffer directly only when it is 16-byte aligned.  A page-locked view that
    starts 8 bytes into its allocation must give the same bits through the
    staged copy path (never a launch on the misaligned address), and a device
    row buffer at such an offset is refused."""
    import torch
    import wayruntime_b200 as wr
    P = port()
    hq, hkv, hd, theta = 32, 8, 128, 5e5
    lens = [200, 65]
    n = len(lens)
    q = _gen.normal(141, (n, hq, hd))
    k_new = _gen.normal(142, (n, hkv, hd))
    v_new = _gen.normal(143, (n, hkv, hd))
    hist_k = [P.f32_to_f16(_gen.normal(150 + i, (ln - 1, hkv, hd))) for i, ln in enumerate(lens)]
    hist_v = [P.f32_to_f16(_gen.normal(160 + i, (ln - 1, hkv, hd))) for i, ln in enumerate(lens)]

    def fresh():
        kvs = [ctx.kv_create(1, hkv, hd, 256) for _ in lens]
        for kv, hk, hv in zip(kvs, hist_k, hist_v):
            kv.write_rows(0, 0, 0, hk)
            kv.write_rows(0, 1, 0, hv)
        return kvs

    def odd_view(a):
        """page-locked float32 tensor shaped like `a`, starting 8 bytes into its allocation"""
        base = torch.empty(a.size + 2, dtype=torch.float32).pin_memory()
        view = base[2:].view(a.shape)
        view.copy_(torch.from_numpy(a))
        assert view.data_ptr() % 16 == 8
        return view

    pos = [ln - 1 for ln in lens]
    results = []
    for odd in (False, True):
        kvs = fresh()
        mk = odd_view if odd else (lambda a: torch.from_numpy(a.copy()).pin_memory())
        hq_, hk_, hv_ = mk(q), mk(k_new), mk(v_new)
        hout = mk(np.full((n, hq, hd), np.nan, np.float32))
        ctx.decode_step(kvs, 0, pos, hq_, hk_, hv_, hout, hq, theta=theta)
        results.append((hout.numpy().copy(), [kv.read_rows(0, 0, ln - 1, 1) for kv, ln in zip(kvs, lens)]))
        for kv in kvs:
            kv.close()
    assert np.array_equal(bits(results[0][0]), bits(results[1][0]))
    for a, b in zip(results[0][1], results[1][1]):
        assert np.array_equal(a, b)
    # device rows at an 8-byte offset: refused before any launch
    kv = ctx.kv_create(1, hkv, hd, 64)
    dev = torch.zeros(4 * hkv * hd + 4, dtype=torch.int16, device="cuda")[4:].view(4, hkv, hd)
    assert dev.data_ptr() % 16 == 8
    with pytest.raises(wr.WrCudaError) as e:
        kv.write_rows(0, 0, 0, dev)
    assert e.value.status == -4
    kv.close()


def test_prepared_decode_step_is_the_same_call(ctx):
    """Context.prepared_decode_step resolves the arguments once; each step(layer) must be
    wr_cuda_decode_step on those arguments: same attention rows, same cache bytes."""
    import torch
    import wayruntime_b200 as wr
    hq, hkv, hd = 8, 2, 128
    lens = [70, 3, 200]
    n = len(lens)
    q = torch.from_numpy(_gen.normal(71, (n, hq, hd))).pin_memory()
    k = torch.from_numpy(_gen.normal(72, (n, hkv, hd))).pin_memory()
    v = torch.from_numpy(_gen.normal(73, (n, hkv, hd))).pin_memory()
    results = []
    for prepared in (False, True):
        kvs = [ctx.kv_create(2, hkv, hd, 256) for _ in lens]
        out = torch.full((n, hq, hd), float("nan")).pin_memory()
        pos = wr.Batch.u32([ln - 1 for ln in lens])
        batch = wr.Batch(kvs)
        step = ctx.prepared_decode_step(batch, pos, q, k, v, out, hq, theta=5e5) if prepared else None
        outs = []
        for t in range(3):
            layer = t % 2
            if prepared:
                step(layer)
            else:
                ctx.decode_step(batch, layer, pos, q, k, v, out, hq, theta=5e5)
            outs.append(out.numpy().copy())
            for i in range(n):
                pos[i] += 1 if layer == 1 else 0          # the caller's own array: advanced in place
        rows = [kv.read_rows(0, 0, lens[i] - 1, 2) for i, kv in enumerate(kvs)]
        results.append((outs, rows))
        for kv in kvs:
            kv.close()
    for a, b in zip(results[0][0], results[1][0]):
        assert np.array_equal(bits(a), bits(b))
    for a, b in zip(results[0][1], results[1][1]):
        assert np.array_equal(a, b)
