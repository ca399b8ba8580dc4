"""Pin the CPU restatement (oracle/wr_oracle.c) to the reference.

Two anchors:
  * the committed fixture tests/golden/reference_outputs.npz — outputs of the
    unmodified reference compiled from its own sources (always checked);
  * the compiled reference itself, on more and larger seeded cases, wherever
    oracle/_ref exists (skipped elsewhere).
The restatement must be bit-identical to both: it runs the same float
operations in the same order.
"""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import cases  # noqa: E402
import _gen  # noqa: E402

GOLD = np.load(os.path.join(HERE, "golden", "reference_outputs.npz"))


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


# ------------------------------------------------------------ golden fixture

@pytest.mark.parametrize("fn", sorted(cases.MATH_POINTS))
def test_math_matches_fixture(port, fn):
    got = getattr(port, fn)(cases.MATH_POINTS[fn])
    assert np.array_equal(bits(got), GOLD[f"math/{fn}"])


def test_f16_encode_matches_fixture(port):
    assert np.array_equal(port.f32_to_f16(cases.F16_POINTS), GOLD["f16/encode"])


def test_f16_decode_matches_fixture(port):
    hs = np.arange(0, 65536, 7, dtype=np.uint16)
    got = port.f16_to_f32(hs)
    assert np.array_equal(bits(got), GOLD["f16/decode_all"])
    # numpy's float16 widening is the same exact map (NaN payloads included).
    assert np.array_equal(bits(hs.view(np.float16).astype(np.float32)), bits(got))


def test_f16_reference_witnesses(port):
    """test/unit_tests.c:98-108: 0x3C00 round trips and the truncation witness."""
    assert port.f16_to_f32_scalar(0x3C00) == 1.0
    assert port.f16_to_f32_scalar(0xC000) == -2.0
    assert port.f16_to_f32_scalar(0x0000) == 0.0
    assert port.f32_to_f16_scalar(1.0) == 0x3C00
    assert port.f32_to_f16_scalar(1.000732421875) == 0x3C00  # RTN would give 0x3C01


@pytest.mark.parametrize("c", cases.ROPE_CASES, ids=lambda c: c["name"])
def test_rope_matches_fixture(port, c):
    x = cases.rope_input(c, cases.case_seed(c["name"]))
    rc, y = port.rope(x, c["pos"], c["theta"], c["n_rot"])
    assert rc == 0
    assert np.array_equal(bits(y), GOLD[f"rope/{c['name']}"])


def test_rope_reference_known_answers(port):
    """src/core/kernels.c:2160-2183: identity at pos 0, the pos-1 value, and
    partial-rotary pass-through."""
    x = np.arange(1, 9, dtype=np.float32).reshape(2, 1, 4)
    rc, y = port.rope(x, 0, 10000.0, 0)
    assert rc == 0
    y = y.ravel()
    assert abs(y[0] - 1.0) < 0.01 and abs(y[2] - 3.0) < 0.01
    assert abs(y[4] - (5.0 * 0.5403 - 7.0 * 0.8415)) < 0.05
    rc, y2 = port.rope(x, 0, 10000.0, 1)
    y2 = y2.ravel()
    assert y2[5] == 6.0 and y2[7] == 8.0
    assert abs(y2[4] - (5.0 * 0.5403 - 7.0 * 0.8415)) < 0.05


@pytest.mark.parametrize("c", cases.ATTN_CASES, ids=lambda c: c["name"])
def test_attention_matches_fixture(port, c):
    q, k, v = cases.attn_inputs(c, cases.case_seed(c["name"]))
    if c["kv"] == "f16":
        k, v = port.f32_to_f16(k), port.f32_to_f16(v)
    rc, o = port.attention(q, k, v, seq_k=c["ctx"], scale=c.get("scale", 0.0),
                           window=c.get("window", 0))
    assert rc == 0
    assert np.array_equal(bits(o), bits(GOLD[f"attn/{c['name']}"]))


@pytest.mark.parametrize("c", cases.PREFILL_CASES, ids=lambda c: c["name"])
def test_prefill_matches_fixture(port, c):
    q, k, v = cases.prefill_inputs(c, cases.case_seed(c["name"]))
    k, v = port.f32_to_f16(k), port.f32_to_f16(v)
    if c["q"] == "f16":
        q = port.f32_to_f16(q)
    rc, o = port.causal_prefill_rows(q, k, v, cases.prefill_rows(c), p0=c["p0"],
                                     window=c.get("window", 0), threads=4)
    assert rc == 0
    assert np.array_equal(bits(o), bits(GOLD[f"prefill/{c['name']}"]))


def test_gqa_head_mapping_known_answer(port):
    """src/core/kernels.c:2185-2208: one key, so each output row is the V row
    of the mapped KV head (q heads 0,1 -> kv 0; 2,3 -> kv 1)."""
    q = np.ones((1, 4, 2), np.float32)
    k = np.ones((1, 2, 2), np.float32)
    v = np.array([10, 20, 30, 40], np.float32).reshape(1, 2, 2)
    rc, o = port.attention(q, k, v)
    assert rc == 0
    o = o.ravel()
    for idx, want in ((0, 10.0), (1, 20.0), (2, 10.0), (4, 30.0), (6, 30.0)):
        assert abs(o[idx] - want) < 0.5


def test_attention_refusals(port):
    """src/core/kernels.c:1429-1447: shape errors and the hard sequence cap."""
    one = np.ones((1, 1, 1), np.float32)
    z = np.zeros((4097, 1, 1), np.float32)
    rc, _ = port.attention(one, z, z)
    assert rc == -8 == int(GOLD["status/over_cap"][0])
    rc, _ = port.attention(np.ones((1, 3, 4), np.float32), np.ones((2, 2, 4), np.float32),
                           np.ones((2, 2, 4), np.float32))
    assert rc == -4  # 3 q heads over 2 kv heads
    rc, _ = port.attention(one, z[:4096], z[:4096])
    assert rc == 0


def test_kv_append_row_semantics(port):
    """src/core/session.c:139-154: cursor advance, truncation, CTX_FULL."""
    import ctypes as C
    cache = np.zeros((2, 6), np.uint16)
    valid = C.c_uint32(0)
    row = np.array([1.0, 1.000732421875, -2.0, 1e-9, 1e9, 0.5], np.float32)
    u16p, f32p = C.POINTER(C.c_uint16), C.POINTER(C.c_float)
    fn = port.lib.wro_kv_append_row
    for want_rc, want_valid in ((0, 1), (0, 2), (-6, 2)):
        rc = fn(cache.ctypes.data_as(u16p), C.c_uint32(2), C.byref(valid),
                row.ctypes.data_as(f32p), C.c_uint32(6))
        assert rc == want_rc and valid.value == want_valid
    assert list(cache[0]) == [0x3C00, 0x3C00, 0xC000, 0x0000, 0x7C00, 0x3800]
    assert np.array_equal(cache[0], cache[1])


def test_partials_merge_to_full_attention(port):
    """Split-KV algebra: shard triples merged with the online-softmax rule
    reproduce the unsplit op (to float associativity)."""
    q = _gen.normal(11, (1, 8, 128))
    k = port.f32_to_f16(_gen.normal(12, (500, 2, 128)))
    v = port.f32_to_f16(_gen.normal(13, (500, 2, 128)))
    rc, full = port.attention(q, k, v)
    assert rc == 0
    cuts = [0, 130, 256, 391, 500]
    ms, ls, os_ = [], [], []
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        rc, m, l, o = port.partial(q[0], k, v, lo, hi)
        assert rc == 0
        ms.append(m), ls.append(l), os_.append(o)
    ms, ls, os_ = np.array(ms), np.array(ls), np.array(os_)
    mstar = ms.max(axis=0)
    w = np.exp(ms - mstar)
    merged = (w[..., None] * os_).sum(0) / (w * ls).sum(0)[:, None]
    assert np.abs(merged - full[0]).max() < 2e-5


# ------------------------------------------------- against the live reference

def test_math_bit_exact_vs_reference(port, ref):
    xs = (_gen.normal(21, (4000,)) * np.float32(30.0)).astype(np.float32)
    for fn in ("exp", "sin", "cos"):
        assert np.array_equal(bits(getattr(port, fn)(xs)), bits(getattr(ref, fn)(xs))), fn
    pos = np.abs(xs) + np.float32(1e-3)
    for fn in ("log", "sqrt"):
        assert np.array_equal(bits(getattr(port, fn)(pos)), bits(getattr(ref, fn)(pos))), fn


def test_f16_encode_bit_exact_vs_reference(port, ref):
    x = _gen.normal(31, (200000,))
    scale = np.exp2((_gen.uniform_u32(32, (200000,)) % 60).astype(np.float32) - 30).astype(np.float32)
    x = (x * scale).astype(np.float32)
    assert np.array_equal(port.f32_to_f16(x), ref.f32_to_f16(x))


@pytest.mark.parametrize("theta", [1e4, 5e5, 1e6])
def test_rope_bit_exact_vs_reference(port, ref, theta):
    x = _gen.normal(41, (2, 3, 128))
    for pos in list(range(0, 4096, 97)) + [4094, 8191, 16384, 32766]:
        ra, a = port.rope(x, pos, theta, 0)
        rb, b = ref.rope(x, pos, theta, 0)
        assert ra == rb == 0
        assert np.array_equal(bits(a), bits(b)), pos


def test_decode_bit_exact_vs_reference(port, ref):
    q = _gen.normal(51, (3, 32, 128))
    lens = [1024 + 7, 2000, 555]
    ks = [ref.f32_to_f16(_gen.normal(52 + i, (n, 8, 128))) for i, n in enumerate(lens)]
    vs = [ref.f32_to_f16(_gen.normal(62 + i, (n, 8, 128))) for i, n in enumerate(lens)]
    ra, a = port.decode_batch(q, ks, vs, threads=3)
    rb, b = ref.decode_batch(q, ks, vs, threads=3)
    assert ra == rb == 0
    assert np.array_equal(bits(a), bits(b))


def test_long_context_cap(port, ref, ref_long):
    """The cap is compile-time (src/core/internal.h:186): 4097 keys are refused
    by the default build and served by the -DWR_ATTN_MAX_SEQ=32768 build."""
    q = _gen.normal(71, (1, 4, 128))
    k = ref.f32_to_f16(_gen.normal(72, (5000, 1, 128)))
    v = ref.f32_to_f16(_gen.normal(73, (5000, 1, 128)))
    assert ref.attention(q, k, v)[0] == -8
    assert port.attention(q, k, v)[0] == -8
    rb, b = ref_long.attention(q, k, v)
    ra, a = port.attention(q, k, v, max_seq=32768)
    assert ra == rb == 0
    assert np.array_equal(bits(a), bits(b))
