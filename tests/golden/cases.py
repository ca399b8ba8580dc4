"""Case tables shared by the fixture generator and the parity tests.

Inputs are regenerated from ``tests/_gen.py`` (integer hashing, bit-stable);
the fixtures hold only what the reference computed from them.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import _gen  # noqa: E402

# Attention through the reference op (src/core/kernels.c:1414).  kv/q name the
# storage type; "f16" inputs are made by the reference's truncating convert.
# The kat_* rows have the shapes of the reference's own known-answer tests
# (src/core/kernels.c:1907-2062, :2185-2208) with hashed fills.
ATTN_CASES = [
    dict(name="kat_small_mha", sq=2, hq=1, hkv=1, hd=4, ctx=8, cap=8, q="f32", kv="f32", std=0.5),
    dict(name="kat_scale_override", sq=2, hq=1, hkv=1, hd=4, ctx=8, cap=8, q="f32", kv="f32", std=0.5, scale=0.25),
    dict(name="kat_window4", sq=2, hq=1, hkv=1, hd=4, ctx=8, cap=8, q="f32", kv="f32", std=0.5, window=4),
    dict(name="kat_grow_64", sq=2, hq=1, hkv=1, hd=8, ctx=64, cap=4096, q="f32", kv="f32", std=0.3),
    dict(name="kat_grow_256", sq=2, hq=1, hkv=1, hd=8, ctx=256, cap=4096, q="f32", kv="f32", std=0.3),
    dict(name="kat_grow_1024", sq=2, hq=1, hkv=1, hd=8, ctx=1024, cap=4096, q="f32", kv="f32", std=0.3),
    dict(name="kat_grow_4096", sq=2, hq=1, hkv=1, hd=8, ctx=4096, cap=4096, q="f32", kv="f32", std=0.3),
    dict(name="kat_gqa_map", sq=1, hq=4, hkv=2, hd=2, ctx=1, cap=1, q="f32", kv="f32", std=1.0),
    dict(name="decode_llama_333", sq=1, hq=32, hkv=8, hd=128, ctx=333, cap=384, q="f32", kv="f16", std=1.0),
    dict(name="decode_qwen_65", sq=1, hq=16, hkv=8, hd=128, ctx=65, cap=128, q="f32", kv="f16", std=1.0),
    dict(name="decode_wide_129", sq=1, hq=40, hkv=8, hd=128, ctx=129, cap=192, q="f32", kv="f16", std=1.0),
    dict(name="decode_window_100", sq=1, hq=32, hkv=8, hd=128, ctx=300, cap=320, q="f32", kv="f16", std=1.0, window=100),
    dict(name="decode_scale_one", sq=1, hq=8, hkv=8, hd=128, ctx=200, cap=256, q="f32", kv="f16", std=0.25, scale=1.0),
    dict(name="decode_one_key", sq=1, hq=32, hkv=8, hd=128, ctx=1, cap=64, q="f32", kv="f16", std=1.0),
    dict(name="decode_tile_edge_64", sq=1, hq=32, hkv=8, hd=128, ctx=64, cap=64, q="f32", kv="f16", std=1.0),
    dict(name="decode_mha_hd64", sq=1, hq=4, hkv=4, hd=64, ctx=100, cap=128, q="f32", kv="f16", std=1.0),
]

# Causal prefill = the reference's loop of single-token bodies
# (src/core/session.c:599-630): row i sees keys [0, p0+i].
PREFILL_CASES = [
    dict(name="prefill_f16q_96", n=96, p0=0, hq=8, hkv=2, hd=128, q="f16", std=1.0),
    dict(name="prefill_f32q_70_p0_50", n=70, p0=50, hq=8, hkv=4, hd=128, q="f32", std=1.0),
    dict(name="prefill_wide_130", n=130, p0=0, hq=10, hkv=2, hd=128, q="f16", std=1.0),
    dict(name="prefill_window_40", n=100, p0=20, hq=4, hkv=2, hd=128, q="f16", std=1.0, window=40),
]

ROPE_CASES = [
    dict(name="rope_kat_shape", seq=2, heads=1, hd=4, pos=0, theta=10000.0, n_rot=0),
    dict(name="rope_kat_partial", seq=2, heads=1, hd=4, pos=0, theta=10000.0, n_rot=1),
    dict(name="rope_llama3_pos0", seq=4, heads=8, hd=128, pos=0, theta=500000.0, n_rot=0),
    dict(name="rope_llama3_pos4093", seq=3, heads=8, hd=128, pos=4093, theta=500000.0, n_rot=0),
    dict(name="rope_qwen3_pos32765", seq=3, heads=2, hd=128, pos=32765, theta=1000000.0, n_rot=0),
    dict(name="rope_1e4_pos1000", seq=2, heads=4, hd=64, pos=1000, theta=10000.0, n_rot=0),
    dict(name="rope_partial_16", seq=2, heads=2, hd=128, pos=777, theta=10000.0, n_rot=16),
    dict(name="rope_theta_default", seq=1, heads=1, hd=8, pos=9, theta=0.5, n_rot=0),
]

MATH_POINTS = {
    "exp": np.concatenate([np.linspace(-95, 95, 381), [-88.0, 88.0, -87.99, 0.0, -0.0, 1e-8]]).astype(np.float32),
    "log": np.concatenate([np.geomspace(1e-30, 1e30, 301), [1e4, 5e5, 1e6, 1.0, 2.0]]).astype(np.float32),
    "sqrt": np.concatenate([np.geomspace(1e-6, 4096, 201), [128.0, 64.0, 2.0, 0.0, -1.0]]).astype(np.float32),
    "sin": np.concatenate([np.linspace(-40, 40, 321), [3.0, 3.14, 22.0, 4095.0, 32767.0]]).astype(np.float32),
    "cos": np.concatenate([np.linspace(-40, 40, 321), [3.0, 3.14, 22.0, 4095.0, 32767.0]]).astype(np.float32),
}

F16_POINTS = np.concatenate([
    np.array([1.0, 1.000732421875, -2.0, 0.0, -0.0, 65504.0, 65520.0, 1e5, -1e5, 6.1e-5,
              6.0e-5, 5.96e-8, 1e-10, np.inf, -np.inf, np.nan, 0.333333, -0.1],
             dtype=np.float32),
    _gen.normal(901, (256,)) * np.float32(3.0),
    (_gen.normal(902, (128,)) * np.float32(1e-4)).astype(np.float32),
])


def attn_inputs(c, seed):
    """(q, k, v) float32 for an ATTN case; k/v have `cap` rows."""
    q = _gen.normal(seed, (c["sq"], c["hq"], c["hd"]), c["std"])
    k = _gen.normal(seed + 1, (c["cap"], c["hkv"], c["hd"]), c["std"])
    v = _gen.normal(seed + 2, (c["cap"], c["hkv"], c["hd"]), c["std"])
    return q, k, v


def prefill_inputs(c, seed):
    tot = c["p0"] + c["n"]
    q = _gen.normal(seed, (c["n"], c["hq"], c["hd"]), c["std"])
    k = _gen.normal(seed + 1, (tot, c["hkv"], c["hd"]), c["std"])
    v = _gen.normal(seed + 2, (tot, c["hkv"], c["hd"]), c["std"])
    return q, k, v


def prefill_rows(c):
    """Rows kept in the fixture: edges, the 64-key tile boundary, every 9th."""
    n = c["n"]
    keep = {0, 1, n - 1, 62, 63, 64, 65} | set(range(0, n, 9))
    return np.array(sorted(r for r in keep if 0 <= r < n), dtype=np.uint32)


def rope_input(c, seed):
    return _gen.normal(seed, (c["seq"], c["heads"], c["hd"]), 1.0)


def case_seed(name):
    """Stable per-case seed (no Python hash randomisation)."""
    s = 0
    for ch in name.encode():
        s = (s * 131 + ch) % 1000003
    return 1000 + s
