"""Regenerate tests/golden/reference_outputs.npz from the compiled reference.

Run in a checkout that has the reference sources (it builds oracle/_ref first):

    python tests/golden/make_golden.py

Everything stored is an OUTPUT of the unmodified reference; the inputs are
rebuilt from tests/_gen.py by the tests.  The file is committed so that the
restatement and the CUDA kernels can be pinned where the reference is absent.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

import oracle  # noqa: E402
from oracle import bindings  # noqa: E402
import cases  # noqa: E402


def main():
    bindings.build()
    ref = oracle.reference()
    assert ref is not None, "reference build missing"
    out = {}
    for fn, xs in cases.MATH_POINTS.items():
        out[f"math/{fn}"] = getattr(ref, fn)(xs).view(np.uint32)
    out["f16/encode"] = ref.f32_to_f16(cases.F16_POINTS)
    out["f16/decode_all"] = ref.f16_to_f32(np.arange(0, 65536, 7, dtype=np.uint16)).view(np.uint32)
    for c in cases.ROPE_CASES:
        x = cases.rope_input(c, cases.case_seed(c["name"]))
        rc, y = ref.rope(x, c["pos"], c["theta"], c["n_rot"])
        assert rc == 0
        out[f"rope/{c['name']}"] = y.view(np.uint32)
    for c in cases.ATTN_CASES:
        q, k, v = cases.attn_inputs(c, cases.case_seed(c["name"]))
        if c["kv"] == "f16":
            k, v = ref.f32_to_f16(k), ref.f32_to_f16(v)
        rc, o = ref.attention(q, k, v, seq_k=c["ctx"], scale=c.get("scale", 0.0),
                              window=c.get("window", 0), growable=True)
        assert rc == 0, (c["name"], rc)
        out[f"attn/{c['name']}"] = o
    for c in cases.PREFILL_CASES:
        q, k, v = cases.prefill_inputs(c, cases.case_seed(c["name"]))
        k, v = ref.f32_to_f16(k), ref.f32_to_f16(v)
        if c["q"] == "f16":
            q = ref.f32_to_f16(q)
        rows = cases.prefill_rows(c)
        rc, o = ref.causal_prefill_rows(q, k, v, rows, p0=c["p0"],
                                        window=c.get("window", 0), threads=8)
        assert rc == 0, (c["name"], rc)
        out[f"prefill/{c['name']}"] = o
    # The sequence cap is a hard error (src/core/kernels.c:1444).
    z = np.zeros((ref.max_seq + 1, 1, 1), np.float32)
    rc, _ = ref.attention(np.ones((1, 1, 1), np.float32), z, z, growable=False)
    out["status/over_cap"] = np.array([rc], dtype=np.int32)
    path = os.path.join(HERE, "reference_outputs.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
