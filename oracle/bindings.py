"""ctypes bindings for the two CPU checkers.  TEST INFRASTRUCTURE ONLY.

Both checkers expose the same Python methods, so a test can run the same case
through the restatement (always available) and through the compiled reference
(available wherever ``oracle/_ref`` was built) and demand identical bits.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

F32, F16 = 0, 1
_u16p = C.POINTER(C.c_uint16)
_f32p = C.POINTER(C.c_float)
_u32p = C.POINTER(C.c_uint32)
_u8p = C.POINTER(C.c_uint8)


def _ptr(a, typ):
    return a.ctypes.data_as(typ)


def _dtype_code(a):
    if a.dtype == np.float32:
        return F32
    if a.dtype in (np.uint16, np.float16):
        return F16
    raise TypeError(f"unsupported dtype {a.dtype}")


def reference_root() -> str:
    """The reference checkout: $WR_REFERENCE_ROOT, else a `reference` folder
    beside this repository."""
    return os.environ.get("WR_REFERENCE_ROOT") or os.path.join(
        os.path.dirname(os.path.dirname(_HERE)), "reference")


def build(ref_root: str | None = None) -> None:
    """Compile liboracle.so and, when the reference checkout exists, _ref/*.so."""
    ref_root = ref_root or reference_root()
    res = subprocess.run(["make", "-C", _HERE, f"REF={ref_root}"],
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"oracle build failed:\n{res.stdout}")


class Checker:
    """One loaded checker library (restatement or compiled reference)."""

    def __init__(self, path: str, kind: str):
        self.kind = kind
        self.path = path
        self.lib = C.CDLL(path)
        L = self.lib
        pre = "wro_" if kind == "port" else "refshim_"
        self._pre = pre
        for name in ("exp", "log", "sqrt", "sin", "cos"):
            fn = getattr(L, pre + name)
            fn.restype = C.c_float
            fn.argtypes = [C.c_float]
        getattr(L, pre + "f16_to_f32").restype = C.c_float
        getattr(L, pre + "f16_to_f32").argtypes = [C.c_uint16]
        getattr(L, pre + "f32_to_f16").restype = C.c_uint16
        getattr(L, pre + "f32_to_f16").argtypes = [C.c_float]
        if kind == "reference":
            L.refshim_attn_max_seq.restype = C.c_uint32
            self.max_seq = int(L.refshim_attn_max_seq())
        else:
            self.max_seq = 4096

    # ---- scalar math -------------------------------------------------
    def _scalar(self, name, x):
        fn = getattr(self.lib, self._pre + name)
        x = np.asarray(x, dtype=np.float32)
        out = np.empty_like(x)
        xf, of = x.ravel(), out.ravel()
        for i in range(xf.size):
            of[i] = fn(float(xf[i]))
        return out if out.ndim else np.float32(out)

    def exp(self, x): return self._scalar("exp", x)
    def log(self, x): return self._scalar("log", x)
    def sqrt(self, x): return self._scalar("sqrt", x)
    def sin(self, x): return self._scalar("sin", x)
    def cos(self, x): return self._scalar("cos", x)

    # ---- f16 ---------------------------------------------------------
    def f32_to_f16(self, x):
        """Truncating conversion; returns uint16 bit patterns."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        if self.kind == "reference":
            out = np.empty(x.shape, dtype=np.uint16)
            self.lib.refshim_f32_to_f16_n(_ptr(x, _f32p), _ptr(out, _u16p),
                                          C.c_uint64(x.size))
            return out
        out = np.empty(x.shape, dtype=np.uint16)
        self.lib.wro_f32_to_f16_n(_ptr(x, _f32p), _ptr(out, _u16p), C.c_uint64(x.size))
        return out

    def f16_to_f32(self, h):
        """Exact widening of uint16 bit patterns."""
        h = np.ascontiguousarray(h, dtype=np.uint16)
        out = np.empty(h.shape, dtype=np.float32)
        getattr(self.lib, self._pre + "f16_to_f32_n")(_ptr(h, _u16p), _ptr(out, _f32p), C.c_uint64(h.size))
        return out

    def f32_to_f16_scalar(self, x):
        return int(getattr(self.lib, self._pre + "f32_to_f16")(float(x)))

    def f16_to_f32_scalar(self, h):
        return float(getattr(self.lib, self._pre + "f16_to_f32")(int(h)))

    # ---- RoPE --------------------------------------------------------
    def rope(self, x, pos, theta, n_rot_pairs=0):
        x = np.ascontiguousarray(x, dtype=np.float32)
        seq, heads, hd = x.shape
        out = np.empty_like(x)
        fn = getattr(self.lib, self._pre + "rope")
        rc = fn(_ptr(x, _f32p), _ptr(out, _f32p), C.c_uint32(seq), C.c_uint32(heads),
                C.c_uint32(hd), C.c_uint32(pos), C.c_float(theta), C.c_uint32(n_rot_pairs))
        return int(rc), out

    def rope_table(self, pos, hd, theta, n_rot_pairs=0):
        assert self.kind == "port"
        half = hd // 2
        cs = np.empty(half, np.float32)
        sn = np.empty(half, np.float32)
        rot = np.empty(half, np.uint8)
        self.lib.wro_rope_table(C.c_uint32(pos), C.c_uint32(hd), C.c_float(theta),
                                C.c_uint32(n_rot_pairs), _ptr(cs, _f32p),
                                _ptr(sn, _f32p), _ptr(rot, _u8p))
        return cs, sn, rot

    # ---- attention ---------------------------------------------------
    def attention(self, q, k, v, seq_k=None, scale=0.0, window=0, growable=True,
                  max_seq=None):
        """q [sq,Hq,hd] f32|u16, k/v [rows,Hkv,hd] f32|u16 -> (rc, out f32)."""
        q = np.ascontiguousarray(q)
        k = np.ascontiguousarray(k)
        v = np.ascontiguousarray(v)
        sq, hq, hd = q.shape
        cap, hkv, _ = k.shape
        if seq_k is None:
            seq_k = cap
        out = np.zeros((sq, hq, hd), np.float32)
        qd, kd = _dtype_code(q), _dtype_code(k)
        if self.kind == "port":
            rc = self.lib.wro_gqa_attention(
                q.ctypes.data_as(C.c_void_p), qd, k.ctypes.data_as(C.c_void_p),
                v.ctypes.data_as(C.c_void_p), kd, _ptr(out, _f32p), C.c_uint32(sq),
                C.c_uint32(hq), C.c_uint32(hkv), C.c_uint32(hd), C.c_uint32(seq_k),
                C.c_float(scale), C.c_uint32(window),
                C.c_uint32(max_seq if max_seq is not None else self.max_seq))
        else:
            rc = self.lib.refshim_attention(
                q.ctypes.data_as(C.c_void_p), qd, k.ctypes.data_as(C.c_void_p),
                v.ctypes.data_as(C.c_void_p), kd, _ptr(out, _f32p), C.c_uint32(sq),
                C.c_uint32(hq), C.c_uint32(hkv), C.c_uint32(hd), C.c_uint32(cap),
                C.c_uint32(seq_k), C.c_int(1 if growable else 0), C.c_float(scale),
                C.c_uint32(window))
        return int(rc), out

    def decode_batch(self, q, ks, vs, scale=0.0, window=0, threads=1, max_seq=None):
        """q [n,Hq,hd] f32; ks/vs: lists of uint16 [ctx_i,Hkv,hd] -> (rc, out)."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        n, hq, hd = q.shape
        hkv = ks[0].shape[1]
        ks = [np.ascontiguousarray(a, dtype=np.uint16) for a in ks]
        vs = [np.ascontiguousarray(a, dtype=np.uint16) for a in vs]
        kp = (C.c_void_p * n)(*[a.ctypes.data for a in ks])
        vp = (C.c_void_p * n)(*[a.ctypes.data for a in vs])
        lens = np.array([a.shape[0] for a in ks], dtype=np.uint32)
        out = np.zeros_like(q)
        if self.kind == "port":
            rc = self.lib.wro_decode_batch(
                _ptr(q, _f32p), kp, vp, _ptr(lens, _u32p), _ptr(out, _f32p),
                C.c_uint32(n), C.c_uint32(hq), C.c_uint32(hkv), C.c_uint32(hd),
                C.c_float(scale), C.c_uint32(window),
                C.c_uint32(max_seq if max_seq is not None else self.max_seq),
                C.c_int(threads))
        else:
            rc = self.lib.refshim_decode_batch(
                _ptr(q, _f32p), kp, vp, _ptr(lens, _u32p), _ptr(out, _f32p),
                C.c_uint32(n), C.c_uint32(hq), C.c_uint32(hkv), C.c_uint32(hd),
                C.c_float(scale), C.c_uint32(window), C.c_int(threads))
        return int(rc), out

    def causal_prefill_rows(self, q, k, v, rows, p0=0, scale=0.0, window=0,
                            threads=1, max_seq=None):
        """Rows i of a causal prefill: q [n,Hq,hd], k/v uint16 [p0+n,Hkv,hd]."""
        q = np.ascontiguousarray(q)
        k = np.ascontiguousarray(k, dtype=np.uint16)
        v = np.ascontiguousarray(v, dtype=np.uint16)
        n, hq, hd = q.shape
        hkv = k.shape[1]
        rows = np.ascontiguousarray(rows, dtype=np.uint32)
        out = np.zeros((rows.size, hq, hd), np.float32)
        qd = _dtype_code(q)
        if self.kind == "port":
            rc = self.lib.wro_causal_prefill_rows(
                q.ctypes.data_as(C.c_void_p), qd, _ptr(k, _u16p), _ptr(v, _u16p),
                _ptr(out, _f32p), C.c_uint32(n), C.c_uint32(p0), _ptr(rows, _u32p),
                C.c_uint32(rows.size), C.c_uint32(hq), C.c_uint32(hkv), C.c_uint32(hd),
                C.c_float(scale), C.c_uint32(window),
                C.c_uint32(max_seq if max_seq is not None else self.max_seq),
                C.c_int(threads))
        else:
            rc = self.lib.refshim_causal_prefill_rows(
                q.ctypes.data_as(C.c_void_p), qd, _ptr(k, _u16p), _ptr(v, _u16p),
                _ptr(out, _f32p), C.c_uint32(n), C.c_uint32(p0), _ptr(rows, _u32p),
                C.c_uint32(rows.size), C.c_uint32(hq), C.c_uint32(hkv), C.c_uint32(hd),
                C.c_float(scale), C.c_uint32(window), C.c_int(threads))
        return int(rc), out

    def partial(self, q, k, v, key_lo, key_hi, scale=0.0):
        """(m, l, o) of one decode row over keys [key_lo, key_hi); port only."""
        assert self.kind == "port"
        q = np.ascontiguousarray(q, dtype=np.float32)
        k = np.ascontiguousarray(k, dtype=np.uint16)
        v = np.ascontiguousarray(v, dtype=np.uint16)
        hq, hd = q.shape[-2:]
        hkv = k.shape[1]
        m = np.empty(hq, np.float32)
        l = np.empty(hq, np.float32)
        o = np.empty((hq, hd), np.float32)
        rc = self.lib.wro_gqa_partial(_ptr(q, _f32p), _ptr(k, _u16p), _ptr(v, _u16p),
                                      _ptr(m, _f32p), _ptr(l, _f32p), _ptr(o, _f32p),
                                      C.c_uint32(hq), C.c_uint32(hkv), C.c_uint32(hd),
                                      C.c_uint32(key_lo), C.c_uint32(key_hi),
                                      C.c_float(scale))
        return int(rc), m, l, o


_cache: dict = {}


def restatement() -> Checker:
    """The C restatement (liboracle.so); built on demand with gcc."""
    if "port" not in _cache:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True,
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
        _cache["port"] = Checker(path, "port")
    return _cache["port"]


def reference(long_context: bool = False):
    """The compiled reference, or None where oracle/_ref was never built."""
    key = "ref_long" if long_context else "ref"
    if key not in _cache:
        name = "libwayruntime_ref_long.so" if long_context else "libwayruntime_ref.so"
        path = os.path.join(_HERE, "_ref", name)
        _cache[key] = Checker(path, "reference") if os.path.exists(path) else None
    return _cache[key]
