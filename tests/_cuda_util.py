"""Helpers for the GPU parity tests: build device caches from numpy arrays."""
import numpy as np

import oracle
import wayruntime_b200 as wr

TOL = 2e-3   # max-abs attention-output error allowed against the reference CPU path


def port():
    return oracle.restatement()


def make_cache(ctx, k16, v16, max_ctx=None, n_layers=1, layer=0):
    """A KVCache holding uint16 rows k16/v16 [n, Hkv, hd] in `layer`."""
    n, hkv, hd = k16.shape
    kv = ctx.kv_create(n_layers, hkv, hd, max_ctx or max(n, 1))
    if n:
        kv.write_rows(layer, 0, 0, np.ascontiguousarray(k16))
        kv.write_rows(layer, 1, 0, np.ascontiguousarray(v16))
    return kv


def decode(ctx, kvs, lens, q, hq, scale=0.0, window=0, layer=0):
    out = np.full(q.shape, np.nan, np.float32)
    ctx.attn_decode(kvs, layer, lens, np.ascontiguousarray(q), out, hq, scale=scale, window=window)
    return out
