"""GPU: the device-resident layer stack (wr_cuda_model) against numpy.

The stack restates the reference's decode body around attention
(src/core/session.c:405-568).  Whole-model parity with the reference library
is covered by the drop-in tests; here each piece outside attention is checked
on its own, in float64 numpy, using the attention rows the call itself reports
(attn_tap_out) as the fixed point in the middle of a layer:
    hidden_out = embed + attn @ wo^T + FFN(RMSNorm(.))   (one layer)
    normed_out = RMSNorm(hidden_out) * final_norm
    logits     = normed_out @ lm_head^T,  argmax = first maximum
and the K rows that reach the cache are RMSNorm(embed) @ wk^T with QK-norm and
RoPE (the reference's rotation, through the CPU restatement).  Row-count
independence — a row's bits do not depend on how many rows share the call — is
what keeps a batched step byte-equal to serial ones (src/core/batch.c).
"""
import numpy as np
import pytest

import _gen

pytestmark = pytest.mark.gpu

SHAPE = dict(n_layers=1, hidden=256, n_q_heads=4, n_kv_heads=2, head_dim=128, vocab=1003, ffn=520)
EPS = 1e-6


def _weights(shape, seed, tied=True, qk_norm=True):
    hid, nq, nkv = shape["hidden"], shape["n_q_heads"] * shape["head_dim"], shape["n_kv_heads"] * shape["head_dim"]
    ffn, vocab, hd = shape["ffn"], shape["vocab"], shape["head_dim"]
    w = {"embed": _gen.normal(seed, (vocab, hid), 0.5), "final_norm": 1.0 + _gen.normal(seed + 1, (hid,), 0.1)}
    w["lm_head"] = w["embed"] if tied else _gen.normal(seed + 2, (vocab, hid), 0.05)
    for i in range(shape["n_layers"]):
        s = seed + 100 * (i + 1)
        w[f"l{i}.attn_norm"] = 1.0 + _gen.normal(s, (hid,), 0.1)
        w[f"l{i}.ffn_norm"] = 1.0 + _gen.normal(s + 1, (hid,), 0.1)
        w[f"l{i}.wq"] = _gen.normal(s + 2, (nq, hid), 0.05)
        w[f"l{i}.wk"] = _gen.normal(s + 3, (nkv, hid), 0.05)
        w[f"l{i}.wv"] = _gen.normal(s + 4, (nkv, hid), 0.05)
        w[f"l{i}.wo"] = _gen.normal(s + 5, (hid, nq), 0.05)
        w[f"l{i}.w_gate"] = _gen.normal(s + 6, (ffn, hid), 0.05)
        w[f"l{i}.w_up"] = _gen.normal(s + 7, (ffn, hid), 0.05)
        w[f"l{i}.w_down"] = _gen.normal(s + 8, (hid, ffn), 0.05)
        if qk_norm:
            w[f"l{i}.q_norm"] = 1.0 + _gen.normal(s + 9, (hd,), 0.1)
            w[f"l{i}.k_norm"] = 1.0 + _gen.normal(s + 10, (hd,), 0.1)
    return {k: np.ascontiguousarray(v, np.float32) for k, v in w.items()}


def _rms(x, w, eps=EPS):
    x = x.astype(np.float64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * w.astype(np.float64)


def _after_attention(w, resid, attn, i=0):
    """The rest of layer i in float64, from the residual entering it and its attention rows."""
    r = resid.astype(np.float64) + attn.astype(np.float64) @ w[f"l{i}.wo"].astype(np.float64).T
    x = _rms(r, w[f"l{i}.ffn_norm"])
    g = x @ w[f"l{i}.w_gate"].astype(np.float64).T
    u = x @ w[f"l{i}.w_up"].astype(np.float64).T
    return r + (g / (1.0 + np.exp(-g)) * u) @ w[f"l{i}.w_down"].astype(np.float64).T


def _model(ctx, w, shape, **kw):
    import wayruntime_b200 as wr
    return wr.DeviceModel(ctx, w, rms_eps=EPS, rope_theta=1e6, **shape, **kw)


@pytest.mark.parametrize("rows", [1, 3, 16])
def test_decode_rows_match_numpy_piecewise(rows):
    import wayruntime_b200 as wr
    ctx = wr.Context(0)
    w = _weights(SHAPE, 900)
    dm = _model(ctx, w, SHAPE)
    kvs = [ctx.kv_create(1, SHAPE["n_kv_heads"], SHAPE["head_dim"], 64) for _ in range(rows)]
    tokens = [(37 * r + 5) % SHAPE["vocab"] for r in range(rows)]
    # two steps, so that the second attends over two keys
    dm.forward(dm.FWD_DECODE, kvs, [0] * rows, tokens)
    tokens2 = [(11 * r + 2) % SHAPE["vocab"] for r in range(rows)]
    res = dm.forward(dm.FWD_DECODE, kvs, [1] * rows, tokens2, hidden=True, normed=True, logits=True,
                     argmax=True, attn_tap=True)
    emb = w["embed"][tokens2]
    want_hidden = _after_attention(w, emb, res["attn"][0])
    assert np.abs(res["hidden"] - want_hidden).max() <= 2e-4 * max(1.0, np.abs(want_hidden).max())
    want_normed = _rms(res["hidden"], w["final_norm"])
    assert np.abs(res["normed"] - want_normed).max() <= 1e-4
    want_logits = res["normed"].astype(np.float64) @ w["lm_head"].astype(np.float64).T
    assert np.abs(res["logits"] - want_logits).max() <= 1e-4 * max(1.0, np.abs(want_logits).max())
    assert list(res["argmax"]) == [int(np.argmax(row)) for row in res["logits"]]
    # V rows reach the cache as trunc_f16(RMSNorm(embed) @ wv^T) (no rotation on V)
    from _cuda_util import port
    P = port()
    x = _rms(emb, w["l0.attn_norm"])
    want_v = (x @ w["l0.wv"].astype(np.float64).T).astype(np.float32)
    got_v = P.f16_to_f32(kvs[0].read_rows(0, 1, 1, 1)).reshape(-1)
    assert np.abs(got_v - want_v[0]).max() <= 2e-3 * max(1.0, np.abs(want_v[0]).max())
    for kv in kvs:
        kv.close()
    dm.close()
    ctx.close()


def test_a_rows_bits_do_not_depend_on_the_batch():
    import wayruntime_b200 as wr
    ctx = wr.Context(0)
    w = _weights(SHAPE, 901)
    dm = _model(ctx, w, SHAPE)
    n = 7
    tokens = [(91 * r + 13) % SHAPE["vocab"] for r in range(n)]
    serial = []
    for r in range(n):
        kv = ctx.kv_create(1, SHAPE["n_kv_heads"], SHAPE["head_dim"], 16)
        serial.append(dm.forward(dm.FWD_DECODE, [kv], [0], [tokens[r]], logits=True)["logits"][0])
        kv.close()
    kvs = [ctx.kv_create(1, SHAPE["n_kv_heads"], SHAPE["head_dim"], 16) for _ in range(n)]
    batched = dm.forward(dm.FWD_DECODE, kvs, [0] * n, tokens, logits=True)["logits"]
    for r in range(n):
        assert np.array_equal(batched[r].view(np.uint32), serial[r].view(np.uint32)), r
    for kv in kvs:
        kv.close()
    dm.close()
    ctx.close()


def test_prefill_rows_match_token_by_token_decode():
    """40 prompt rows in one pass (three row groups of the GEMV, the tensor-core
    prefill kernel) against the same tokens fed one at a time (decode kernel)."""
    import wayruntime_b200 as wr
    ctx = wr.Context(0)
    shape = dict(SHAPE, n_layers=2)
    w = _weights(shape, 902, tied=False)
    dm = _model(ctx, w, shape, max_rows=64)
    n = 40
    tokens = [(17 * r + 3) % shape["vocab"] for r in range(n)]
    kv_a = ctx.kv_create(2, shape["n_kv_heads"], shape["head_dim"], 64)
    kv_b = ctx.kv_create(2, shape["n_kv_heads"], shape["head_dim"], 64)
    one = dm.forward(dm.FWD_PREFILL, [kv_a], [0], tokens, out_from=n - 1, hidden=True, logits=True)
    for r in range(n):
        last = dm.forward(dm.FWD_DECODE, [kv_b], [r], [tokens[r]], hidden=True, logits=True)
    assert np.abs(one["hidden"] - last["hidden"]).max() <= 2e-3 * max(1.0, np.abs(last["hidden"]).max())
    assert np.abs(one["logits"] - last["logits"]).max() <= 2e-3 * max(1.0, np.abs(last["logits"]).max())
    kv_a.close()
    kv_b.close()
    dm.close()
    ctx.close()


def test_argmax_takes_the_first_maximum_and_bad_tokens_are_refused():
    import wayruntime_b200 as wr
    ctx = wr.Context(0)
    shape = dict(SHAPE)
    w = _weights(shape, 903, tied=False, qk_norm=False)
    # rows 10 and 500 of the LM head are equal and dominant: their logits tie, the lower id must win
    w["lm_head"][500] = w["lm_head"][10] = 4.0 * np.sign(_gen.normal(7, (shape["hidden"],)))
    dm = _model(ctx, w, shape)
    kv = ctx.kv_create(1, shape["n_kv_heads"], shape["head_dim"], 16)
    res = dm.forward(dm.FWD_DECODE, [kv], [0], [5], logits=True, argmax=True)
    lg = res["logits"][0]
    assert lg[10] == lg[500]
    top = int(res["argmax"][0])
    assert top == int(np.argmax(lg))
    if lg[10] == lg.max():
        assert top == 10
    with pytest.raises(wr.WrCudaError) as e:
        dm.forward(dm.FWD_DECODE, [kv], [1], [shape["vocab"]], logits=True)
    assert e.value.status == -4
    res = dm.forward(dm.FWD_DECODE, [kv], [1], [6], logits=True)          # nothing was consumed
    assert np.isfinite(res["logits"]).all()
    assert dm.launches > 0 and dm.device_bytes > 0
    kv.close()
    dm.close()
    ctx.close()


def _prefill(dm, kv, tokens, chunk=64):
    done = 0
    while done < len(tokens):
        part = tokens[done:done + chunk]
        dm.forward(dm.FWD_PREFILL, [kv], [done], part, out_from=len(part))
        done += len(part)


def test_short_context_step_kernel_matches_the_three_kernel_path(monkeypatch):
    """Sessions of at most 1024 keys take QK-norm + RoPE + append + attention in one
    kernel; the same steps through head-norm / append / split-KV decode kernels must
    store the same cache bytes (layer 0, whose inputs are identical) and give the
    same logits within the attention tolerance."""
    import wayruntime_b200 as wr
    ctx = wr.Context(0)
    shape = dict(SHAPE, n_layers=2)
    w = _weights(shape, 905)
    dm = _model(ctx, w, shape, max_rows=64)
    lens = [5, 70, 130]
    out = {}
    for mode in ("one_kernel", "three_kernels"):
        if mode == "three_kernels":
            monkeypatch.setenv("WR_CUDA_STEP_SMALL_OFF", "1")
        kvs = [ctx.kv_create(2, shape["n_kv_heads"], shape["head_dim"], 256) for _ in lens]
        for kv, n in zip(kvs, lens):
            _prefill(dm, kv, [(13 * i + n) % shape["vocab"] for i in range(n)])
        steps = []
        for t in range(3):
            toks = [(7 * i + t + 1) % shape["vocab"] for i in range(len(lens))]
            steps.append(dm.forward(dm.FWD_DECODE, kvs, [n + t for n in lens], toks, logits=True, attn_tap=True))
        rows = [(kv.read_rows(0, 0, n, 3), kv.read_rows(0, 1, n, 3)) for kv, n in zip(kvs, lens)]
        out[mode] = (steps, rows)
        for kv in kvs:
            kv.close()
    monkeypatch.delenv("WR_CUDA_STEP_SMALL_OFF")
    for (ka, va), (kb, vb) in zip(out["one_kernel"][1], out["three_kernels"][1]):
        assert np.array_equal(ka, kb) and np.array_equal(va, vb)            # cache bytes of layer 0
    for a, b in zip(out["one_kernel"][0], out["three_kernels"][0]):
        assert np.abs(a["attn"][0] - b["attn"][0]).max() <= 2e-3
        assert np.abs(a["logits"] - b["logits"]).max() <= 2e-3 * max(1.0, np.abs(b["logits"]).max())
    dm.close()
    ctx.close()


def test_mixed_short_and_long_sessions_in_one_batch_stay_byte_equal_to_serial():
    """Sessions beyond 1024 keys keep the split-KV kernels; a batch that mixes both
    kinds reorders its rows internally.  Every row must still carry the bits it has
    when its session steps alone."""
    import wayruntime_b200 as wr
    ctx = wr.Context(0)
    shape = dict(SHAPE)
    w = _weights(shape, 906)
    dm = _model(ctx, w, shape, max_rows=256)
    lens = [1100, 10, 1300, 3, 1024]
    toks = [(31 * i + 7) % shape["vocab"] for i in range(len(lens))]

    def sessions():
        kvs = [ctx.kv_create(1, shape["n_kv_heads"], shape["head_dim"], 1536) for _ in lens]
        for kv, n in zip(kvs, lens):
            _prefill(dm, kv, [(11 * i + n) % shape["vocab"] for i in range(n)], chunk=256)
        return kvs

    a = sessions()
    serial = [dm.forward(dm.FWD_DECODE, [kv], [n], [t], logits=True, hidden=True, argmax=True)
              for kv, n, t in zip(a, lens, toks)]
    b = sessions()
    batched = dm.forward(dm.FWD_DECODE, b, lens, toks, logits=True, hidden=True, argmax=True, normed=True)
    for i in range(len(lens)):
        assert np.array_equal(batched["logits"][i].view(np.uint32), serial[i]["logits"][0].view(np.uint32)), i
        assert np.array_equal(batched["hidden"][i].view(np.uint32), serial[i]["hidden"][0].view(np.uint32)), i
        assert batched["argmax"][i] == serial[i]["argmax"][0]
    # a partial output range on a reordered batch: rows 2.. only
    c = sessions()
    part = dm.forward(dm.FWD_DECODE, c, lens, toks, out_from=2, logits=True, argmax=True)
    for i in range(2, len(lens)):
        assert np.array_equal(part["logits"][i - 2].view(np.uint32), serial[i]["logits"][0].view(np.uint32)), i
    for kv in a + b + c:
        kv.close()
    dm.close()
    ctx.close()
