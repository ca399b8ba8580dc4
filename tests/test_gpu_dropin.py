"""GPU: the B200 session objects as a drop-in inside the reference library.

`wayruntime_b200/lib/libwayruntime_b200.so` is the reference built WITHOUT its
session.c / batch.c, with wayruntime_b200/host/wr_b200_session.c linked in
their place and the engine gate of wr_b200_engine.c in front of its
wr_engine_create (wayruntime_b200/host/Makefile); `oracle/_ref/libwayruntime_ref*.so`
is the unmodified reference.  Both are driven through the reference's public API
(include/wayruntime/wayruntime.h) on the same seeded GGUF and token ids:
  * teacher-forced greedy decoding, with the layer glue on the device (the
    default) and on the host (WR_B200_GLUE=host), the prompt through the prefill
    kernel and token by token: identical argmax at every step, logits
    within tolerance (benchmark config 1: Qwen3-0.6B shape, 64-token prompt),
    and every layer's attention output of every token within tolerance: the
    reference's rows are captured by `libwayruntime_ref_tap.so` (same sources,
    the session code's attention calls routed through a hook by the linker),
    the device rows by the session objects' own observer;
  * batched step byte-equal to serial steps (test/sdk_gen.c:209-279 contract);
  * cursor / CTX_FULL / refusal semantics (src/core/session.c:888-999);
  * a gemma4-class model (sliding-window and shared-KV layers, per-layer head_dim,
    per-layer-input embeddings): the same teacher-forced and batched checks.
Skipped where the two libraries were not built (they are built where the
reference checkout exists and travel with the repository snapshot).
"""
import ctypes as C
import os
import tempfile

import numpy as np
import pytest

import _mkgguf

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "libwayruntime_ref_tap.so")
B200 = os.path.join(ROOT, "wayruntime_b200", "lib", "libwayruntime_b200.so")


REF_TAP = C.CFUNCTYPE(None, C.c_void_p, C.c_uint32, C.POINTER(C.c_float), C.c_uint32)
B200_TAP = C.CFUNCTYPE(None, C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(C.c_float), C.c_uint32)


class Lib:
    def __init__(self, path):
        L = self.L = C.CDLL(path)
        L.wr_engine_create.restype = C.c_int
        L.wr_model_load.restype = C.c_int
        L.wr_session_create.restype = C.c_int
        L.wr_prefill.restype = C.c_int
        L.wr_step.restype = C.POINTER(C.c_float)
        L.wr_batch_step.restype = C.c_int
        L.wr_session_pos.restype = C.c_uint32
        L.wr_session_status.restype = C.c_int
        self.engine = C.c_void_p()
        cfg = (C.c_uint8 * 512)()
        assert L.wr_engine_create(cfg, C.byref(self.engine)) == 0

    def load(self, path):
        m = C.c_void_p()
        params = (C.c_uint8 * 512)()
        rc = self.L.wr_model_load(self.engine, path.encode(), params, C.byref(m))
        assert rc == 0, rc
        return m

    def session(self, model):
        s = C.c_void_p()
        rc = self.L.wr_session_create(model, None, C.byref(s))
        assert rc == 0, rc
        return s

    def prefill(self, s, ids):
        arr = (C.c_uint32 * len(ids))(*ids)
        return self.L.wr_prefill(s, arr, len(ids))

    def step(self, s, tok, vocab):
        p = self.L.wr_step(s, C.c_uint32(tok))
        return None if not p else np.ctypeslib.as_array(p, (vocab,)).copy()


@pytest.fixture(scope="module")
def libs():
    if not (os.path.exists(REF) and os.path.exists(B200)):
        pytest.skip("the drop-in library and the compiled reference were not built on this machine")
    return Lib(REF), Lib(B200)


def test_session_self_tests_pass_on_device(libs):
    _ref, b = libs
    assert b.L.wri_self_test_llm_step() == 0
    assert b.L.wri_self_test_batch_step() == 0


RUNS = (("device", "kernel"), ("device", "decode"), ("host", "kernel"), ("host", "decode"))


def _teacher_forced(libs, shape, n_prompt, n_steps, seed, logit_tol, attn_tol=2e-3, runs=RUNS,
                    writer=_mkgguf.write_qwen3):
    ref, b = libs
    vocab = shape["vocab"]
    path = os.path.join(tempfile.mkdtemp(prefix="wr_gguf_"), "model.gguf")
    writer(path, seed=seed, **shape)
    rng = np.random.Generator(np.random.Philox(seed + 1))
    prompt = [int(x) for x in rng.integers(0, vocab, n_prompt)]
    out = {}
    # the reference first: its greedy ids drive every other run (teacher forcing)
    ref_rows, seen = {}, {}

    def on_ref(_user, seq_k, data, n):          # calls for one token arrive in layer order
        layer = seen.get(seq_k, 0)
        seen[seq_k] = layer + 1
        ref_rows[(layer, seq_k - 1)] = np.ctypeslib.as_array(data, (n,)).copy()

    ref_cb = REF_TAP(on_ref)
    ref.L.refshim_set_attn_tap(ref_cb, None)
    m = ref.load(path)
    s = ref.session(m)
    assert ref.prefill(s, prompt[:-1]) == n_prompt - 1
    ids, ref_logits, tok = [], [], prompt[-1]
    for _ in range(n_steps):
        lg = ref.step(s, tok, vocab)
        assert lg is not None
        ref_logits.append(lg)
        tok = int(lg.argmax())
        ids.append(tok)
    ref.L.wr_session_destroy(s)
    ref.L.wr_model_free(m)
    ref.L.refshim_set_attn_tap(REF_TAP(0), None)
    assert len(ref_rows) == shape["n_layers"] * (n_prompt - 1 + n_steps)
    attn = {"worst": 0.0, "rows": 0}

    def on_b200(_user, layer, pos, data, n):
        got = np.ctypeslib.as_array(data, (n,))
        attn["worst"] = max(attn["worst"], float(np.abs(got - ref_rows[(layer, pos)]).max()))
        attn["rows"] += 1

    b_cb = B200_TAP(on_b200)
    b.L.wr_b200_set_attn_tap(b_cb, None)
    mb = b.load(path)
    for glue, pf in runs:
        mode = f"{glue}/{pf}"
        os.environ["WR_B200_PREFILL"] = pf
        os.environ["WR_B200_GLUE"] = glue               # read when the session is created
        sb = b.session(mb)
        assert b.prefill(sb, prompt[:-1]) == n_prompt - 1
        assert b.L.wr_session_pos(sb) == n_prompt - 1
        tok, same, worst, margins = prompt[-1], 0, 0.0, []
        for t in range(n_steps):
            lg = b.step(sb, tok, vocab)
            assert lg is not None, b.L.wr_session_status(sb)
            worst = max(worst, float(np.abs(lg - ref_logits[t]).max()))
            top2 = np.partition(ref_logits[t], -2)[-2:]
            margins.append(float(top2[1] - top2[0]))
            same += int(lg.argmax() == ids[t])
            tok = ids[t]                                   # teacher forcing with the reference's ids
        b.L.wr_session_destroy(sb)
        out[mode] = (same, worst, min(margins))
        # per-layer attention outputs of every prompt and generated token (the hidden states
        # entering attention already differ by earlier layers' rounding, hence not 1e-6)
        assert attn["rows"] == len(ref_rows), (mode, attn)
        assert attn["worst"] <= attn_tol, (mode, attn)
        out[mode] += (attn["worst"],)
        attn.update(worst=0.0, rows=0)
    b.L.wr_b200_set_attn_tap(B200_TAP(0), None)
    os.environ.pop("WR_B200_PREFILL", None)
    os.environ.pop("WR_B200_GLUE", None)
    b.L.wr_model_free(mb)
    os.remove(path)
    print("teacher-forced parity (argmax matches, worst logit err, min top-2 margin, worst attn err):", out)
    for mode, (same, worst, margin, _attn) in out.items():
        assert worst <= logit_tol, (mode, worst, margin)
        assert same == n_steps, (mode, same, n_steps, worst, margin)
    return out


def test_small_model_teacher_forced_argmax(libs):
    shape = dict(n_layers=2, hidden=256, n_q=4, n_kv=2, head_dim=128, ffn=512, vocab=1000)
    _teacher_forced(libs, shape, n_prompt=40, n_steps=24, seed=11, logit_tol=2e-3)


def test_config1_qwen3_0p6b_shape(libs):
    """benchmark config 1: 28 layers, hidden 1024, 16 Q / 8 KV heads, head_dim 128,
    theta 1e6, QK-norm, SwiGLU 3072, vocab 151936, F16 weights ~N(0, 0.02);
    64-token prompt, then 128 teacher-forced greedy steps (24 with
    WR_TEST_QUICK=1: each step is a full CPU forward in both libraries)."""
    shape = dict(n_layers=28, hidden=1024, n_q=16, n_kv=8, head_dim=128, ffn=3072, vocab=151936)
    steps = 24 if os.environ.get("WR_TEST_QUICK") == "1" else 128
    _teacher_forced(libs, shape, n_prompt=64, n_steps=steps, seed=20261125, logit_tol=2e-3,
                    runs=(("device", "kernel"), ("device", "decode"), ("host", "kernel")))


GEMMA = dict(n_layers=6, hidden=256, n_q=4, n_kv=2, head_dim=128, head_dim_swa=64,
             ffn=[512, 384, 512, 384, 512, 512], vocab=600, swa_pattern=[1, 1, 0, 1, 1, 0], sliding_window=16,
             shared_kv_layers=2, pl_emb=32)


def test_gemma_class_model_teacher_forced(libs):
    """A gemma4-class model (src/core/session.c:251-437): sliding-window layers of head_dim 64 with
    their own RoPE base and a 16-key window, global layers of head_dim 128 with partial rotary, the
    last two layers attending over the caches of layers 1 and 2, sandwich norms, GeGLU, per-layer
    FFN width, per-layer-input embeddings, embedding scale, logit soft-cap, attention scale 1.  A
    40-token prompt (longer than the window) and 24 teacher-forced steps: every layer's attention
    rows within tolerance, logits within tolerance, argmax identical."""
    _teacher_forced(libs, GEMMA, n_prompt=40, n_steps=24, seed=77, logit_tol=2e-3,
                    runs=(("host", "decode"),), writer=_mkgguf.write_gemma4)


def test_gemma_class_batched_step_is_byte_equal_to_serial(libs):
    _ref, b = libs
    path = os.path.join(tempfile.mkdtemp(prefix="wr_gguf_"), "model.gguf")
    _mkgguf.write_gemma4(path, seed=78, **GEMMA)
    m = b.load(path)
    n, vocab = 4, GEMMA["vocab"]
    prompts = [[(7 * i + 3 * j + 1) % vocab for j in range(5 + 11 * i)] for i in range(n)]
    serial, batched = [b.session(m) for _ in range(n)], [b.session(m) for _ in range(n)]
    for s1, s2, p in zip(serial, batched, prompts):
        assert b.prefill(s1, p) == len(p) and b.prefill(s2, p) == len(p)
    for t in range(4):
        toks = [(11 * i + t) % vocab for i in range(n)]
        want = [b.step(s, tok, vocab) for s, tok in zip(serial, toks)]
        arr = (C.c_void_p * n)(*[s.value for s in batched])
        tk = (C.c_uint32 * n)(*toks)
        outp = (C.POINTER(C.c_float) * n)()
        assert b.L.wr_batch_step(arr, tk, n, outp) == n
        for i in range(n):
            got = np.ctypeslib.as_array(outp[i], (vocab,))
            assert np.array_equal(got.view(np.uint32), want[i].view(np.uint32)), (t, i)
    for s in serial + batched:
        b.L.wr_session_destroy(s)
    b.L.wr_model_free(m)
    os.remove(path)


@pytest.mark.parametrize("glue", ["device", "host"])
def test_batched_step_is_byte_equal_to_serial(libs, glue, monkeypatch):
    _ref, b = libs
    monkeypatch.setenv("WR_B200_GLUE", glue)
    shape = dict(n_layers=2, hidden=256, n_q=8, n_kv=2, head_dim=128, ffn=512, vocab=777)
    path = os.path.join(tempfile.mkdtemp(prefix="wr_gguf_"), "model.gguf")
    _mkgguf.write_qwen3(path, seed=5, **shape)
    m = b.load(path)
    n, vocab = 5, shape["vocab"]
    prompts = [[(7 * i + 3 * j + 1) % vocab for j in range(10 + 9 * i)] for i in range(n)]
    serial, batched = [b.session(m) for _ in range(n)], [b.session(m) for _ in range(n)]
    for s1, s2, p in zip(serial, batched, prompts):
        assert b.prefill(s1, p) == len(p) and b.prefill(s2, p) == len(p)
    for t in range(6):
        toks = [(11 * i + t) % vocab for i in range(n)]
        want = [b.step(s, tok, vocab) for s, tok in zip(serial, toks)]
        arr = (C.c_void_p * n)(*[s.value for s in batched])
        tk = (C.c_uint32 * n)(*toks)
        outp = (C.POINTER(C.c_float) * n)()
        assert b.L.wr_batch_step(arr, tk, n, outp) == n
        for i in range(n):
            got = np.ctypeslib.as_array(outp[i], (vocab,))
            assert np.array_equal(got.view(np.uint32), want[i].view(np.uint32)), (t, i)
    for s in serial + batched:
        b.L.wr_session_destroy(s)
    b.L.wr_model_free(m)
    os.remove(path)
