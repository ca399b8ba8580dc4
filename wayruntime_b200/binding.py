"""ctypes mirror of include/wr_cuda.h.

Argument meaning and error behaviour are the C-ABI's: every call returns a
``wr_status`` value, and a negative one is raised as :class:`WrCudaError`
carrying that code.  Buffers may be numpy arrays or CPU torch tensors (host
memory: the call copies and synchronises) or CUDA torch tensors (device
memory: the call only enqueues on the context's stream).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libwr_cuda.so")

MEM_HOST, MEM_DEVICE = 0, 1
F32, F16 = 0, 1
APPEND_ROPE = 1
TRIPLE_PAD = 4
BATCH_MAX = 16

_STATUS = {
    0: "WR_OK", -3: "WR_ERR_UNSUPPORTED", -4: "WR_ERR_INVAL", -5: "WR_ERR_NOMEM",
    -6: "WR_ERR_CTX_FULL", -7: "WR_ERR_STATE", -8: "WR_ERR_LIMIT", -10: "WR_ERR_INTERNAL",
}

EXPORTS = [
    "wr_cuda_device_check", "wr_cuda_ctx_create", "wr_cuda_ctx_destroy", "wr_cuda_ctx_sync",
    "wr_cuda_ctx_stream", "wr_cuda_ctx_set_attn_max_seq", "wr_cuda_ctx_set_wait_limit",
    "wr_cuda_ctx_last_device_error",
    "wr_cuda_ctx_launch_count", "wr_cuda_host_alloc", "wr_cuda_host_free",
    "wr_cuda_kv_create", "wr_cuda_kv_destroy", "wr_cuda_kv_max_ctx", "wr_cuda_kv_write_rows",
    "wr_cuda_kv_read_rows", "wr_cuda_kv_append", "wr_cuda_attn_decode", "wr_cuda_attn_prefill",
    "wr_cuda_attn_decode_partial", "wr_cuda_attn_combine", "wr_cuda_decode_step",
    "wr_cuda_attn_decode_static",
    "wr_cuda_xchg_create", "wr_cuda_xchg_handle", "wr_cuda_xchg_connect", "wr_cuda_xchg_connect_local",
    "wr_cuda_xchg_destroy",
    "wr_cuda_attn_exchange_combine", "wr_cuda_attn_decode_exchange",
    "wr_cuda_model_create", "wr_cuda_model_destroy", "wr_cuda_model_bytes", "wr_cuda_model_launches", "wr_cuda_model_last_enqueue_ns",
    "wr_cuda_model_forward",
]


def status_name(rc: int) -> str:
    return _STATUS.get(rc, f"wr_status({rc})")


class WrCudaError(RuntimeError):
    def __init__(self, rc: int, what: str):
        super().__init__(f"{what}: {status_name(rc)}")
        self.status = rc


class LayerDesc(C.Structure):
    """wr_cuda_layer_desc (include/wr_cuda.h)."""
    _fields_ = [(n, C.c_void_p) for n in ("attn_norm", "wq", "wk", "wv", "q_norm", "k_norm", "wo",
                                          "ffn_norm", "w_gate", "w_up", "w_down")] + \
               [("ffn_dim", C.c_uint32), ("reserved", C.c_uint32)]


class ModelDesc(C.Structure):
    """wr_cuda_model_desc (include/wr_cuda.h)."""
    _fields_ = [(n, C.c_uint32) for n in ("n_layers", "hidden", "n_q_heads", "n_kv_heads", "head_dim",
                                          "vocab", "n_rot_pairs", "max_rows")] + \
               [(n, C.c_float) for n in ("rms_eps", "rope_theta", "attn_scale", "reserved")] + \
               [("embed", C.c_void_p), ("lm_head", C.c_void_p), ("final_norm", C.c_void_p),
                ("layers", C.POINTER(LayerDesc))]


_lib = None


def load_library():
    """Load libwr_cuda.so; raises if it was never built (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; "
            "g.build()'` (needs nvcc); wayruntime_b200 has no CPU path")
    lib = C.CDLL(LIB_PATH)
    vp, u32, i32, f32 = C.c_void_p, C.c_uint32, C.c_int, C.c_float
    sig = {
        "wr_cuda_device_check": (i32, [i32]),
        "wr_cuda_ctx_create": (i32, [i32, C.POINTER(vp)]),
        "wr_cuda_ctx_destroy": (None, [vp]),
        "wr_cuda_ctx_sync": (i32, [vp]),
        "wr_cuda_ctx_stream": (vp, [vp]),
        "wr_cuda_ctx_set_attn_max_seq": (i32, [vp, u32]),
        "wr_cuda_ctx_set_wait_limit": (i32, [vp, C.c_int64]),
        "wr_cuda_ctx_last_device_error": (i32, [vp]),
        "wr_cuda_ctx_launch_count": (C.c_uint64, [vp]),
        "wr_cuda_host_alloc": (i32, [vp, C.c_uint64, C.POINTER(vp)]),
        "wr_cuda_host_free": (None, [vp, vp]),
        "wr_cuda_kv_create": (i32, [vp, u32, u32, u32, u32, C.POINTER(vp)]),
        "wr_cuda_kv_destroy": (None, [vp]),
        "wr_cuda_kv_max_ctx": (u32, [vp]),
        "wr_cuda_kv_write_rows": (i32, [vp, vp, u32, i32, u32, u32, vp, i32]),
        "wr_cuda_kv_read_rows": (i32, [vp, vp, u32, i32, u32, u32, vp, i32]),
        "wr_cuda_kv_append": (i32, [vp, u32, C.POINTER(vp), u32, C.POINTER(u32), u32, vp, vp, vp,
                                    u32, f32, u32, u32, i32]),
        "wr_cuda_attn_decode": (i32, [vp, u32, C.POINTER(vp), u32, C.POINTER(u32), vp, vp, u32,
                                      f32, u32, i32]),
        "wr_cuda_attn_prefill": (i32, [vp, vp, u32, u32, u32, vp, i32, vp, u32, f32, u32, i32]),
        "wr_cuda_attn_decode_partial": (i32, [vp, u32, C.POINTER(vp), u32, C.POINTER(u32), vp, vp,
                                              u32, f32, i32]),
        "wr_cuda_attn_combine": (i32, [vp, u32, u32, u32, vp, vp, i32]),
        "wr_cuda_decode_step": (i32, [vp, u32, C.POINTER(vp), u32, C.POINTER(u32), vp, vp, vp, vp,
                                      u32, f32, u32, u32, f32, u32, i32]),
        "wr_cuda_attn_decode_static": (i32, [vp, u32, C.POINTER(vp), u32, C.POINTER(u32), vp, vp,
                                             u32, f32, u32]),
        "wr_cuda_xchg_create": (i32, [vp, u32, u32, u32, u32, C.POINTER(vp)]),
        "wr_cuda_xchg_handle": (i32, [vp, vp]),
        "wr_cuda_xchg_connect": (i32, [vp, vp]),
        "wr_cuda_xchg_connect_local": (i32, [vp, C.POINTER(vp)]),
        "wr_cuda_xchg_destroy": (None, [vp]),
        "wr_cuda_attn_exchange_combine": (i32, [vp, vp, u32, vp, vp]),
        "wr_cuda_attn_decode_exchange": (i32, [vp, vp, u32, C.POINTER(vp), u32, C.POINTER(u32), vp, vp, u32, f32]),
        "wr_cuda_model_create": (i32, [vp, C.POINTER(ModelDesc), C.POINTER(vp)]),
        "wr_cuda_model_destroy": (None, [vp]),
        "wr_cuda_model_bytes": (C.c_uint64, [vp]),
        "wr_cuda_model_launches": (C.c_uint64, [vp]),
        "wr_cuda_model_last_enqueue_ns": (C.c_uint64, [vp]),
        "wr_cuda_model_forward": (i32, [vp, vp, i32, u32, C.POINTER(vp), C.POINTER(u32), C.POINTER(u32), u32,
                                        vp, vp, C.POINTER(vp), C.POINTER(u32), vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def device_check(device: int = 0) -> int:
    """wr_status: 0 when `device` is an sm_100 GPU, WR_ERR_UNSUPPORTED otherwise."""
    return int(load_library().wr_cuda_device_check(device))


def _buf(x):
    """(address, mem kind, keep-alive) of a numpy array / torch tensor."""
    if x is None:
        return None, None, None
    if isinstance(x, np.ndarray):
        if not x.flags["C_CONTIGUOUS"]:
            raise ValueError("buffers must be C-contiguous")
        return x.ctypes.data, MEM_HOST, x
    if hasattr(x, "data_ptr"):
        if not x.is_contiguous():
            raise ValueError("buffers must be contiguous")
        return x.data_ptr(), (MEM_DEVICE if x.is_cuda else MEM_HOST), x
    raise TypeError(f"unsupported buffer {type(x)}")


def _same_mem(*kinds):
    ks = {k for k in kinds if k is not None}
    if len(ks) != 1:
        raise ValueError("all buffers of one call must live on the same side (host or device)")
    return ks.pop()


def _check(rc, what):
    if rc != 0:
        raise WrCudaError(int(rc), what)


class Context:
    """One device, one stream, one page pool (wr_cuda_ctx)."""

    def __init__(self, device: int = 0, attn_max_seq: int | None = None):
        self._lib = load_library()
        h = C.c_void_p()
        _check(self._lib.wr_cuda_ctx_create(device, C.byref(h)), "wr_cuda_ctx_create")
        self._h = h
        self.device = device
        if attn_max_seq is not None:
            self.set_attn_max_seq(attn_max_seq)

    def close(self):
        if getattr(self, "_h", None):
            self._lib.wr_cuda_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self):
        _check(self._lib.wr_cuda_ctx_sync(self._h), "wr_cuda_ctx_sync")

    @property
    def stream(self) -> int:
        return int(self._lib.wr_cuda_ctx_stream(self._h) or 0)

    @property
    def launch_count(self) -> int:
        return int(self._lib.wr_cuda_ctx_launch_count(self._h))

    def set_attn_max_seq(self, n: int):
        _check(self._lib.wr_cuda_ctx_set_attn_max_seq(self._h, n), "wr_cuda_ctx_set_attn_max_seq")

    @property
    def last_device_error(self) -> int:
        """Error word of the last device-side give-up that was reported (0: none)."""
        return int(self._lib.wr_cuda_ctx_last_device_error(self._h))

    def set_wait_limit(self, cycles: int):
        """SM clock cycles after which a device-side wait gives up (default about 2 s)."""
        _check(self._lib.wr_cuda_ctx_set_wait_limit(self._h, int(cycles)), "wr_cuda_ctx_set_wait_limit")

    def kv_create(self, n_layers, n_kv_heads, head_dim, max_ctx) -> "KVCache":
        return KVCache(self, n_layers, n_kv_heads, head_dim, max_ctx)

    # ---- the hot path -------------------------------------------------
    @staticmethod
    def _handles(kvs):
        if isinstance(kvs, Batch):
            return kvs.handles
        return (C.c_void_p * len(kvs))(*[k._h for k in kvs])

    @staticmethod
    def _u32s(vals):
        if isinstance(vals, C.Array):
            return vals
        return (C.c_uint32 * len(vals))(*[int(v) for v in vals])

    def decode_step(self, kvs, layer, positions, q, k_rows, v_rows, out, n_q_heads, theta=10000.0,
                    n_rot_pairs=0, rope=True, scale=0.0, window=0):
        qp, qm, _q = _buf(q)
        kp, km, _k = _buf(k_rows)
        vp, vm, _v = _buf(v_rows)
        op, om, _o = _buf(out)
        mem = _same_mem(qm, km, vm, om)
        rc = self._lib.wr_cuda_decode_step(self._h, len(kvs), self._handles(kvs), layer,
                                           self._u32s(positions), qp, kp, vp, op, n_q_heads, theta,
                                           n_rot_pairs, APPEND_ROPE if rope else 0, scale, window,
                                           mem)
        _check(rc, "wr_cuda_decode_step")

    def prepared_decode_step(self, kvs, positions, q, k_rows, v_rows, out, n_q_heads, theta=10000.0,
                             n_rot_pairs=0, rope=True, scale=0.0, window=0):
        """wr_cuda_decode_step with everything but the layer resolved once: returns `step(layer)`.
        For a serving loop that steps the same sessions and buffers over and over — the C caller's
        situation, where the arguments are pointers it already holds — so that a call costs the
        library's work and not the marshalling of its arguments.  positions: a list (copied once) or
        a ctypes array from Batch.u32 that the caller updates in place between steps."""
        qp, qm, _q = _buf(q)
        kp, km, _k = _buf(k_rows)
        vp, vm, _v = _buf(v_rows)
        op, om, _o = _buf(out)
        mem = _same_mem(qm, km, vm, om)
        handles, pos = self._handles(kvs), self._u32s(positions)
        n = len(kvs)
        fn, ctx_h = self._lib.wr_cuda_decode_step, self._h
        flags = APPEND_ROPE if rope else 0
        keep = (_q, _k, _v, _o, handles, pos)

        def step(layer, _keep=keep):
            rc = fn(ctx_h, n, handles, layer, pos, qp, kp, vp, op, n_q_heads, theta, n_rot_pairs, flags, scale,
                    window, mem)
            if rc != 0:
                raise WrCudaError(int(rc), "wr_cuda_decode_step")

        return step

    def kv_append(self, kvs, layer, positions, k_rows, v_rows, q_rows=None, n_q_heads=0,
                  theta=10000.0, n_rot_pairs=0, rope=True, n_tokens=1):
        kp, km, _k = _buf(k_rows)
        vp, vm, _v = _buf(v_rows)
        qp, qm, _q = _buf(q_rows)
        mem = _same_mem(km, vm, qm)
        pos = self._u32s(positions)
        rc = self._lib.wr_cuda_kv_append(self._h, len(kvs), self._handles(kvs), layer, pos,
                                         n_tokens, kp, vp, qp, n_q_heads, theta, n_rot_pairs,
                                         APPEND_ROPE if rope else 0, mem)
        _check(rc, "wr_cuda_kv_append")

    def attn_decode(self, kvs, layer, seq_lens, q, out, n_q_heads, scale=0.0, window=0):
        qp, qm, _q = _buf(q)
        op, om, _o = _buf(out)
        mem = _same_mem(qm, om)
        lens = self._u32s(seq_lens)
        rc = self._lib.wr_cuda_attn_decode(self._h, len(kvs), self._handles(kvs), layer, lens, qp,
                                           op, n_q_heads, scale, window, mem)
        _check(rc, "wr_cuda_attn_decode")

    def attn_decode_static(self, kvs, layer, seq_lens, q, out, n_q_heads, scale=0.0, window=0):
        """wr_cuda_attn_decode_static: the decode kernel over the library's fixed
        scratch array, for callers that may not allocate.  q and out must be
        device buffers; oversize calls raise WR_ERR_LIMIT."""
        qp, qm, _q = _buf(q)
        op, om, _o = _buf(out)
        if qm != MEM_DEVICE or om != MEM_DEVICE:
            raise ValueError("wr_cuda_attn_decode_static takes device buffers only")
        rc = self._lib.wr_cuda_attn_decode_static(self._h, len(kvs), self._handles(kvs), layer,
                                                  self._u32s(seq_lens), qp, op, n_q_heads, scale,
                                                  window)
        _check(rc, "wr_cuda_attn_decode_static")

    def attn_decode_partial(self, kvs, layer, seq_lens, q, triples, n_q_heads, scale=0.0):
        qp, qm, _q = _buf(q)
        tp, tm, _t = _buf(triples)
        mem = _same_mem(qm, tm)
        lens = self._u32s(seq_lens)
        rc = self._lib.wr_cuda_attn_decode_partial(self._h, len(kvs), self._handles(kvs), layer,
                                                   lens, qp, tp, n_q_heads, scale, mem)
        _check(rc, "wr_cuda_attn_decode_partial")

    def attn_combine(self, n_shards, n_rows, head_dim, triples, out):
        tp, tm, _t = _buf(triples)
        op, om, _o = _buf(out)
        mem = _same_mem(tm, om)
        rc = self._lib.wr_cuda_attn_combine(self._h, n_shards, n_rows, head_dim, tp, op, mem)
        _check(rc, "wr_cuda_attn_combine")

    def attn_prefill(self, kv, layer, p0, n, q, out, n_q_heads, scale=0.0, window=0):
        qp, qm, qa = _buf(q)
        op, om, _o = _buf(out)
        mem = _same_mem(qm, om)
        if isinstance(qa, np.ndarray):
            q_dtype = F32 if qa.dtype == np.float32 else F16
        else:
            q_dtype = F32 if qa.element_size() == 4 else F16
        rc = self._lib.wr_cuda_attn_prefill(self._h, kv._h, layer, p0, n, qp, q_dtype, op,
                                            n_q_heads, scale, window, mem)
        _check(rc, "wr_cuda_attn_prefill")


XCHG_HANDLE_BYTES = 64


class Exchange:
    """Peer buffers for the fused all-gather + merge of split-KV triples
    (wr_cuda_xchg): create on every rank, pass everybody's `handle` (rank order)
    to `connect`, then call `combine` once per step on every rank."""

    def __init__(self, ctx: "Context", world: int, rank: int, max_rows: int, head_dim: int):
        self._ctx = ctx
        self._lib = ctx._lib
        self.world, self.rank = world, rank
        h = C.c_void_p()
        _check(self._lib.wr_cuda_xchg_create(ctx._h, world, rank, max_rows, head_dim, C.byref(h)),
               "wr_cuda_xchg_create")
        self._h = h

    @property
    def handle(self) -> bytes:
        buf = C.create_string_buffer(XCHG_HANDLE_BYTES)
        _check(self._lib.wr_cuda_xchg_handle(self._h, buf), "wr_cuda_xchg_handle")
        return buf.raw

    def connect(self, handles) -> None:
        blob = b"".join(handles)
        if len(blob) != self.world * XCHG_HANDLE_BYTES:
            raise ValueError("one 64-byte handle per rank, in rank order")
        _check(self._lib.wr_cuda_xchg_connect(self._h, C.c_char_p(blob)), "wr_cuda_xchg_connect")

    @staticmethod
    def connect_local(objs) -> None:
        """Connect exchange objects that live in this process (rank order)."""
        arr = (C.c_void_p * len(objs))(*[o._h for o in objs])
        for o in objs:
            _check(o._lib.wr_cuda_xchg_connect_local(o._h, arr), "wr_cuda_xchg_connect_local")

    def combine(self, n_rows: int, triples, out) -> None:
        tp, tm, _t = _buf(triples)
        op, om, _o = _buf(out)
        if tm != MEM_DEVICE or om != MEM_DEVICE:
            raise ValueError("wr_cuda_attn_exchange_combine takes device buffers only")
        _check(self._lib.wr_cuda_attn_exchange_combine(self._ctx._h, self._h, n_rows, tp, op),
               "wr_cuda_attn_exchange_combine")

    def decode(self, kvs, layer, seq_lens, q, out, n_q_heads, scale=0.0) -> None:
        """wr_cuda_attn_decode_exchange: partial attention over this rank's keys with the
        exchange and the merge fused in (device buffers)."""
        qp, qm, _q = _buf(q)
        op, om, _o = _buf(out)
        if qm != MEM_DEVICE or om != MEM_DEVICE:
            raise ValueError("wr_cuda_attn_decode_exchange takes device buffers only")
        _check(self._lib.wr_cuda_attn_decode_exchange(self._ctx._h, self._h, len(kvs), Context._handles(kvs), layer,
                                                      Context._u32s(seq_lens), qp, op, n_q_heads, scale),
               "wr_cuda_attn_decode_exchange")

    def close(self) -> None:
        if self._h:
            self._lib.wr_cuda_xchg_destroy(self._h)
            self._h = None


class DeviceModel:
    """wr_cuda_model: a model's F32 weights mirrored on the device and the layer
    stack around attention run there.  `weights` maps names to C-contiguous
    float32 numpy arrays in GGML layout (a [in -> out] projection is [out][in]):
    embed, lm_head (may be the same array), final_norm, and per layer i
    `l{i}.attn_norm|wq|wk|wv|q_norm|k_norm|wo|ffn_norm|w_gate|w_up|w_down`."""

    FWD_DECODE, FWD_PREFILL = 0, 1

    def __init__(self, ctx: "Context", weights: dict, *, n_layers, hidden, n_q_heads, n_kv_heads, head_dim,
                 vocab, ffn, rms_eps=1e-6, rope_theta=10000.0, n_rot_pairs=0, attn_scale=0.0, max_rows=256):
        self._ctx, self._lib = ctx, ctx._lib
        self.vocab, self.hidden, self.n_layers = vocab, hidden, n_layers
        self.n_q, self.hd = n_q_heads, head_dim

        def ptr(name, optional=False):
            a = weights.get(name)
            if a is None:
                if optional:
                    return None
                raise KeyError(name)
            if a.dtype != np.float32 or not a.flags["C_CONTIGUOUS"]:
                raise ValueError(f"{name}: C-contiguous float32 expected")
            return a.ctypes.data

        layers = (LayerDesc * n_layers)()
        for i in range(n_layers):
            for f in ("attn_norm", "wq", "wk", "wv", "wo", "ffn_norm", "w_gate", "w_up", "w_down"):
                setattr(layers[i], f, ptr(f"l{i}.{f}"))
            layers[i].q_norm = ptr(f"l{i}.q_norm", optional=True)
            layers[i].k_norm = ptr(f"l{i}.k_norm", optional=True)
            layers[i].ffn_dim = ffn[i] if isinstance(ffn, (list, tuple)) else ffn
        d = ModelDesc(n_layers=n_layers, hidden=hidden, n_q_heads=n_q_heads, n_kv_heads=n_kv_heads,
                      head_dim=head_dim, vocab=vocab, n_rot_pairs=n_rot_pairs, max_rows=max_rows,
                      rms_eps=rms_eps, rope_theta=rope_theta, attn_scale=attn_scale,
                      embed=ptr("embed"), lm_head=ptr("lm_head"), final_norm=ptr("final_norm"), layers=layers)
        h = C.c_void_p()
        _check(self._lib.wr_cuda_model_create(ctx._h, C.byref(d), C.byref(h)), "wr_cuda_model_create")
        self._h = h

    def close(self):
        if self._h:
            self._lib.wr_cuda_model_destroy(self._h)
            self._h = None

    @property
    def device_bytes(self) -> int:
        return int(self._lib.wr_cuda_model_bytes(self._h))

    @property
    def launches(self) -> int:
        return int(self._lib.wr_cuda_model_launches(self._h))

    @property
    def last_enqueue_ms(self) -> float:
        """Host time the last forward pass spent enqueueing work, before waiting for the device."""
        return self._lib.wr_cuda_model_last_enqueue_ns(self._h) * 1e-6

    def forward(self, mode, kvs, positions, tokens, out_from=0, *, hidden=False, normed=False, logits=False,
                argmax=False, attn_tap=False) -> dict:
        """One forward pass; returns the requested results for rows [out_from, n) as numpy arrays."""
        n = len(tokens)
        n_out = n - out_from
        res = {}
        hid = np.empty((n_out, self.hidden), np.float32) if hidden else None
        nrm = np.empty((n_out, self.hidden), np.float32) if normed else None
        lg = np.empty((n_out, self.vocab), np.float32) if logits else None
        am = (C.c_uint32 * max(n_out, 1))() if argmax else None
        tap = np.empty((self.n_layers, n, self.n_q * self.hd), np.float32) if attn_tap else None
        lptrs = (C.c_void_p * max(n_out, 1))(*[lg[i].ctypes.data for i in range(n_out)]) if logits else None
        _check(self._lib.wr_cuda_model_forward(
            self._ctx._h, self._h, mode, n, Context._handles(kvs), Context._u32s(positions),
            Context._u32s(tokens), out_from, hid.ctypes.data if hidden else None,
            nrm.ctypes.data if normed else None, lptrs, am, tap.ctypes.data if attn_tap else None),
            "wr_cuda_model_forward")
        if hidden: res["hidden"] = hid
        if normed: res["normed"] = nrm
        if logits: res["logits"] = lg
        if argmax: res["argmax"] = np.array([am[i] for i in range(n_out)], np.uint32)
        if attn_tap: res["attn"] = tap
        return res


class Batch:
    """A fixed list of sessions with its handle array built once (saves the
    per-call marshalling when the same batch steps many times)."""

    def __init__(self, kvs):
        self.kvs = list(kvs)
        self.handles = (C.c_void_p * len(self.kvs))(*[k._h for k in self.kvs])

    def __len__(self):
        return len(self.kvs)

    @staticmethod
    def u32(vals):
        return (C.c_uint32 * len(vals))(*[int(v) for v in vals])


class KVCache:
    """One session's paged F16 K/V cache (wr_cuda_kv)."""

    def __init__(self, ctx: Context, n_layers, n_kv_heads, head_dim, max_ctx):
        self._ctx = ctx
        self._lib = ctx._lib
        h = C.c_void_p()
        _check(self._lib.wr_cuda_kv_create(ctx._h, n_layers, n_kv_heads, head_dim, max_ctx,
                                           C.byref(h)), "wr_cuda_kv_create")
        self._h = h
        self.n_layers, self.n_kv_heads, self.head_dim, self.max_ctx = (
            n_layers, n_kv_heads, head_dim, max_ctx)

    def close(self):
        if getattr(self, "_h", None) and getattr(self._ctx, "_h", None):
            self._lib.wr_cuda_kv_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def write_rows(self, layer, which, row0, rows):
        """rows: uint16/float16 [n, n_kv_heads, head_dim] in the reference's row layout."""
        p, mem, _a = _buf(rows)
        n = rows.shape[0]
        _check(self._lib.wr_cuda_kv_write_rows(self._ctx._h, self._h, layer, which, row0, n, p, mem),
               "wr_cuda_kv_write_rows")

    def read_rows(self, layer, which, row0, n):
        out = np.empty((n, self.n_kv_heads, self.head_dim), np.uint16)
        _check(self._lib.wr_cuda_kv_read_rows(self._ctx._h, self._h, layer, which, row0, n,
                                              out.ctypes.data, MEM_HOST), "wr_cuda_kv_read_rows")
        return out
