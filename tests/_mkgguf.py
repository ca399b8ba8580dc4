"""Seeded GGUF writers for the whole-model parity tests (benchmark config 1, and a
Gemma-class model for the sliding-window / shared-KV / per-layer-input paths).

Writes a GGUF v3 file with the metadata and tensors the reference loader
demands for a qwen3-class model (src/core/gguf.c:892-1008,
src/core/loader.c:283-429, :522-668): F16 matmul weights ~N(0, std), F32 norm
vectors = 1.0, tied LM head (no output.weight), no tokenizer arrays.
"""
import struct

import numpy as np

GGUF_U32, GGUF_F32, GGUF_BOOL, GGUF_STR, GGUF_ARRAY = 4, 6, 7, 8, 9
T_F32, T_F16 = 0, 1
ALIGN = 32


def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def _kv_u32(key, v):
    return _s(key.encode()) + struct.pack("<II", GGUF_U32, v)


def _kv_f32(key, v):
    return _s(key.encode()) + struct.pack("<If", GGUF_F32, v)


def _kv_str(key, v):
    return _s(key.encode()) + struct.pack("<I", GGUF_STR) + _s(v.encode())


def write_qwen3(path, *, n_layers, hidden, n_q, n_kv, head_dim, ffn, vocab, theta=1e6,
                eps=1e-6, ctx=4096, std=0.02, seed=1234):
    rng = np.random.Generator(np.random.Philox(seed))
    kvs = [
        _kv_str("general.architecture", "qwen3"),
        _kv_u32("qwen3.block_count", n_layers),
        _kv_u32("qwen3.embedding_length", hidden),
        _kv_u32("qwen3.feed_forward_length", ffn),
        _kv_u32("qwen3.attention.head_count", n_q),
        _kv_u32("qwen3.attention.head_count_kv", n_kv),
        _kv_u32("qwen3.attention.key_length", head_dim),
        _kv_u32("qwen3.attention.value_length", head_dim),
        _kv_f32("qwen3.attention.layer_norm_rms_epsilon", eps),
        _kv_f32("qwen3.rope.freq_base", theta),
        _kv_u32("qwen3.context_length", ctx),
    ]
    tensors = [("token_embd.weight", (hidden, vocab), T_F16), ("output_norm.weight", (hidden,), T_F32)]
    for L in range(n_layers):
        p = f"blk.{L}."
        tensors += [
            (p + "attn_norm.weight", (hidden,), T_F32),
            (p + "attn_q.weight", (hidden, n_q * head_dim), T_F16),
            (p + "attn_k.weight", (hidden, n_kv * head_dim), T_F16),
            (p + "attn_v.weight", (hidden, n_kv * head_dim), T_F16),
            (p + "attn_q_norm.weight", (head_dim,), T_F32),
            (p + "attn_k_norm.weight", (head_dim,), T_F32),
            (p + "attn_output.weight", (n_q * head_dim, hidden), T_F16),
            (p + "ffn_norm.weight", (hidden,), T_F32),
            (p + "ffn_gate.weight", (hidden, ffn), T_F16),
            (p + "ffn_up.weight", (hidden, ffn), T_F16),
            (p + "ffn_down.weight", (ffn, hidden), T_F16),
        ]
    infos, off = [], 0
    for name, dims, typ in tensors:          # dims are innermost-first, as GGUF stores them
        n = int(np.prod(dims))
        nbytes = n * (4 if typ == T_F32 else 2)
        infos.append((name, dims, typ, off, n))
        off += (nbytes + ALIGN - 1) // ALIGN * ALIGN
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kvs)) + b"".join(kvs)
    for name, dims, typ, toff, _n in infos:
        head += _s(name.encode()) + struct.pack("<I", len(dims))
        head += b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", typ, toff)
    pad = (-len(head)) % ALIGN
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        for name, dims, typ, toff, n in infos:
            if typ == T_F32:
                buf = np.ones(n, np.float32).tobytes()
            else:
                buf = (rng.standard_normal(n, dtype=np.float32) * np.float32(std)).astype(np.float16).tobytes()
            f.write(buf)
            f.write(b"\0" * ((-len(buf)) % ALIGN))
    return path


def _kv_bool_array(key, vals):
    return (_s(key.encode()) + struct.pack("<IIQ", GGUF_ARRAY, GGUF_BOOL, len(vals)) +
            bytes(1 if v else 0 for v in vals))


def _write(path, kvs, tensors, fill):
    """tensors: (name, dims innermost-first, type); fill(name, n, typ) -> bytes."""
    infos, off = [], 0
    for name, dims, typ in tensors:
        n = int(np.prod(dims))
        nbytes = n * (4 if typ == T_F32 else 2)
        infos.append((name, dims, typ, off, n))
        off += (nbytes + ALIGN - 1) // ALIGN * ALIGN
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kvs)) + b"".join(kvs)
    for name, dims, typ, toff, _n in infos:
        head += _s(name.encode()) + struct.pack("<I", len(dims))
        head += b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", typ, toff)
    pad = (-len(head)) % ALIGN
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        for name, dims, typ, toff, n in infos:
            buf = fill(name, n, typ)
            f.write(buf)
            f.write(b"\0" * ((-len(buf)) % ALIGN))
    return path


def write_gemma4(path, *, n_layers, hidden, n_q, n_kv, head_dim, head_dim_swa, ffn, vocab, swa_pattern,
                 sliding_window, shared_kv_layers, pl_emb, softcap=30.0, theta=1e6, theta_swa=1e4, eps=1e-6,
                 ctx=4096, std=0.05, seed=4321, output_scale=None, zero=()):
    """A gemma4-class model as the reference loader wants it (src/core/loader.c:283-429, :575-627;
    metadata keys src/core/gguf.c:892-940): per-layer head_dim (sliding-window layers use
    head_dim_swa), sandwich norms, per-layer-input tensors, per-layer FFN width (ffn may be a list),
    tied LM head.  Norm vectors are 1 + small noise so that every norm matters."""
    rng = np.random.Generator(np.random.Philox(seed))
    a = "gemma4"
    kvs = [
        _kv_str("general.architecture", a),
        _kv_u32(a + ".block_count", n_layers),
        _kv_u32(a + ".embedding_length", hidden),
        _kv_u32(a + ".feed_forward_length", ffn if isinstance(ffn, int) else max(ffn)),
        _kv_u32(a + ".attention.head_count", n_q),
        _kv_u32(a + ".attention.head_count_kv", n_kv),
        _kv_u32(a + ".attention.key_length", head_dim),
        _kv_u32(a + ".attention.value_length", head_dim),
        _kv_u32(a + ".attention.key_length_swa", head_dim_swa),
        _kv_u32(a + ".attention.value_length_swa", head_dim_swa),
        _kv_f32(a + ".attention.layer_norm_rms_epsilon", eps),
        _kv_f32(a + ".rope.freq_base", theta),
        _kv_f32(a + ".rope.freq_base_swa", theta_swa),
        _kv_u32(a + ".context_length", ctx),
        _kv_u32(a + ".attention.sliding_window", sliding_window),
        _kv_u32(a + ".attention.shared_kv_layers", shared_kv_layers),
        _kv_u32(a + ".embedding_length_per_layer_input", pl_emb),
        _kv_f32(a + ".final_logit_softcapping", softcap),
        _kv_bool_array(a + ".attention.sliding_window_pattern", swa_pattern),
    ]
    plw = n_layers * pl_emb
    tensors = [("token_embd.weight", (hidden, vocab), T_F16), ("output_norm.weight", (hidden,), T_F32)]
    if pl_emb:
        tensors += [("per_layer_token_embd.weight", (plw, vocab), T_F16),
                    ("per_layer_model_proj.weight", (hidden, plw), T_F16),
                    ("per_layer_proj_norm.weight", (pl_emb,), T_F32)]
    for L in range(n_layers):
        hd = head_dim_swa if (swa_pattern[L] and head_dim_swa) else head_dim
        f = ffn if isinstance(ffn, int) else ffn[L]
        p = f"blk.{L}."
        tensors += [
            (p + "attn_norm.weight", (hidden,), T_F32),
            (p + "attn_q.weight", (hidden, n_q * hd), T_F16),
            (p + "attn_k.weight", (hidden, n_kv * hd), T_F16),
            (p + "attn_v.weight", (hidden, n_kv * hd), T_F16),
            (p + "attn_q_norm.weight", (hd,), T_F32),
            (p + "attn_k_norm.weight", (hd,), T_F32),
            (p + "attn_output.weight", (n_q * hd, hidden), T_F16),
            (p + "post_attention_norm.weight", (hidden,), T_F32),
            (p + "ffn_norm.weight", (hidden,), T_F32),
            (p + "ffn_gate.weight", (hidden, f), T_F16),
            (p + "ffn_up.weight", (hidden, f), T_F16),
            (p + "ffn_down.weight", (f, hidden), T_F16),
            (p + "post_ffw_norm.weight", (hidden,), T_F32),
        ]
        if pl_emb:
            tensors += [
                (p + "post_norm.weight", (hidden,), T_F32),
                (p + "inp_gate.weight", (hidden, pl_emb), T_F16),
                (p + "proj.weight", (pl_emb, hidden), T_F16),
                (p + "layer_output_scale.weight", (1,), T_F32),
            ]

    def fill(name, n, typ):
        if any(name.endswith(z) for z in zero):          # (test knob: switch a tensor off)
            return bytes(n * (4 if typ == T_F32 else 2))
        if typ == T_F32:
            if name.endswith("layer_output_scale.weight") and output_scale is not None:
                return np.full(n, output_scale, np.float32).tobytes()
            if name.endswith("layer_output_scale.weight"):
                return (np.float32(0.9) + 0.05 * rng.random(n, dtype=np.float32)).astype(np.float32).tobytes()
            w = np.float32(1.0) + np.float32(0.1) * rng.standard_normal(n, dtype=np.float32)
            if name.endswith("attn_q_norm.weight") or name.endswith("attn_k_norm.weight"):
                w = w * np.float32(0.3)      # scores of RMS-normed Q.K at scale 1 stay in a trained model's range
            return w.astype(np.float32).tobytes()
        return (rng.standard_normal(n, dtype=np.float32) * np.float32(std)).astype(np.float16).tobytes()

    return _write(path, kvs, tensors, fill)
