"""Seeded GGUF writer for the whole-model parity tests (BASELINE config 1).

Writes a GGUF v3 file with the metadata and tensors the reference loader
demands for a qwen3-class model (src/core/gguf.c:892-1008,
src/core/loader.c:283-429, :522-668): F16 matmul weights ~N(0, std), F32 norm
vectors = 1.0, tied LM head (no output.weight), no tokenizer arrays.
"""
import struct

import numpy as np

GGUF_U32, GGUF_F32, GGUF_STR = 4, 6, 8
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
