"""`wayrt bench` for a wayruntime shared library, through its public C API.

Restates the reference CLI's bench command (src/cli/wayrt.c:694-854) so that the
drop-in library (lib/libwayruntime_b200.so) and an unmodified reference build
can be timed by the same code on the same model and printed in the reference's
own format: a `prefill:` line, a `decode:` line (tokens, ms, tok/s) and the
engine counters (wayrt.c:388-404).  As there: every prompt token but the last
is prefilled (no LM head), then N tokens are decoded greedily from the last
prompt token, straight through any end-of-sequence token; the clock is
CLOCK_MONOTONIC around each phase.

One difference, stated in the output: the reference tokenises the fixed prompt
"Once upon a time"; a generated GGUF has no tokenizer, so the prompt here is a
seeded list of token ids of a given length.

    python -m wayruntime_b200.wayrt_bench --lib PATH model.gguf --tokens 32 --prompt-tokens 64
"""
from __future__ import annotations

import argparse
import ctypes as C
import time

import numpy as np

COUNTER_NAMES = [
    "matmul_calls", "matmul_elems", "softmax_calls", "attention_calls", "fused_calls",
    "matmul_variant", "softmax_variant", "matmul_ggml_simd", "matmul_ggml_variant",
    "matmul_ggml_quant", "matmul_perelem", "matmul_par_n",
]
WR_ERR_CTX_FULL = -6


class ModelInfo(C.Structure):
    # wr_model_info, include/wayruntime/wayruntime.h: read as raw words (arch / quant strings first)
    _fields_ = [("raw", C.c_uint8 * 256)]


class Library:
    """One loaded wayruntime library with one engine (v1 is single-engine per process)."""

    def __init__(self, path: str, n_threads: int = 0):
        self.path = path
        L = self.L = C.CDLL(path)
        L.wr_engine_create.restype = C.c_int
        L.wr_engine_destroy.restype = None
        L.wr_model_load.restype = C.c_int
        L.wr_model_free.restype = None
        L.wr_session_create.restype = C.c_int
        L.wr_session_destroy.restype = None
        L.wr_prefill.restype = C.c_int
        L.wr_step.restype = C.POINTER(C.c_float)
        L.wr_session_status.restype = C.c_int
        L.wr_engine_counters.restype = C.c_int
        L.wr_engine_thread_count.restype = C.c_int
        L.wr_engine_simd_variant.restype = C.c_int
        self.engine = C.c_void_p()
        cfg = (C.c_uint8 * 512)()                      # zeroed wr_engine_config; n_threads is its first field
        C.cast(cfg, C.POINTER(C.c_uint32))[0] = n_threads
        rc = L.wr_engine_create(cfg, C.byref(self.engine))
        if rc != 0:
            raise RuntimeError(f"wr_engine_create({path}) returned {rc}")

    def close(self):
        if self.engine:
            self.L.wr_engine_destroy(self.engine)
            self.engine = C.c_void_p()

    def counters(self) -> list[int]:
        c = (C.c_uint64 * 16)()
        self.L.wr_engine_counters(self.engine, c)
        return [int(c[i]) for i in range(len(COUNTER_NAMES))]


def bench(lib: Library, model_path: str, prompt_ids, n_tokens: int, vocab: int) -> dict:
    """Prefill len(prompt_ids) - 1 tokens, decode n_tokens greedily; returns the figures."""
    L = lib.L
    model = C.c_void_p()
    params = (C.c_uint8 * 512)()
    rc = L.wr_model_load(lib.engine, model_path.encode(), params, C.byref(model))
    if rc != 0:
        raise RuntimeError(f"wr_model_load returned {rc}")
    session = C.c_void_p()
    rc = L.wr_session_create(model, None, C.byref(session))
    if rc != 0:
        L.wr_model_free(model)
        raise RuntimeError(f"wr_session_create returned {rc}")
    try:
        c0 = lib.counters()
        n_prefill = len(prompt_ids) - 1
        prefill_s = 0.0
        if n_prefill > 0:
            arr = (C.c_uint32 * n_prefill)(*prompt_ids[:n_prefill])
            t0 = time.clock_gettime(time.CLOCK_MONOTONIC)
            pf = L.wr_prefill(session, arr, n_prefill)
            prefill_s = time.clock_gettime(time.CLOCK_MONOTONIC) - t0
            if pf < 0:
                raise RuntimeError(f"wr_prefill returned {pf}")
        prev, produced, ctx_hit, ids = int(prompt_ids[-1]), 0, False, []
        t0 = time.clock_gettime(time.CLOCK_MONOTONIC)
        for _ in range(n_tokens):
            logits = L.wr_step(session, C.c_uint32(prev))
            if not logits:
                st = L.wr_session_status(session)
                if st == WR_ERR_CTX_FULL:
                    ctx_hit = True
                    break
                raise RuntimeError(f"wr_step failed: wr_status {st}")
            prev = int(np.argmax(np.ctypeslib.as_array(logits, (vocab,))))     # first maximum: lowest id wins ties
            ids.append(prev)
            produced += 1
        decode_s = time.clock_gettime(time.CLOCK_MONOTONIC) - t0
        c1 = lib.counters()
    finally:
        L.wr_session_destroy(session)
        L.wr_model_free(model)
    return {
        "n_prefill": n_prefill, "prefill_s": prefill_s, "produced": produced, "decode_s": decode_s,
        "ctx_hit": ctx_hit, "ids": ids, "threads": int(L.wr_engine_thread_count(lib.engine)),
        "simd_variant": int(L.wr_engine_simd_variant(lib.engine)),
        "counters": [b - a if i not in (5, 6, 8) else b for i, (a, b) in enumerate(zip(c0, c1))],
    }


def bench_batch(lib: Library, model_path: str, prompts, n_steps: int, vocab: int) -> dict:
    """len(prompts) sessions of one model: each prefills its own prompt (all tokens but the last),
    then the batch decodes n_steps tokens per session greedily through wr_batch_step
    (include/wayruntime/wayruntime.h:423-444), one call per step for all sessions."""
    L = lib.L
    L.wr_batch_step.restype = C.c_int
    model = C.c_void_p()
    params = (C.c_uint8 * 512)()
    rc = L.wr_model_load(lib.engine, model_path.encode(), params, C.byref(model))
    if rc != 0:
        raise RuntimeError(f"wr_model_load returned {rc}")
    n = len(prompts)
    sessions = []
    try:
        for _ in range(n):
            s = C.c_void_p()
            rc = L.wr_session_create(model, None, C.byref(s))
            if rc != 0:
                raise RuntimeError(f"wr_session_create returned {rc}")
            sessions.append(s)
        t0 = time.clock_gettime(time.CLOCK_MONOTONIC)
        n_prefill = 0
        for s, ids in zip(sessions, prompts):
            if len(ids) > 1:
                arr = (C.c_uint32 * (len(ids) - 1))(*ids[:-1])
                pf = L.wr_prefill(s, arr, len(ids) - 1)
                if pf < 0:
                    raise RuntimeError(f"wr_prefill returned {pf}")
                n_prefill += len(ids) - 1
        prefill_s = time.clock_gettime(time.CLOCK_MONOTONIC) - t0
        handles = (C.c_void_p * n)(*[s.value for s in sessions])
        toks = (C.c_uint32 * n)(*[int(ids[-1]) for ids in prompts])
        outp = (C.POINTER(C.c_float) * n)()
        ids_out = [[] for _ in range(n)]
        t0 = time.clock_gettime(time.CLOCK_MONOTONIC)
        for _ in range(n_steps):
            rc = L.wr_batch_step(handles, toks, n, outp)
            if rc != n:
                raise RuntimeError(f"wr_batch_step returned {rc}")
            for i in range(n):
                nxt = int(np.argmax(np.ctypeslib.as_array(outp[i], (vocab,))))
                toks[i] = nxt
                ids_out[i].append(nxt)
        decode_s = time.clock_gettime(time.CLOCK_MONOTONIC) - t0
    finally:
        for s in sessions:
            L.wr_session_destroy(s)
        L.wr_model_free(model)
    return {"sessions": n, "n_prefill": n_prefill, "prefill_s": prefill_s, "steps": n_steps, "decode_s": decode_s,
            "ids": ids_out}


def rate(n: int, s: float) -> float:
    return n / s if s > 0 else 0.0


def report(res: dict, model_path: str, lib_path: str) -> str:
    """The reference's bench output (wayrt.c:819-841), plus the library's path."""
    lines = [f"library:  {lib_path}", f"model:    {model_path}",
             f"simd:     variant {res['simd_variant']}  threads: {res['threads']}"]
    if res["n_prefill"] > 0:
        lines.append(f"prefill:  {res['n_prefill']} tokens  {res['prefill_s'] * 1e3:.2f} ms  "
                     f"{rate(res['n_prefill'], res['prefill_s']):.1f} tok/s")
    else:
        lines.append("prefill:  0 tokens (single-token prompt)")
    lines.append(f"decode:   {res['produced']} tokens  {res['decode_s'] * 1e3:.2f} ms  "
                 f"{rate(res['produced'], res['decode_s']):.1f} tok/s"
                 + ("  (stopped: context full)" if res["ctx_hit"] else ""))
    lines.append("counters:")
    for name, v in zip(COUNTER_NAMES, res["counters"]):
        lines.append(f"  {name:<22s} {v}")
    return "\n".join(lines)


def seeded_prompt(n: int, vocab: int, seed: int = 20261125) -> list[int]:
    rng = np.random.Generator(np.random.Philox(seed))
    return [int(x) for x in rng.integers(0, vocab, size=n)]


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("model")
    ap.add_argument("--lib", required=True, help="libwayruntime_b200.so or a reference build")
    ap.add_argument("--tokens", type=int, default=32)
    ap.add_argument("--prompt-tokens", type=int, default=64)
    ap.add_argument("--vocab", type=int, required=True, help="vocabulary size of the model")
    args = ap.parse_args()
    lib = Library(args.lib)
    try:
        res = bench(lib, args.model, seeded_prompt(args.prompt_tokens, args.vocab), args.tokens, args.vocab)
        print(report(res, args.model, args.lib))
        print(f"prompt:   {args.prompt_tokens} seeded token ids (the model file carries no tokenizer)")
    finally:
        lib.close()


if __name__ == "__main__":
    main()
