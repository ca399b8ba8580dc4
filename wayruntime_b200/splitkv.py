"""Long-context decode with the KV sequence sharded across devices.

Each rank holds a contiguous range of every session's keys in its own paged
cache, runs the split-KV decode kernel over that range
(``wr_cuda_attn_decode_partial``) and emits one (m, l, o) triple per (session,
q head).  One all-gather of those triples (130-odd floats per row and rank)
and a local merge (``wr_cuda_attn_combine``) give every rank the full result.
The merge is the reference's online-softmax update (src/core/kernels.c:1503-1506)
applied across shards instead of across 64-key tiles.

``torch.distributed`` is the transport: NCCL over NVLink for CUDA tensors, gloo
for the CPU tests of the plumbing.
"""
from __future__ import annotations

import numpy as np

TRIPLE_PAD = 4
NEG_SENTINEL = np.float32(-1e30)


def shard_range(n_keys: int, rank: int, world: int) -> tuple[int, int]:
    """Keys [lo, hi) of an n_keys-long sequence that rank `rank` of `world` holds:
    contiguous ranges of ceil(n_keys / world), the last ones possibly empty."""
    per = (n_keys + world - 1) // world
    lo = min(rank * per, n_keys)
    return lo, min(lo + per, n_keys)


def gather_triples(local, group=None):
    """All-gather [rows, TRIPLE_PAD + hd] triples -> [world, rows, TRIPLE_PAD + hd]."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    # (the concatenated 2-D form of the output is the one every backend accepts)
    dist.all_gather_into_tensor(out.view(world * local.shape[0], *local.shape[1:]),
                                local.contiguous(), group=group)
    return out


def merge_triples_reference(triples: np.ndarray) -> np.ndarray:
    """numpy statement of the merge: triples [G, rows, TRIPLE_PAD + hd] -> [rows, hd]."""
    m = triples[:, :, 0]
    l = triples[:, :, 1]
    o = triples[:, :, TRIPLE_PAD:]
    mstar = m.max(axis=0)
    w = np.where(m == NEG_SENTINEL, np.float32(0), np.exp(m - mstar[None, :])).astype(np.float32)
    num = (w[:, :, None] * o).sum(axis=0)
    den = (w * l).sum(axis=0)
    safe = np.where(den > 0, den, np.float32(1))
    return np.where(den[:, None] > 0, num / safe[:, None], np.float32(0)).astype(np.float32)


def make_exchange(ctx, max_rows, head_dim, group=None):
    """An `Exchange` connected to every rank of `group` (handles travel through
    torch.distributed's object all-gather; the data path afterwards is the
    kernel's own NVLink stores)."""
    import torch.distributed as dist
    import wayruntime_b200 as wr
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    x = wr.Exchange(ctx, world, rank, max_rows, head_dim)
    handles = [None] * world
    dist.all_gather_object(handles, x.handle, group=group)
    try:
        x.connect(handles)
        err = None
    except wr.WrCudaError as exc:
        err = str(exc)
    # every rank learns whether every rank connected: nobody is left waiting in a kernel
    errs = [None] * world
    dist.all_gather_object(errs, err, group=group)         # (also a barrier: nobody closes early)
    if any(e is not None for e in errs):
        x.close()
        raise RuntimeError(f"peer exchange unavailable: {[e for e in errs if e][0]}")
    return x


def close_exchange(x, ctx, group=None):
    """Collective destroy of an `Exchange`: a peer's kernel may still be storing
    into this rank's buffer, so every rank drains its own stream (a step that
    timed out is reported here and does not stop the close), the ranks meet,
    and only then is the buffer freed."""
    import torch.distributed as dist
    try:
        ctx.sync()
    except Exception:
        pass
    dist.barrier(group=group)
    x.close()


def decode_split_kv(ctx, kvs, layer, local_lens, q, out, n_q_heads, scale=0.0, group=None,
                    triples=None, gathered=None, exchange=None, fused_decode=False):
    """One decode step over key-sharded caches.  q, out: CUDA float32 tensors
    [n_sess, n_q_heads, hd]; local_lens: keys of each session held by this rank.
    Everything is enqueued on the context's stream (set it current for NCCL).
    With `exchange` (see make_exchange) the all-gather and the merge are one
    kernel over peer memory instead of an NCCL collective and a merge kernel;
    with `fused_decode` as well, the decode kernel itself stores its triples
    into the peers' buffers (wr_cuda_attn_decode_exchange, head_dim 128)."""
    import torch
    import torch.distributed as dist
    n_sess, _, hd = q.shape
    rows = n_sess * n_q_heads
    if exchange is not None and fused_decode:
        exchange.decode(kvs, layer, local_lens, q, out, n_q_heads, scale=scale)
        return out
    if triples is None:
        triples = torch.empty((rows, TRIPLE_PAD + hd), dtype=torch.float32, device=q.device)
    ctx.attn_decode_partial(kvs, layer, local_lens, q, triples, n_q_heads, scale=scale)
    if exchange is not None:
        exchange.combine(rows, triples, out)
        return out
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        gathered = triples
    else:
        if gathered is None:
            gathered = torch.empty((world, rows, TRIPLE_PAD + hd), dtype=torch.float32, device=q.device)
        dist.all_gather_into_tensor(gathered.view(world * rows, TRIPLE_PAD + hd), triples, group=group)
    ctx.attn_combine(world, rows, hd, gathered, out)
    return out
