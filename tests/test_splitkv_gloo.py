"""CPU, world_size 2 over gloo: the host side of key-sharded decode — shard
ranges, the all-gather layout of the (m, l, o) triples and the merge — checked
against the unsharded reference attention.  Each rank computes its shard's
triples with the CPU oracle (no GPU here); the gather and merge are the code
the GPU path uses."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port_no, result_q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_no)
    import torch
    import torch.distributed as dist
    import _gen
    import oracle
    from wayruntime_b200 import splitkv
    dist.init_process_group("gloo", rank=rank, world_size=world)
    P = oracle.restatement()
    hq, hkv, hd = 8, 2, 128
    lens = [300, 1, 77]                      # the 1-key session leaves rank 1 with an empty shard
    rows = []
    for s, n in enumerate(lens):
        q = _gen.normal(40 + s, (1, hq, hd))
        k = P.f32_to_f16(_gen.normal(50 + s, (n, hkv, hd)))
        v = P.f32_to_f16(_gen.normal(60 + s, (n, hkv, hd)))
        lo, hi = splitkv.shard_range(n, rank, world)
        tri = np.zeros((hq, splitkv.TRIPLE_PAD + hd), np.float32)
        tri[:, 0] = -1e30
        if hi > lo:
            rc, m, l, o = P.partial(q[0], k, v, lo, hi)
            assert rc == 0
            tri[:, 0], tri[:, 1], tri[:, splitkv.TRIPLE_PAD:] = m, l, o
        rows.append(tri)
    local = torch.from_numpy(np.concatenate(rows))
    gathered = splitkv.gather_triples(local)
    assert tuple(gathered.shape) == (world, len(lens) * hq, splitkv.TRIPLE_PAD + hd)
    merged = splitkv.merge_triples_reference(gathered.numpy())
    worst = 0.0
    for s, n in enumerate(lens):
        q = _gen.normal(40 + s, (1, hq, hd))
        k = P.f32_to_f16(_gen.normal(50 + s, (n, hkv, hd)))
        v = P.f32_to_f16(_gen.normal(60 + s, (n, hkv, hd)))
        rc, full = P.attention(q, k, v)
        worst = max(worst, float(np.abs(merged[s * hq:(s + 1) * hq] - full[0]).max()))
    result_q.put((rank, worst))
    dist.destroy_process_group()


def test_shard_ranges_cover_every_key_once():
    from wayruntime_b200 import splitkv
    for n in (0, 1, 5, 64, 65, 1000, 32768):
        for world in (1, 2, 4, 8):
            spans = [splitkv.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a, b), (c, d) in zip(spans[:-1], spans[1:]):
                assert b == c and a <= b and c <= d


def test_two_rank_gather_and_merge_matches_unsharded():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    result_q = ctx.Queue()
    port_no = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port_no, result_q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [result_q.get(timeout=60) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _rank, worst in results:
        assert worst < 2e-5
