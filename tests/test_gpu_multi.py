"""GPU, 2 ranks over NCCL: long-context decode with the key sequence sharded
across devices (partial attention per rank -> one all-gather of the triples ->
local merge) against the unsharded reference attention, and the same step with
the all-gather and the merge fused into one kernel over NVLink peer memory
(wr_cuda_attn_exchange_combine), which must give identical bits.  Skipped on a box with
fewer than two GPUs; the same plumbing runs on CPU ranks in
tests/test_splitkv_gloo.py."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
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
    import wayruntime_b200 as wr
    from wayruntime_b200 import splitkv
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    P = oracle.restatement()
    ctx = wr.Context(rank, attn_max_seq=32768)
    stream = torch.cuda.ExternalStream(ctx.stream, device=rank)
    torch.cuda.set_stream(stream)
    hq, hkv, hd = 32, 8, 128
    lens = [5000, 1, 777, 4096]
    ks = [P.f32_to_f16(_gen.normal(70 + s, (n, hkv, hd))) for s, n in enumerate(lens)]
    vs = [P.f32_to_f16(_gen.normal(80 + s, (n, hkv, hd))) for s, n in enumerate(lens)]
    q = _gen.normal(90, (len(lens), hq, hd))
    kvs, local = [], []
    for k, v, n in zip(ks, vs, lens):
        lo, hi = splitkv.shard_range(n, rank, world)
        kv = ctx.kv_create(1, hkv, hd, max(hi - lo, 1))
        if hi > lo:
            kv.write_rows(0, 0, 0, np.ascontiguousarray(k[lo:hi]))
            kv.write_rows(0, 1, 0, np.ascontiguousarray(v[lo:hi]))
        kvs.append(kv), local.append(hi - lo)
    qd = torch.from_numpy(q).cuda()
    out = torch.empty_like(qd)
    for _ in range(2):                      # twice: scratch and tickets are reused
        splitkv.decode_split_kv(ctx, kvs, 0, local, qd, out, hq)
    ctx.sync()
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    # the same step with the all-gather and the merge fused into one kernel over
    # peer memory: same merge order, so the result has to be identical
    xchg = splitkv.make_exchange(ctx, len(lens) * hq, hd)
    out2 = torch.full_like(qd, float("nan"))
    for _ in range(3):                      # three times: both buffer parities are used again
        splitkv.decode_split_kv(ctx, kvs, 0, local, qd, out2, hq, exchange=xchg)
    ctx.sync()
    torch.cuda.synchronize()
    same = bool(np.array_equal(out2.cpu().numpy().view(np.uint32), got.view(np.uint32)))
    # and with the decode kernel itself delivering the triples to the peers
    out3 = torch.full_like(qd, float("nan"))
    for _ in range(3):
        splitkv.decode_split_kv(ctx, kvs, 0, local, qd, out3, hq, exchange=xchg, fused_decode=True)
    ctx.sync()
    torch.cuda.synchronize()
    same = same and bool(np.array_equal(out3.cpu().numpy().view(np.uint32), got.view(np.uint32)))
    splitkv.close_exchange(xchg, ctx)
    rc, want = P.decode_batch(q, ks, vs, threads=4, max_seq=32768)
    result_q.put((rank, rc, float(np.abs(got - want).max()), same))
    for kv in kvs:
        kv.close()
    ctx.close()
    dist.destroy_process_group()


def test_key_sharded_decode_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mpc = mp.get_context("spawn")
    result_q = mpc.Queue()
    port_no = 29700 + (os.getpid() % 2000)
    procs = [mpc.Process(target=_worker, args=(r, 2, port_no, result_q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [result_q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _rank, rc, err, fused_same in results:
        assert rc == 0
        assert err <= 2e-3
        assert fused_same, "fused exchange+merge differs from all-gather + merge"
