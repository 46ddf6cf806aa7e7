"""Two ranks, one GPU each, NCCL: (batch x head)-sharded prefill gives bit-identical
heads to the single-GPU run, and KV-sequence-sharded decode (fa_decode_kv_sharded: the
local slice -> one in-place all-gather -> packed merge) matches the unsharded oracle.
Skipped on machines with fewer than two GPUs."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge
    from oracle import oracle
    from helpers import run_prefill
    fa = ge.load_package()
    sh = ge.load_module("sharding")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        fa.clear_device_status()
        # (1) head-sharded causal prefill
        bh, s, d = 6, 384, 64
        q, k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(51, (bh, s, d)))
        h0, hc = sh.head_shard(bh, rank, world)
        o_loc, l_loc = run_prefill(fa, dev, q[h0:h0 + hc], k[h0:h0 + hc], v[h0:h0 + hc], 0.125, True)
        o_ref, l_ref = oracle.attention(q[h0:h0 + hc], k[h0:h0 + hc], v[h0:h0 + hc], 0.125, True)
        e1 = float(max(np.abs(o_loc - o_ref).max() / 2e-3, np.abs(l_loc - l_ref).max() / 1e-3))
        # (2) KV-sequence-sharded decode
        bh, skv, d = 8, 6000, 128
        scale = float(1.0 / np.sqrt(np.float32(d)))
        kk, vv = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(52, (bh, skv, d), n=2))
        qq = oracle.round_to(oracle.normal_inputs(53, (bh, 1, d), n=1)[0], "f16")
        k0, kc = sh.kv_shard(skv, rank, world)
        dq = torch.from_numpy(qq.reshape(bh, d)).to(dev, torch.float16)
        dk = torch.from_numpy(kk[:, k0:k0 + kc]).to(dev, torch.float16).contiguous()
        dv = torch.from_numpy(vv[:, k0:k0 + kc]).to(dev, torch.float16).contiguous()
        do = torch.zeros((bh, d), device=dev, dtype=torch.float16)
        dl = torch.zeros((bh,), device=dev, dtype=torch.float32)
        with sh.ShardedDecode(fa, 1, bh, d, kc, dtype="f16", num_splits=3) as run:
            run(dq, dk, dv, do, dl, scale)
            run(dq, dk, dv, do, dl, scale)                 # buffers are reused across calls
            torch.cuda.synchronize()
        o2_ref, l2_ref = oracle.attention(qq, kk, vv, scale, False)
        e2 = float(max(np.abs(do.float().cpu().numpy() - o2_ref[:, 0]).max() / 2e-3,
                       np.abs(dl.cpu().numpy() - l2_ref[:, 0]).max() / 1e-3))
        q_out.put((rank, e1, e2, fa.device_status()))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding(fa):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = 29600 + (os.getpid() % 1000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, e1, e2, status in results:
        assert e1 < 1.0 and e2 < 1.0 and status == 0, (rank, e1, e2, status)
