"""CPU-only, world_size 2 over gloo: the host side of the multi-GPU paths - the
shard planners and the all-gather layout feeding the LSE merge - checked against
the unsharded oracle.  (The GPU kernels themselves are covered by the gpu tests;
here the per-rank partials come from the CPU oracle.)"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_planners():
    import __graft_entry__ as ge
    sh = ge.load_module("sharding")
    for total, world in ((96, 8), (96, 5), (7, 8), (131072, 8), (1000, 3)):
        covered = []
        for r in range(world):
            start, count = sh.head_shard(total, r, world)
            covered.extend(range(start, start + count))
            assert sh.kv_shard(total, r, world) == (start, count)
        assert covered == list(range(total))
        sizes = [sh.head_shard(total, r, world)[1] for r in range(world)]
        assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge
    from oracle import oracle
    sh = ge.load_module("sharding")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bh, skv, d = 6, 1001, 64
        k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(31, (bh, skv, d), n=2))
        q = oracle.round_to(oracle.normal_inputs(32, (bh, 1, d), n=1)[0], "f16")
        # (1) KV-sequence sharding: local partial -> all-gather -> merge
        start, count = sh.kv_shard(skv, rank, world)
        o_loc, l_loc = oracle.attention(q, k[:, start:start + count], v[:, start:start + count], 0.125, False)
        o_parts, l_parts = sh.gather_partials(torch.from_numpy(o_loc[:, 0]), torch.from_numpy(l_loc[:, 0]))
        assert o_parts.shape == (world, bh, d) and l_parts.shape == (world, bh)
        assert np.array_equal(o_parts[rank].numpy(), o_loc[:, 0])
        o_m, l_m = oracle.merge(np.transpose(o_parts.numpy(), (1, 0, 2)), np.transpose(l_parts.numpy(), (1, 0)))
        o_ref, l_ref = oracle.attention(q, k, v, 0.125, False)
        err_o = float(np.abs(o_m - o_ref[:, 0]).max())
        err_l = float(np.abs(l_m - l_ref[:, 0]).max())
        # (2) head sharding: each rank's heads equal the same heads of the unsharded run
        h0, hc = sh.head_shard(bh, rank, world)
        o_h, l_h = oracle.attention(q[h0:h0 + hc], k[h0:h0 + hc], v[h0:h0 + hc], 0.125, False)
        same = bool(np.array_equal(o_h, o_ref[h0:h0 + hc]) and np.array_equal(l_h, l_ref[h0:h0 + hc]))
        q_out.put((rank, err_o, err_l, same))
    finally:
        dist.destroy_process_group()


def test_kv_sharded_merge_and_head_sharding_gloo_world2():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = 29500 + (os.getpid() % 1000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err_o, err_l, same in results:
        assert err_o < 1e-5 and err_l < 1e-5 and same, (rank, err_o, err_l, same)
