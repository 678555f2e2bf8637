"""world_size-2 gloo run of the sharded Linear's host logic: partitioning and
the output all-gather re-layout, with a CPU stand-in for the local contraction."""

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lucid_b200.nn.quantized.sharded import gather_columns, shard_bounds

        rng = np.random.default_rng(0)
        a = torch.from_numpy(rng.integers(-128, 128, (24, 64)).astype(np.int64))
        w = torch.from_numpy(rng.integers(-128, 128, (48, 64)).astype(np.int64))
        n0, n1 = shard_bounds(48, world, rank)
        local = (a @ w[n0:n1].T).to(torch.int32)  # stand-in for this rank's integer GEMM
        full = gather_columns(local)
        ok = torch.equal(full, (a @ w.T).to(torch.int32))
        # float shards gather the same way
        fl = gather_columns(local.float() * 0.5)
        ok = ok and torch.equal(fl, (a @ w.T).float() * 0.5)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_gather_columns_world2():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world))
