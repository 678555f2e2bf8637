"""world_size-2 gloo runs of the sharded layers' host logic: partitioning, the output all-gather
re-layout, and the sharded per-token encode (per-shard abs-max, MAX all-reduce, encode of the
shard with the global scales, gather of the codes), with CPU stand-ins for the kernels."""

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


def _encode_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lucid_b200.nn.quantized.sharded import gather_columns, shard_bounds
        from oracle import lucid_oracle as O

        rng = np.random.default_rng(1)
        h = (rng.standard_normal((40, 96)) * rng.random((40, 1)) * 4).astype(np.float32)
        h[3] = 0  # an all-zero token
        want_codes, want_scales = O.per_token_quantize(h)
        c0, c1 = shard_bounds(96, world, rank)
        shard = h[:, c0:c1]
        # this rank's per-token abs-max (what lq_minmax per row + max(|min|, |max|) computes) ...
        am = torch.from_numpy(np.maximum(np.abs(shard.min(axis=1)), np.abs(shard.max(axis=1))))
        dist.all_reduce(am, op=dist.ReduceOp.MAX)  # ... and the exchange step of the scales
        # scale = max(absmax / ((qmax - qmin) / 2), eps): the per-token encode's expressions
        scales = np.maximum(am.numpy() / np.float32(127.5), np.float32(1e-8)).astype(np.float32)
        codes = O.quantize(shard, scales, np.zeros_like(scales), O.QINT8, ch_axis=0)
        full = gather_columns(torch.from_numpy(codes))  # stand-in for the stores into every rank's buffer
        ok = np.array_equal(scales, want_scales) and np.array_equal(full.numpy(), want_codes)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_sharded_per_token_encode_world2():
    """Encoding column shards with the all-reduced per-token abs-max reproduces the unsharded
    per-token encode bit for bit (max is order-free)."""
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_encode_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world))
