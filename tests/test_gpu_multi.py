"""Two-GPU check of the output-channel sharded Linear: the fused exchange (GEMM epilogue
storing into every rank's buffer over NVLink) and the NCCL all-gather both reproduce the
single-GPU result bit for bit.  Runs as two child processes, one per GPU; skipped on boxes
with fewer than two GPUs."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_DEBUG="WARN")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime

    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        import lucid_b200.quantization as Q
        from lucid_b200 import _lib
        from lucid_b200.nn.quantized import functional as QF
        from lucid_b200.nn.quantized.dynamic import interleave_gate_up
        from lucid_b200.nn.quantized.sharded import ColumnShardedLinear

        g = torch.Generator(device=dev).manual_seed(7)  # same data on every rank
        m, k, n = 520, 512, 1536
        x = torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16)
        wq = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev, generator=g)
        ws = torch.rand(n, device=dev, generator=g) * 1e-2 + 1e-3
        bias = torch.randn(n, device=dev, generator=g)
        a, s = Q.quantize_per_token(x, Q.qint8)
        full = QF.gemm_s8(a, wq, out_dtype=torch.bfloat16, a_scale=s, b_scale=ws, bias=bias)
        lin = ColumnShardedLinear.from_full(wq, ws, bias, world, rank)
        ok = torch.equal(lin.forward_codes(a, s), full)          # NCCL all-gather
        lin.use_peer_outputs(max_rows=m)
        for _ in range(3):                                        # alternating buffers
            ok = ok and torch.equal(lin.forward_codes(a, s), full)
        ok = ok and torch.equal(lin(x), full)
        # gated: [gate; up] interleaved per rank, output columns = ff / world per rank
        ff = 1024
        gq = torch.randint(-127, 128, (ff, k), dtype=torch.int8, device=dev, generator=g)
        uq = torch.randint(-127, 128, (ff, k), dtype=torch.int8, device=dev, generator=g)
        gs = torch.rand(ff, device=dev, generator=g) * 1e-2 + 1e-3
        us = torch.rand(ff, device=dev, generator=g) * 1e-2 + 1e-3
        h_full = QF.gemm_s8(a, interleave_gate_up(gq, uq), out_dtype=torch.bfloat16, a_scale=s,
                            b_scale=interleave_gate_up(gs, us), act=_lib.ACT_SILU_GATE)
        per = ff // world
        sl = slice(rank * per, (rank + 1) * per)
        gl = ColumnShardedLinear(k, 2 * ff, world, rank)
        gl.weight_int8 = interleave_gate_up(gq[sl].contiguous(), uq[sl].contiguous())
        gl.weight_scale = interleave_gate_up(gs[sl].contiguous(), us[sl].contiguous())
        gl = gl.to(dev)
        gl.use_peer_outputs(max_rows=m, gated=True)
        for _ in range(2):
            ok = ok and torch.equal(gl.forward_codes(a, s, act=_lib.ACT_SILU_GATE), h_full)
        # the gated output feeding a per-token encode: shard kept local, abs-max all-reduced,
        # codes stored into every rank's operand buffer == the unsharded per-token encode
        from lucid_b200.nn.quantized.sharded import PeerOutputs, quantize_shard_bcast, shard_absmax

        want_codes, want_scales = Q.quantize_per_token(h_full, Q.qint8)
        h_local = QF.gemm_s8(a, gl.weight_int8, out_dtype=torch.bfloat16, a_scale=s, b_scale=gl.weight_scale,
                             act=_lib.ACT_SILU_GATE)
        ok = ok and torch.equal(h_local, h_full[:, sl])
        codes = PeerOutputs(m, ff, torch.int8, dev)
        for it in range(4):
            # unicast peer stores, then (where the buffers have one) the NVSwitch multicast address
            mc = it >= 2 and codes.has_multicast
            buf, ptrs = codes.next(multicast=mc)
            buf.fill_(77)
            codes.fence()
            scales = quantize_shard_bcast(h_local, shard_absmax(h_local), ptrs, ff, rank * per)
            codes.fence()
            ok = ok and torch.equal(buf, want_codes) and torch.equal(scales, want_scales)
        # the GEMM epilogue through the multicast address
        outs = PeerOutputs(m, n, torch.bfloat16, dev)
        if outs.has_multicast:
            npr = n // world
            for _ in range(2):
                buf, mc_ptr = outs.next(multicast=True)
                buf.fill_(0)
                outs.fence()
                QF.gemm_s8_bcast(a, wq[rank * npr:(rank + 1) * npr].contiguous(), mc_ptr, (m, n), rank * npr,
                                 a_scale=s, b_scale=ws[rank * npr:(rank + 1) * npr].contiguous(),
                                 bias=bias[rank * npr:(rank + 1) * npr].contiguous())
                outs.fence()
                ok = ok and torch.equal(buf, full)
        ret["multicast"] = bool(codes.has_multicast)
        torch.cuda.synchronize()
        _lib.check_device_status(dev)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_linear_two_gpus():
    import torch.multiprocessing as mp

    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)
