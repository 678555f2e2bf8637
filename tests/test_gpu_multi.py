"""Two-GPU check of the output-channel sharded Linear against the CPU oracle: the fused
exchange (GEMM epilogue storing into every rank's buffer over NVLink, ordered by device flags
instead of a collective), the NCCL all-gather baseline, the gated variant, the exchange of a
hidden tensor as per-token codes and the token-sharded input encode all reproduce the oracle's
single-GPU result bit for bit on every rank.  Runs as two child processes, one per GPU; skipped
on boxes with fewer than two GPUs."""

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
    import numpy as np
    import torch.distributed as dist

    from oracle import lucid_oracle as O

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
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
        from lucid_b200.nn.quantized.sharded import (ColumnShardedLinear, HiddenExchange, PeerOutputs,
                                                     TokenShardedEncoder)

        def host(t):
            return (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()

        def same(t, ref):
            return bool(np.array_equal(host(t), ref))

        g = torch.Generator(device=dev).manual_seed(7)  # same data on every rank
        m, k, n = 520, 512, 1536
        x = torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16)
        wq = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev, generator=g)
        ws = torch.rand(n, device=dev, generator=g) * 1e-2 + 1e-3
        bias = torch.randn(n, device=dev, generator=g)
        # the oracle's single-GPU result: per-token encode -> exact accumulators -> f32 epilogue -> bf16
        xq, xs = O.per_token_quantize(host(x))
        acc = O.int_gemm_exact(xq, host(wq))
        full_ref = O.bf16_round(O.epilogue_f32(acc, xs, 0, None, host(ws), host(bias)))
        a, s = Q.quantize_per_token(x, Q.qint8)
        ok = same(a, xq) and same(s, xs.astype(np.float32))
        ok = ok and same(QF.gemm_s8(a, wq, out_dtype=torch.bfloat16, a_scale=s, b_scale=ws, bias=bias), full_ref)
        lin = ColumnShardedLinear.from_full(wq, ws, bias, world, rank)
        ok = ok and same(lin.forward_codes(a, s), full_ref)          # NCCL all-gather
        lin.use_peer_outputs(max_rows=m)
        for _ in range(3):                                            # device-flag exchange, alternating buffers
            ok = ok and same(lin.forward_codes(a, s), full_ref)
        ok = ok and same(lin(x), full_ref)
        ret[f"linear{rank}"] = bool(ok)
        # gated: [gate; up] interleaved per rank, output columns = ff / world per rank
        ff = 1024
        gq = torch.randint(-127, 128, (ff, k), dtype=torch.int8, device=dev, generator=g)
        uq = torch.randint(-127, 128, (ff, k), dtype=torch.int8, device=dev, generator=g)
        gs = torch.rand(ff, device=dev, generator=g) * 1e-2 + 1e-3
        us = torch.rand(ff, device=dev, generator=g) * 1e-2 + 1e-3
        yg = O.epilogue_f32(O.int_gemm_exact(xq, host(gq)), xs, 0, None, host(gs), None)
        yu = O.epilogue_f32(O.int_gemm_exact(xq, host(uq)), xs, 0, None, host(us), None)
        h_oracle = O.silu_f32(yg) * yu
        h_full = QF.gemm_s8(a, interleave_gate_up(gq, uq), out_dtype=torch.bfloat16, a_scale=s,
                            b_scale=interleave_gate_up(gs, us), act=_lib.ACT_SILU_GATE)
        # the SiLU goes through a library exp: tolerance against the oracle, bit-equality between
        # the sharded and the single-GPU kernel
        ok = ok and float(np.abs(host(h_full) - h_oracle).max() / np.abs(h_oracle).max()) < 1e-2
        per = ff // world
        sl = slice(rank * per, (rank + 1) * per)
        gl = ColumnShardedLinear(k, 2 * ff, world, rank)
        gl.weight_int8 = interleave_gate_up(gq[sl].contiguous(), uq[sl].contiguous())
        gl.weight_scale = interleave_gate_up(gs[sl].contiguous(), us[sl].contiguous())
        gl = gl.to(dev)
        gl.use_peer_outputs(max_rows=m, gated=True)
        for _ in range(2):
            ok = ok and torch.equal(gl.forward_codes(a, s, act=_lib.ACT_SILU_GATE), h_full)
        ret[f"gated{rank}"] = bool(ok)
        # the gated output feeding a per-token encode: shard kept local, per-token abs-max
        # exchanged, codes stored into every rank's operand buffer == the oracle's per-token encode
        # of the unsharded tensor
        hq_ref, hs_ref = O.per_token_quantize(host(h_full))
        h_local = QF.gemm_s8(a, gl.weight_int8, out_dtype=torch.bfloat16, a_scale=s, b_scale=gl.weight_scale,
                             act=_lib.ACT_SILU_GATE)
        ok = ok and torch.equal(h_local, h_full[:, sl])
        hx = HiddenExchange(m, ff, dev)
        for it in range(4):
            # unicast peer stores, then (where the buffers have one) the NVSwitch multicast address
            mc = it >= 2 and hx.out.has_multicast
            hx.out.bufs[0].fill_(77)
            torch.cuda.synchronize()
            dist.barrier()
            codes, scales = hx(h_local, multicast=mc)
            ok = ok and same(codes, hq_ref) and same(scales, hs_ref.astype(np.float32))
            torch.cuda.synchronize()
            dist.barrier()
        ret[f"hidden{rank}"] = bool(ok)
        # token-sharded encode of a replicated input: every rank ends up with all rows
        m2 = 512
        x2 = torch.randn(m2, k, device=dev, generator=g).to(torch.bfloat16)
        x2q, x2s = O.per_token_quantize(host(x2))
        enc = TokenShardedEncoder(m2, k, dev)
        for it in range(3):
            codes, scales = enc(x2, multicast=it == 2)
            ok = ok and same(codes, x2q) and same(scales, x2s.astype(np.float32))
            torch.cuda.synchronize()
            dist.barrier()
        codes, scales = enc(x2[rank * (m2 // world):(rank + 1) * (m2 // world)], local=True)
        ok = ok and same(codes, x2q) and same(scales, x2s.astype(np.float32))
        ret[f"encoder{rank}"] = bool(ok)
        # the GEMM epilogue through the multicast address, signalled by the kernel itself
        outs = PeerOutputs(m, n, torch.bfloat16, dev)
        if outs.has_multicast:
            npr = n // world
            for _ in range(2):
                buf, mc_ptr = outs.next(multicast=True)
                buf.fill_(0)
                torch.cuda.synchronize()
                dist.barrier()
                QF.gemm_s8_bcast(a, wq[rank * npr:(rank + 1) * npr].contiguous(), mc_ptr, (m, n), rank * npr,
                                 a_scale=s, b_scale=ws[rank * npr:(rank + 1) * npr].contiguous(),
                                 bias=bias[rank * npr:(rank + 1) * npr].contiguous(), signal=outs.sync.signal_arg)
                outs.sync.wait()
                ok = ok and same(buf, full_ref)
        ret["multicast"] = bool(outs.has_multicast)
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
