"""Quantized embedding tables on the GPU against the oracle (bit-exact: the gather decodes with
the dequantize arithmetic, the bag adds rows in index order)."""

import numpy as np
import pytest
import torch

import lucid_b200 as L
import lucid_b200.nn.quantized as nnq
import lucid_b200.quantization as Q
from gpu_util import dev, host
from lucid_b200 import _lib
from oracle import lucid_oracle as O

pytestmark = pytest.mark.gpu
F32 = np.float32


def _table(rows, dim, seed, padding_idx=None, cls=nnq.Embedding, **kw):
    torch.manual_seed(seed)
    if cls is nnq.Embedding:
        f = torch.nn.Embedding(rows, dim, padding_idx=padding_idx).cuda()
    else:
        f = torch.nn.EmbeddingBag(rows, dim, padding_idx=padding_idx, **kw).cuda()
    q = cls.from_float(f)
    return f, q, host(q.weight_int8), host(q.weight_scale), host(q.weight_zero_point)


@pytest.mark.parametrize("dim", [16, 64, 100, 4096])
@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_embedding_matches_oracle(dim, idx_dtype):
    f, q, wq, ws, wz = _table(500, dim, dim, padding_idx=7)
    # the table itself is the per-row symmetric encode of the float table
    s_o, z_o = O.calculate_qparams(*O.per_channel_minmax_observe(host(f.weight.detach())), True, O.QINT8)
    assert np.array_equal(ws, s_o) and np.array_equal(wq, O.quantize(host(f.weight.detach()), s_o, z_o, O.QINT8, ch_axis=0))
    g = np.random.default_rng(dim)
    idx = g.integers(0, 500, (9, 33))
    idx[0, :5] = 7
    got = q(dev(idx).to(idx_dtype))
    assert got.shape == (9, 33, dim) and got.dtype == torch.float32
    want = O.quantized_embedding(wq, ws, wz, idx, padding_idx=7)
    assert np.array_equal(host(got), want)
    assert float(np.abs(want - host(f(dev(idx)).detach())).max()) <= float(ws.max()) * 0.5 + 1e-7
    _lib.check_device_status(torch.device("cuda", 0))
    # bfloat16 output: the float32 row rounded once
    q.out_dtype = torch.bfloat16
    assert np.array_equal(host(q(dev(idx))), host(torch.from_numpy(want).to(torch.bfloat16)))


def test_embedding_out_of_range_is_recorded_not_read():
    _, q, wq, ws, wz = _table(50, 32, 1)
    idx = torch.tensor([3, 50, -1, 4], device="cuda")
    out = q(idx)
    want = O.quantized_embedding(wq, ws, wz, np.array([3, 0, 0, 4]))
    want[1:3] = 0
    assert np.array_equal(host(out), want)
    with pytest.raises(L.ShapeMismatch):
        _lib.check_device_status(torch.device("cuda", 0))
    _lib.check_device_status(torch.device("cuda", 0))  # the word was cleared


@pytest.mark.parametrize("mode", ["sum", "mean", "max"])
@pytest.mark.parametrize("dim", [8, 30, 256])
def test_embedding_bag_matches_oracle(mode, dim):
    _, q, wq, ws, wz = _table(300, dim, dim + 1, padding_idx=2, cls=nnq.EmbeddingBag, mode=mode)
    g = np.random.default_rng(dim)
    idx = g.integers(0, 300, 200)
    idx[10:14] = 2
    offsets = np.array([0, 5, 5, 40, 41, 120, 199])  # includes an empty bag
    got = q(dev(idx), dev(offsets))
    want = O.quantized_embedding_bag(wq, ws, wz, idx, offsets, mode=mode, padding_idx=2)
    assert np.array_equal(host(got), want)
    # 2-D input: one bag per row
    idx2 = g.integers(0, 300, (12, 17))
    got2 = q(dev(idx2))
    want2 = O.quantized_embedding_bag(wq, ws, wz, idx2.ravel(), np.arange(0, 12 * 17, 17), mode=mode, padding_idx=2)
    assert np.array_equal(host(got2), want2)
    # int32 indices
    assert np.array_equal(host(q(dev(idx).to(torch.int32), dev(offsets).to(torch.int32))), want)


def test_quantize_dynamic_swaps_embeddings():
    model = torch.nn.Sequential(torch.nn.Embedding(1000, 64), torch.nn.Linear(64, 32)).cuda()
    qmodel = Q.quantize_dynamic(model)
    assert type(qmodel[0]) is nnq.Embedding and type(qmodel[1]) is nnq.dynamic.Linear
    idx = torch.randint(0, 1000, (4, 10), device="cuda")
    y, yq = model(idx).detach(), qmodel(idx)
    assert float((y - yq).abs().mean() / y.abs().mean()) < 0.05
    assert list(qmodel[0].state_dict()) == ["weight_int8", "weight_scale", "weight_zero_point"]


def test_embedding_large_table_gather_only_reads_rows():
    """A 2^20 x 256 table (256 MB of codes): the lookup touches 4096 rows, not the table."""
    rows, dim = 1 << 20, 256
    q = nnq.Embedding(rows, dim).cuda()
    g = torch.Generator(device="cuda").manual_seed(0)
    q.weight_int8 = torch.randint(-127, 128, (rows, dim), device="cuda", generator=g, dtype=torch.int32).to(torch.int8)
    q.weight_scale = torch.rand(rows, device="cuda", generator=g) * 0.01 + 1e-3
    idx = torch.randint(0, rows, (4096,), device="cuda", generator=g)
    out = q(idx)
    sel = idx.cpu().numpy()
    want = O.dequantize(host(q.weight_int8[idx]), host(q.weight_scale[idx]), np.zeros(4096, dtype=F32), ch_axis=0)
    assert np.array_equal(host(out), want) and sel.shape == (4096,)


def test_static_convert_and_qat_swap_embeddings():
    """Tables convert without calibration (the always-convert set of
    lucid/quantization/_quantize.py:416), and ``prepare_qat`` routes them through
    ``nn.qat.Embedding`` (lucid/nn/qat/sparse.py:21-132), whose trained table converts to the same
    inference layer."""
    import lucid_b200.nn.qat as nnqat

    torch.manual_seed(9)
    model = torch.nn.Sequential(torch.nn.Embedding(500, 64, padding_idx=0), torch.nn.Linear(64, 32)).cuda()
    idx = torch.randint(0, 500, (4, 10), device="cuda")
    y = model(idx).detach()
    qstatic = Q.convert(model)  # no observers anywhere: only the table converts
    assert type(qstatic[0]) is nnq.Embedding and type(qstatic[1]) is torch.nn.Linear
    assert float((y - qstatic(idx)).abs().mean() / y.abs().mean()) < 0.05
    qat = Q.prepare_qat(model)
    assert type(qat[0]) is nnqat.Embedding and type(qat[1]) is nnqat.Linear
    qat(idx).square().mean().backward()
    assert qat[0].weight.grad is not None
    qnet = Q.convert(qat.eval())
    assert type(qnet[0]) is nnq.Embedding and type(qnet[1]) is nnq.Linear
    assert qnet[0].padding_idx == 0
    assert list(qnet[0].state_dict()) == ["weight_int8", "weight_scale", "weight_zero_point"]
    assert float((y - qnet(idx)).abs().mean() / y.abs().mean()) < 0.1
