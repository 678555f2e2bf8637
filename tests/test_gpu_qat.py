"""FakeQuantize module and the QAT workflow on the GPU (fixtures made by executing the
reference's _fake_quantize.py)."""

import numpy as np
import pytest
import torch

import lucid_b200.nn.qat as nnqat
import lucid_b200.nn.quantized as nnq
import lucid_b200.quantization as Q
from gpu_util import dev, host

pytestmark = pytest.mark.gpu


def test_fake_quantize_module_golden(golden):
    fq = Q.FakeQuantize(observer=Q.MovingAverageMinMaxObserver, averaging_constant=0.1)
    for i in range(3):
        y = fq(dev(golden[f"fqm_x{i}"]))
        assert np.array_equal(host(y), golden[f"fqm_y{i}"]), i
        assert [fq.scale.item(), fq.zero_point.item()] == golden[f"fqm_qp{i}"].tolist()
    fq.disable_observer()
    assert np.array_equal(host(fq(dev(golden["fqm_xwide"]))), golden["fqm_ywide"])
    assert [fq.scale.item(), fq.zero_point.item()] == golden["fqm_qpwide"].tolist()
    x = dev(golden["fqm_xwide"])
    assert fq.disable_fake_quant()(x) is x
    wfq = Q.FakeQuantize(observer=Q.PerChannelMinMaxObserver, ch_axis=0, qscheme=Q.per_channel_symmetric,
                         qdtype=Q.qint8)
    assert np.array_equal(host(wfq(dev(golden["fqm_w"]))), golden["fqm_wy"])
    assert np.array_equal(host(wfq.scale), golden["fqm_wscale"])
    assert np.array_equal(host(wfq.zero_point), golden["fqm_wzp"])


def test_fake_quantize_module_ste_gradient():
    """The backward is the straight-through mask: 1 inside the grid, 0 where the code clipped
    (lucid/quantization/_functional.py:315-331)."""
    fq = Q.FakeQuantize(observer=Q.MinMaxObserver)
    fq(torch.tensor([-1.0, 0.0, 2.0], device="cuda"))
    fq.disable_observer()
    x = torch.tensor([-100.0, -0.9, 0.3, 1.9, 100.0], device="cuda", requires_grad=True)
    fq(x).sum().backward()
    assert x.grad.tolist() == [0.0, 1.0, 1.0, 1.0, 0.0]


def test_qat_workflow_trains_and_converts():
    torch.manual_seed(0)
    model = torch.nn.Sequential(Q.QuantStub(), torch.nn.Linear(64, 128), torch.nn.ReLU(),
                                torch.nn.Linear(128, 32), Q.DeQuantStub()).cuda()
    qat = Q.prepare_qat(model)
    assert type(qat[1]) is nnqat.Linear and isinstance(qat[1].weight_fake_quant, Q.FakeQuantize)
    assert qat.training
    x = torch.randn(256, 64, device="cuda")
    target = model(x).detach()
    opt = torch.optim.SGD(qat.parameters(), lr=1e-2)
    losses = []
    for _ in range(5):
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(qat(x), target)
        loss.backward()
        assert qat[1].weight.grad is not None and torch.isfinite(qat[1].weight.grad).all()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] <= losses[0]
    qat.eval()
    y_qat = qat(x)
    qmodel = Q.convert(qat)
    assert type(qmodel[1]) is nnq.Linear and type(qmodel[3]) is nnq.Linear
    assert qmodel[1].weight_int8.dtype == torch.int8
    y_q = qmodel(x)
    # the converted model reproduces what QAT simulated, up to the input grid it adds
    err = float((y_q - y_qat).abs().mean() / y_qat.abs().mean())
    assert err < 0.05, err


def test_prepare_qat_conv_and_no_match():
    m = Q.prepare_qat(torch.nn.Sequential(torch.nn.Conv2d(16, 16, 3, padding=1)).cuda())
    assert type(m[0]) is nnqat.Conv2d
    y = m(torch.randn(2, 16, 8, 8, device="cuda"))
    assert y.shape == (2, 16, 8, 8)
    with pytest.warns(UserWarning):
        Q.prepare_qat(torch.nn.Sequential(torch.nn.ReLU()))
