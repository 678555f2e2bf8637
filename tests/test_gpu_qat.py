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
    # a target the copied weights do not already meet: the loss starts far above the rounding
    # noise of the grids, so its descent does not depend on that noise
    target = model(x).detach() * 1.5
    opt = torch.optim.SGD(qat.parameters(), lr=1e-2)
    losses = []
    for _ in range(5):
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(qat(x), target)
        loss.backward()
        assert qat[1].weight.grad is not None and torch.isfinite(qat[1].weight.grad).all()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]
    qat.eval()
    y_qat = qat(x)
    qmodel = Q.convert(qat)
    assert type(qmodel[0]) is nnq.Quantize  # the entry grid trained by the stub's fake-quantizer
    assert type(qmodel[1]) is nnq.Linear and type(qmodel[3]) is nnq.Linear
    assert qmodel[1].weight_int8.dtype == torch.int8
    y_q = qmodel(x)
    # the converted model reproduces what QAT simulated
    err = float((y_q - y_qat).abs().mean() / y_qat.abs().mean())
    assert err < 0.05, err


def test_prepare_qat_conv_and_no_match():
    m = Q.prepare_qat(torch.nn.Sequential(torch.nn.Conv2d(16, 16, 3, padding=1)).cuda())
    assert type(m[0]) is nnqat.Conv2d
    y = m(torch.randn(2, 16, 8, 8, device="cuda"))
    assert y.shape == (2, 16, 8, 8)
    with pytest.warns(UserWarning):
        Q.prepare_qat(torch.nn.Sequential(torch.nn.ReLU()))


class _ConvBnNet(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.quant = Q.QuantStub()
        self.conv1, self.bn1, self.relu1 = torch.nn.Conv2d(16, 32, 3, padding=1, bias=False), torch.nn.BatchNorm2d(32), torch.nn.ReLU()
        self.conv2, self.bn2 = torch.nn.Conv2d(32, 32, 3, stride=2, padding=1), torch.nn.BatchNorm2d(32)
        self.dequant = Q.DeQuantStub()

    def forward(self, x):
        x = self.relu1(self.bn1(self.conv1(self.quant(x))))
        return self.dequant(self.bn2(self.conv2(x)))


def _bn_net():
    torch.manual_seed(3)
    net = _ConvBnNet().cuda()
    with torch.no_grad():
        for bn in (net.bn1, net.bn2):
            bn.running_mean.normal_(0, 0.2)
            bn.running_var.uniform_(0.5, 1.5)
            bn.weight.uniform_(0.5, 1.5)
            bn.bias.normal_(0, 0.2)
    return net


def test_static_ptq_with_batchnorm_reaches_the_integer_conv():
    """fuse_modules -> prepare -> calibrate -> convert on a Conv/BN/ReLU model: BatchNorm is folded
    (exact at eval time, the reference's gate test_static_ptq.py:90-99) and the converted model
    runs integer convolutions only (the strided one included)."""
    from lucid_b200 import _lib

    net = _bn_net().eval()
    x = torch.randn(4, 16, 20, 20, device="cuda")
    fused = Q.fuse_modules(net, [["conv1", "bn1", "relu1"], ["conv2", "bn2"]])
    with _lib.ieee_float32(), torch.no_grad():  # the library's convolutions default to TF32
        y_float = net(x)
        assert torch.allclose(fused(x), y_float, atol=1e-4)
    prepared = Q.prepare(fused, Q.QConfig(activation=Q.MinMaxObserver, weight=Q.get_default_qconfig().weight))
    with torch.no_grad():
        prepared(x)
    qnet = Q.convert(prepared)
    assert type(qnet.conv1) is nnq.ConvReLU2d and type(qnet.conv2) is nnq.Conv2d
    assert qnet.conv1._int8_ok() and qnet.conv2._int8_ok() and qnet.conv2.stride == (2, 2)
    y_q = qnet(x)
    assert float((y_q - y_float).abs().mean() / y_float.abs().mean()) < 0.05


@pytest.mark.parametrize("rank", [1, 3])
def test_qat_conv_bn_fusion_of_the_other_ranks(rank):
    """ConvBn1d / ConvBn3d (lucid/nn/intrinsic/qat/modules.py:30-90, 796-833;
    lucid/quantization/fuse_modules.py:190-205): the fused module trains, keeps its BatchNorm
    live, and converts to the inference layer of its rank, which reproduces what QAT simulated."""
    from lucid_b200.nn.intrinsic import qat as nniqat

    conv_t = (torch.nn.Conv1d, None, torch.nn.Conv3d)[rank - 1]
    bn_t = (torch.nn.BatchNorm1d, None, torch.nn.BatchNorm3d)[rank - 1]
    torch.manual_seed(5 + rank)
    net = torch.nn.Sequential(Q.QuantStub(), conv_t(16, 32, 3, padding=1, bias=False), bn_t(32), torch.nn.ReLU(),
                              conv_t(32, 32, 3, stride=2, padding=1), bn_t(32), Q.DeQuantStub()).cuda().train()
    with torch.no_grad():
        for bn in (net[2], net[5]):
            bn.running_mean.normal_(0, 0.2)
            bn.running_var.uniform_(0.5, 1.5)
            bn.weight.uniform_(0.5, 1.5)
            bn.bias.normal_(0, 0.2)
    qcfg = Q.get_default_qat_qconfig()
    fused = Q.fuse_modules_qat(net, [["1", "2", "3"], ["4", "5"]], qcfg)
    assert type(fused[1]) is getattr(nniqat, f"ConvBnReLU{rank}d") and type(fused[4]) is getattr(nniqat, f"ConvBn{rank}d")
    qat = Q.prepare_qat(fused, qcfg)
    assert type(qat[1]) is getattr(nniqat, f"ConvBnReLU{rank}d") and type(qat[1].conv) is conv_t
    x = torch.randn(4, 16, *([12] * rank), device="cuda")
    opt = torch.optim.SGD(qat.parameters(), lr=1e-3)
    mean0 = qat[1].bn.running_mean.clone()
    for _ in range(2):
        opt.zero_grad()
        qat(x).square().mean().backward()
        assert qat[1].conv.weight.grad is not None and qat[1].bn.weight.grad is not None
        opt.step()
    assert not torch.equal(qat[1].bn.running_mean, mean0)
    qat.eval()
    with torch.no_grad():
        y_qat = qat(x)
    qnet = Q.convert(qat)
    assert type(qnet[1]) is getattr(nnq, f"ConvReLU{rank}d") and type(qnet[4]) is getattr(nnq, f"Conv{rank}d")
    _, b_fold = qat[1]._fold()
    assert torch.equal(qnet[1].bias, b_fold.detach())
    with torch.no_grad():
        y_q = qnet(x)
    assert y_q.shape == y_qat.shape
    assert float((y_q - y_qat).abs().mean() / y_qat.abs().mean()) < 0.05


def test_qat_conv_bn_fusion_trains_and_converts():
    """fuse_modules_qat -> prepare_qat -> a few steps -> convert
    (lucid/nn/intrinsic/qat/modules.py:30-90, 796-833): BatchNorm stays trainable inside the fused
    module, the weight grid is that of the FOLDED weight, and the converted integer layers
    reproduce what QAT simulated."""
    from lucid_b200.nn.intrinsic import qat as nniqat

    net = _bn_net().train()
    qcfg = Q.get_default_qat_qconfig()
    fused = Q.fuse_modules_qat(net, [["conv1", "bn1", "relu1"], ["conv2", "bn2"]], qcfg)
    assert type(fused.conv1) is nniqat.ConvBnReLU2d and type(fused.conv2) is nniqat.ConvBn2d
    qat = Q.prepare_qat(fused, qcfg)
    assert type(qat.conv1) is nniqat.ConvBnReLU2d and type(qat.conv1.conv) is torch.nn.Conv2d
    x = torch.randn(4, 16, 20, 20, device="cuda")
    target = torch.randn(4, 32, 10, 10, device="cuda")
    opt = torch.optim.SGD(qat.parameters(), lr=1e-3)
    mean0 = qat.conv1.bn.running_mean.clone()
    for _ in range(3):
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(qat(x), target)
        loss.backward()
        assert qat.conv1.conv.weight.grad is not None and qat.conv1.bn.weight.grad is not None
        opt.step()
    assert not torch.equal(qat.conv1.bn.running_mean, mean0)  # the statistics kept learning
    qat.eval()
    with torch.no_grad():
        y_qat = qat(x)
    qnet = Q.convert(qat)
    assert type(qnet.conv1) is nnq.ConvReLU2d and type(qnet.conv2) is nnq.Conv2d
    w_fold, b_fold = qat.conv1._fold()
    assert torch.equal(qnet.conv1.bias, b_fold.detach())
    assert torch.equal(Q.dequantize(qnet.conv1.weight_int8, qnet.conv1.weight_scale, qnet.conv1.weight_zero_point,
                                    ch_axis=0), qat.conv1.weight_fake_quant(w_fold.detach()))
    with torch.no_grad():
        y_q = qnet(x)
    assert float((y_q - y_qat).abs().mean() / y_qat.abs().mean()) < 0.05


@pytest.mark.parametrize("rank", [1, 2, 3])
def test_qat_fused_relu_layers_of_every_rank_convert(rank):
    """[Conv, ReLU] / [Linear, ReLU] runs under QAT (lucid/quantization/_quantize.py:557-572,
    lucid/nn/qat/conv.py:469-800): prepare_qat builds nn.qat.ConvReLU{rank}d / LinearReLU, they
    train through the straight-through mask, and convert produces the fused inference layers."""
    conv_t = (torch.nn.Conv1d, torch.nn.Conv2d, torch.nn.Conv3d)[rank - 1]
    torch.manual_seed(20 + rank)
    net = torch.nn.Sequential(Q.QuantStub(), conv_t(16, 32, 3, padding=1), torch.nn.ReLU(), conv_t(32, 16, 1),
                              torch.nn.Flatten(), torch.nn.LazyLinear(16), torch.nn.ReLU(), Q.DeQuantStub()).cuda()
    x = torch.randn(4, 16, *([8] * rank), device="cuda")
    net(x)  # materialise the lazy layer
    qcfg = Q.get_default_qat_qconfig()
    qat = Q.prepare_qat(Q.fuse_modules_qat(net, [["1", "2"], ["5", "6"]], qcfg), qcfg)
    assert type(qat[1]) is getattr(nnqat, f"ConvReLU{rank}d") and type(qat[3]) is getattr(nnqat, f"Conv{rank}d")
    assert type(qat[5]) is nnqat.LinearReLU
    assert isinstance(qat[0].activation_post_process, Q.FakeQuantize)  # the entry grid is trained too
    opt = torch.optim.SGD(qat.parameters(), lr=1e-3)
    for _ in range(2):
        opt.zero_grad()
        qat(x).square().mean().backward()
        assert qat[1].weight.grad is not None and qat[5].weight.grad is not None
        opt.step()
    qat.eval()
    with torch.no_grad():
        y_qat = qat(x)
        assert float(y_qat.min()) >= 0.0  # the fused ReLU sits ahead of the output grid
    qnet = Q.convert(qat)
    assert type(qnet[1]) is getattr(nnq, f"ConvReLU{rank}d") and type(qnet[3]) is getattr(nnq, f"Conv{rank}d")
    assert type(qnet[5]) is nnq.LinearReLU and type(qnet[0]) is nnq.Quantize
    assert float(qnet[0].scale) == float(qat[0].activation_post_process.scale)
    with torch.no_grad():
        y_q = qnet(x)
    assert y_q.shape == y_qat.shape and bool(torch.isfinite(y_q).all())
    assert float((y_q - y_qat).abs().mean() / y_qat.abs().mean().clamp_min(1e-6)) < 0.15
