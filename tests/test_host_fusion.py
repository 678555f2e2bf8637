"""Host logic of ``fuse_modules`` / ``fuse_modules_qat`` (CPU; the float model is plain torch):
the reference's fusion gate lucid/test/unit/quantization/test_static_ptq.py:86-99 (folding
BatchNorm into the convolution is exact at eval time, atol 1e-4) and its pattern rules
(lucid/quantization/fuse_modules.py:62-90)."""

import pytest
import torch

import lucid_b200.quantization as Q
from lucid_b200.nn.intrinsic import qat as nniqat


class _ConvNet(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.conv = torch.nn.Conv2d(3, 8, 3, padding=1)
        self.bn = torch.nn.BatchNorm2d(8)
        self.relu = torch.nn.ReLU()
        self.fc = torch.nn.Linear(8, 4)
        self.act = torch.nn.ReLU()

    def forward(self, x):
        y = self.relu(self.bn(self.conv(x)))
        return self.act(self.fc(y.mean(dim=(2, 3))))


def _net():
    torch.manual_seed(1)
    net = _ConvNet().eval()
    with torch.no_grad():
        net.bn.running_mean.normal_()
        net.bn.running_var.uniform_(0.5, 2.0)
        net.bn.weight.normal_()
        net.bn.bias.normal_()
    return net


def test_conv_bn_fold_matches():
    net = _net()
    x = torch.randn(2, 3, 8, 8)
    y_ref = net(x)
    fused = Q.fuse_modules(net, [["conv", "bn"]])
    assert torch.allclose(fused(x), y_ref, atol=1e-4)
    assert isinstance(fused.bn, torch.nn.Identity) and isinstance(net.bn, torch.nn.BatchNorm2d)  # a copy
    fused3 = Q.fuse_modules(net, [["conv", "bn", "relu"], ["fc", "act"]])
    assert type(fused3.conv).__name__ == "ConvReLU2d" and type(fused3.fc).__name__ == "LinearReLU"
    assert isinstance(fused3.relu, torch.nn.Identity) and isinstance(fused3.act, torch.nn.Identity)
    assert torch.allclose(fused3(x), y_ref, atol=1e-4)
    same = Q.fuse_modules(net, [["conv", "relu"]], inplace=True)
    assert same is net


def test_unsupported_patterns_raise():
    net = _net()
    with pytest.raises(ValueError):
        Q.fuse_modules(net, [["bn", "relu"]])
    with pytest.raises(ValueError):
        Q.fuse_modules(net, [["fc", "act", "relu"]])
    with pytest.raises(ValueError):
        Q.fuse_modules_qat(net, [["bn", "relu"]], Q.get_default_qat_qconfig())


def test_qat_fusion_keeps_batchnorm_live():
    net = _net()
    qcfg = Q.QConfig(activation=torch.nn.Identity, weight=torch.nn.Identity)  # structure only: no kernels on CPU
    fused = Q.fuse_modules_qat(net, [["conv", "bn", "relu"]], qcfg)
    assert isinstance(fused.conv, nniqat.ConvBnReLU2d) and isinstance(fused.conv.bn, torch.nn.BatchNorm2d)
    assert isinstance(fused.bn, torch.nn.Identity)
    x = torch.randn(2, 3, 8, 8)
    assert torch.allclose(fused.eval()(x), net(x), atol=1e-4)  # identity "fake-quantizers": the fold alone
    w, b = fused.conv._fold()
    ref = Q.fuse_conv_bn_eval(net.conv, net.bn)
    assert torch.equal(w, ref.weight) and torch.equal(b, ref.bias)
    with pytest.raises(ValueError):
        nniqat.ConvBn2d(net.conv, net.bn, qconfig=None)


def _ranked(rank):
    """Conv + BatchNorm + ReLU of one rank with non-trivial statistics, and an input for it."""
    torch.manual_seed(10 + rank)
    conv_t = (torch.nn.Conv1d, torch.nn.Conv2d, torch.nn.Conv3d)[rank - 1]
    bn_t = (torch.nn.BatchNorm1d, torch.nn.BatchNorm2d, torch.nn.BatchNorm3d)[rank - 1]
    net = torch.nn.Sequential(conv_t(3, 8, 3, padding=1, bias=rank != 2), bn_t(8), torch.nn.ReLU()).eval()
    with torch.no_grad():
        net[1].running_mean.normal_()
        net[1].running_var.uniform_(0.5, 2.0)
        net[1].weight.normal_()
        net[1].bias.normal_()
    return net, torch.randn(2, 3, *([6] * rank))


@pytest.mark.parametrize("rank", [1, 2, 3])
def test_fusion_covers_the_three_ranks(rank):
    """The rank picks the fused type (lucid/quantization/fuse_modules.py:62-90, 190-205): static
    fusion folds BatchNorm{1,2,3}d exactly and wraps the ReLU in ConvReLU{1,2,3}d; QAT fusion
    builds ConvBn{1,2,3}d / ConvBnReLU{1,2,3}d with the BatchNorm kept live."""
    net, x = _ranked(rank)
    y_ref = net(x)
    fused = Q.fuse_modules(net, [["0", "1", "2"]])
    assert type(fused[0]).__name__ == f"ConvReLU{rank}d"
    assert isinstance(fused[1], torch.nn.Identity) and isinstance(fused[2], torch.nn.Identity)
    assert torch.allclose(fused(x), y_ref, atol=1e-4)
    plain = Q.fuse_modules(net, [["0", "1"]])
    assert type(plain[0]) is type(net[0]) and torch.allclose(plain(x), y_ref, atol=1e-4)
    qcfg = Q.QConfig(activation=torch.nn.Identity, weight=torch.nn.Identity)  # structure only: no kernels on CPU
    qat = Q.fuse_modules_qat(net, [["0", "1", "2"]], qcfg)
    assert type(qat[0]) is getattr(nniqat, f"ConvBnReLU{rank}d") and type(qat[0].bn) is type(net[1])
    assert torch.allclose(qat.eval()(x), y_ref, atol=1e-4)
    qat2 = Q.fuse_modules_qat(net, [["0", "1"]], qcfg)
    assert type(qat2[0]) is getattr(nniqat, f"ConvBn{rank}d")
    w, b = qat2[0]._fold()
    ref = Q.fuse_conv_bn_eval(net[0], net[1])
    assert torch.equal(w, ref.weight) and torch.equal(b, ref.bias)


def test_fusion_rejects_a_batchnorm_of_another_rank():
    net, _ = _ranked(1)
    other = torch.nn.BatchNorm2d(8)
    with pytest.raises(TypeError):
        Q.fuse_conv_bn_eval(net[0], other)
    with pytest.raises(TypeError):
        nniqat.ConvBn1d(net[0], other, qconfig=Q.QConfig(activation=torch.nn.Identity, weight=torch.nn.Identity))
    with pytest.raises(TypeError):
        nniqat.ConvBn3d(net[0], net[1], qconfig=Q.QConfig(activation=torch.nn.Identity, weight=torch.nn.Identity))


def test_prepare_qat_maps_every_rank_and_fused_container():
    """The QAT map of lucid/quantization/_quantize.py:557-572: Linear, Conv{1,2,3}d and the fused
    LinearReLU / ConvReLU{1,2,3}d containers each become the ``nn.qat`` layer of the same name; the
    fused forms apply their ReLU before the output fake-quantize.  Identity "fake-quantizers"
    keep this on the CPU: the forward must then equal the float model's."""
    import lucid_b200.nn.qat as nnqat

    torch.manual_seed(4)
    qcfg = Q.QConfig(activation=torch.nn.Identity, weight=torch.nn.Identity)
    for rank in (1, 2, 3):
        conv_t = (torch.nn.Conv1d, torch.nn.Conv2d, torch.nn.Conv3d)[rank - 1]
        net = torch.nn.Sequential(conv_t(3, 8, 3, padding=1), torch.nn.ReLU(), conv_t(8, 4, 1, bias=False)).eval()
        x = torch.randn(2, 3, *([6] * rank))
        y_ref = net(x)
        fused = Q.fuse_modules_qat(net, [["0", "1"]], qcfg)
        qat = Q.prepare_qat(fused, qcfg)
        assert type(qat[0]) is getattr(nnqat, f"ConvReLU{rank}d") and type(qat[2]) is getattr(nnqat, f"Conv{rank}d")
        assert isinstance(qat[0], conv_t) and qat.training
        assert qat[0].weight is fused[0][0].weight or torch.equal(qat[0].weight, net[0].weight)
        assert torch.allclose(qat.eval()(x), y_ref, atol=1e-6)
    lin = torch.nn.Sequential(torch.nn.Linear(8, 4), torch.nn.ReLU(), torch.nn.Linear(4, 2)).eval()
    x = torch.randn(5, 8)
    qat = Q.prepare_qat(Q.fuse_modules_qat(lin, [["0", "1"]], qcfg), qcfg)
    assert type(qat[0]) is nnqat.LinearReLU and type(qat[2]) is nnqat.Linear
    assert torch.allclose(qat.eval()(x), lin(x), atol=1e-6)
    with pytest.raises(ValueError):
        nnqat.ConvReLU1d(3, 8, 3, qconfig=None)
    with pytest.raises(ValueError):
        nnqat.LinearReLU(3, 8, qconfig=None)


def test_prepare_qat_swaps_embedding_tables():
    """``nn.qat.Embedding`` (lucid/nn/qat/sparse.py:21-132): the table is looked up through its
    weight fake-quantizer, there is no output fake-quantizer, and a qconfig is mandatory."""
    import lucid_b200.nn.qat as nnqat

    torch.manual_seed(6)
    qcfg = Q.QConfig(activation=torch.nn.Identity, weight=torch.nn.Identity)
    net = torch.nn.Sequential(torch.nn.Embedding(20, 8, padding_idx=0), torch.nn.Linear(8, 4)).eval()
    idx = torch.tensor([[1, 0, 5], [19, 3, 3]])
    qat = Q.prepare_qat(net, qcfg)
    assert type(qat[0]) is nnqat.Embedding and isinstance(qat[0], torch.nn.Embedding)
    assert qat[0].padding_idx == 0 and not hasattr(qat[0], "activation_post_process")
    assert qat[0].weight is net[0].weight or torch.equal(qat[0].weight, net[0].weight)
    assert torch.equal(qat.eval()(idx), net(idx))
    with pytest.raises(ValueError):
        nnqat.Embedding(20, 8)


def test_qconfig_mapping_resolution_and_routing():
    """``QConfigMapping`` (lucid/quantization/qconfig.py:261-425): per-name beats per-type beats
    global, ``None`` excludes; ``prepare`` / ``prepare_qat`` observe or swap only what the mapping
    gives a qconfig (lucid/quantization/_quantize.py:195-201, 291-305, 661-681)."""
    import lucid_b200.nn.qat as nnqat

    a = Q.QConfig(activation=torch.nn.Identity, weight=torch.nn.Identity)
    b = Q.QConfig(activation=torch.nn.ReLU, weight=torch.nn.Identity)
    m = Q.QConfigMapping().set_global(a).set_object_type(torch.nn.Conv2d, b).set_module_name("head", None)
    assert m.get_qconfig(torch.nn.Linear, "body.fc") is a
    assert m.get_qconfig(torch.nn.Conv2d, "body.conv") is b
    assert m.get_qconfig(torch.nn.Conv2d, "head") is None          # the name wins over the type
    assert Q.QConfigMapping().get_qconfig(torch.nn.Linear, "x") is None
    assert isinstance(Q.get_default_qconfig_mapping().get_qconfig(torch.nn.Linear, "x"), Q.QConfig)
    assert isinstance(Q.get_default_qat_qconfig_mapping().get_qconfig(torch.nn.Linear, "x"), Q.QConfig)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.body = torch.nn.Sequential(torch.nn.Conv2d(3, 4, 1), torch.nn.Flatten(), torch.nn.Linear(64, 8))
            self.head = torch.nn.Linear(8, 2)

        def forward(self, x):
            return self.head(self.body(x))

    net = Net().eval()
    mapping = Q.QConfigMapping().set_global(a).set_object_type(torch.nn.Conv2d, b).set_module_name("head", None)
    prepared = Q.prepare(net, mapping)
    assert isinstance(prepared.body[0].activation_post_process, torch.nn.ReLU)       # by type
    assert isinstance(prepared.body[2].activation_post_process, torch.nn.Identity)   # global
    assert not hasattr(prepared.head, "activation_post_process")                     # excluded by name
    x = torch.randn(2, 3, 4, 4)
    assert torch.equal(prepared(x), net(x))  # observers change nothing
    qat = Q.prepare_qat(net, mapping)
    assert type(qat.body[0]) is nnqat.Conv2d and type(qat.body[2]) is nnqat.Linear
    assert type(qat.head) is torch.nn.Linear
    stubbed = Q.prepare_qat(Q.QuantWrapper(net), a)
    assert isinstance(stubbed.quant.activation_post_process, torch.nn.Identity) and stubbed.quant.qconfig is a
    assert not hasattr(stubbed.dequant, "activation_post_process")
    assert torch.equal(stubbed.eval()(x), net(x))  # only a FakeQuantize is applied by the stub
    skipped = Q.prepare_qat(Q.QuantWrapper(net), Q.QConfigMapping().set_global(a).set_module_name("quant", None))
    assert not hasattr(skipped.quant, "activation_post_process")
    with pytest.warns(UserWarning):
        Q.prepare(net, Q.QConfigMapping().set_object_type(torch.nn.Conv3d, a))
    with pytest.warns(UserWarning):
        Q.prepare_qat(net, Q.QConfigMapping())
    # a bare QConfig is the global tier
    assert hasattr(Q.prepare(net, a).head, "activation_post_process")


def test_stubs_and_wrapper_are_exported_where_the_reference_has_them():
    """``QuantStub`` / ``DeQuantStub`` / ``QuantWrapper`` (lucid/nn/quantized/modules.py:29-183,
    351-424; exported by lucid/nn/quantized/__init__.py:36-42): optional ``qconfig`` argument,
    identity forwards, wrapper = quant -> module -> dequant."""
    import lucid_b200.nn.quantized as nnq

    assert nnq.QuantStub is Q.QuantStub and nnq.DeQuantStub is Q.DeQuantStub and nnq.QuantWrapper is Q.QuantWrapper
    cfg = Q.QConfig(activation=torch.nn.Identity, weight=torch.nn.Identity)
    assert nnq.QuantStub(cfg).qconfig is cfg and not hasattr(nnq.QuantStub(), "qconfig")
    assert nnq.DeQuantStub(cfg).qconfig is cfg
    x = torch.randn(3, 5)
    assert nnq.QuantStub()(x) is x and nnq.DeQuantStub()(x) is x
    w = nnq.QuantWrapper(torch.nn.Linear(5, 2))
    assert [n for n, _ in w.named_children()] == ["quant", "module", "dequant"]
    assert torch.equal(w(x), w.module(x))
    prepared = Q.prepare(w.eval(), cfg)
    assert hasattr(prepared.quant, "activation_post_process") and hasattr(prepared.module, "activation_post_process")


def test_graph_mode_entry_points_wrap_the_model():
    """``prepare_fx`` (lucid/quantization/_quantize_fx.py:21-92; gate test_graph_mode.py:20-25): no
    hand-placed stubs, the model comes back inside a ``QuantWrapper`` with observers attached."""
    cfg = Q.QConfig(activation=torch.nn.Identity, weight=torch.nn.Identity)
    net = torch.nn.Sequential(torch.nn.Linear(6, 4), torch.nn.ReLU(), torch.nn.Linear(4, 2)).eval()
    prepared = Q.prepare_fx(net, cfg, example_inputs=torch.randn(1, 6))
    assert isinstance(prepared, Q.QuantWrapper) and prepared.module is not net
    assert hasattr(prepared.quant, "activation_post_process") and hasattr(prepared.module[0], "activation_post_process")
    x = torch.randn(3, 6)
    assert torch.equal(prepared(x), net(x))
    assert Q.convert_fx.__module__.endswith("_quantize_fx")


def test_reference_constructor_forms():
    """``ConvBnReLU*d(conv, bn, relu=True, qconfig=None)`` (lucid/nn/intrinsic/qat/modules.py:553-561)
    and the dynamic ``LSTM(shell)`` (lucid/nn/quantized/dynamic/rnn.py:54-64) take the reference's
    positional forms."""
    import lucid_b200.nn.quantized as nnq

    cfg = Q.QConfig(activation=torch.nn.Identity, weight=torch.nn.Identity)
    conv, bn = torch.nn.Conv2d(3, 4, 3), torch.nn.BatchNorm2d(4)
    x = torch.randn(2, 3, 8, 8)
    with torch.no_grad():
        assert float(nniqat.ConvBnReLU2d(conv, bn, True, cfg).eval()(x).min()) >= 0.0
        assert float(nniqat.ConvBnReLU2d(conv, bn, relu=False, qconfig=cfg).eval()(x).min()) < 0.0
    assert nniqat.ConvBnReLU2d(conv, bn, qconfig=cfg).relu is True
    with pytest.raises(ValueError):
        nniqat.ConvBnReLU2d(conv, bn, True)
    assert callable(nniqat.convbnrelu2d_to_quantized)
    shell = torch.nn.LSTM(8, 16, 2, bidirectional=True, batch_first=True)
    q = nnq.dynamic.LSTM(shell)
    assert (q.input_size, q.hidden_size, q.num_layers, q.bidirectional, q.batch_first) == (8, 16, 2, True, True)
    assert sorted(q.state_dict()) == sorted(nnq.dynamic.LSTM(8, 16, 2, True, True, True).state_dict())
    with pytest.raises(TypeError):
        nnq.dynamic.LSTM(8)
