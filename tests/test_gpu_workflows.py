"""Eager-mode workflows on the GPU: prepare -> calibrate -> convert, quantize_dynamic and
the checkpoint round trip, with the accuracy gates of the reference's own tests
(lucid/test/unit/quantization/test_static_ptq.py:86,131-145, test_dynamic_ptq.py:46)."""

import io

import pytest
import torch

pytestmark = pytest.mark.gpu

import lucid_b200.nn.quantized as nnq  # noqa: E402
import lucid_b200.quantization as Q  # noqa: E402


def _mlp():
    torch.manual_seed(0)
    return torch.nn.Sequential(Q.QuantStub(), torch.nn.Linear(128, 256), torch.nn.ReLU(),
                               torch.nn.Linear(256, 64), Q.DeQuantStub()).cuda()


def _mean_rel_err(a, b):
    return float((a - b).abs().mean() / b.abs().mean())


def test_static_ptq_mlp_and_checkpoint_round_trip():
    model = _mlp()
    x = torch.randn(512, 128, device="cuda")
    y_float = model(x)
    prepared = Q.prepare(model)
    for _ in range(3):
        prepared(torch.randn(512, 128, device="cuda"))
    prepared(x)
    qmodel = Q.convert(prepared)
    assert type(qmodel[0]) is nnq.Quantize and type(qmodel[1]) is nnq.Linear
    assert type(qmodel[3]) is nnq.Linear and type(qmodel[4]) is nnq.DeQuantize
    assert qmodel[1].weight_int8.dtype == torch.int8
    assert list(qmodel[1].state_dict()) == ["weight_int8", "weight_scale", "weight_zero_point",
                                            "bias", "scale", "zero_point"]
    y_q = qmodel(x)
    assert _mean_rel_err(y_q, y_float) < 0.05
    # checkpoint round trip: bit-equal outputs
    buf = io.BytesIO()
    torch.save(qmodel.state_dict(), buf)
    buf.seek(0)
    assert type(qmodel[2]) is nnq.ReLU  # plain ReLU on floats; keeps integer codes alive
    clone = torch.nn.Sequential(nnq.Quantize(), nnq.Linear(128, 256), nnq.ReLU(),
                                nnq.Linear(256, 64), nnq.DeQuantize()).cuda()
    clone.load_state_dict(torch.load(buf))
    for a, b in ((clone[1], qmodel[1]), (clone[3], qmodel[3])):
        a.out_qdtype = b.out_qdtype
    clone[0].qdtype = qmodel[0].qdtype
    assert torch.equal(clone(x), y_q)


def test_static_ptq_conv_stack():
    torch.manual_seed(1)
    import torch.ao.nn.intrinsic as nni

    model = torch.nn.Sequential(
        Q.QuantStub(),
        nni.ConvReLU2d(torch.nn.Conv2d(16, 32, 3, padding=1), torch.nn.ReLU()),
        nni.ConvReLU2d(torch.nn.Conv2d(32, 32, 1), torch.nn.ReLU()),
        torch.nn.Conv2d(32, 16, 3, padding=1),
    ).cuda()
    x = torch.randn(4, 16, 14, 14, device="cuda")
    y_float = model(x)
    prepared = Q.prepare(model)
    prepared(x)
    qmodel = Q.convert(prepared)
    assert type(qmodel[1]) is nnq.ConvReLU2d and type(qmodel[3]) is nnq.Conv2d
    qmodel[0].nhwc = True  # hand NHWC codes to the conv stack
    y_q = qmodel(x)
    assert y_q.shape == y_float.shape
    assert _mean_rel_err(y_q, y_float) < 0.05


def test_quantize_dynamic_mlp():
    torch.manual_seed(2)
    model = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.ReLU(),
                                torch.nn.Linear(512, 32)).cuda()
    x = torch.randn(64, 256, device="cuda")
    qmodel = Q.quantize_dynamic(model)
    assert type(qmodel[0]) is nnq.dynamic.Linear and type(qmodel[2]) is nnq.dynamic.Linear
    assert _mean_rel_err(qmodel(x), model(x)) < 0.05
    with pytest.warns(UserWarning):
        Q.quantize_dynamic(torch.nn.Sequential(torch.nn.Conv2d(16, 16, 3)).cuda())


def test_prepare_without_match_warns():
    with pytest.warns(UserWarning):
        Q.prepare(torch.nn.Sequential(torch.nn.ReLU()))


def test_conv_transpose_runs_the_reference_sequence():
    """dequantize(weight, ch_axis=1) -> float transposed conv -> fake_quantize
    (lucid/nn/quantized/conv_transpose.py:112-130), through prepare / convert."""
    import numpy as np

    from gpu_util import host
    from oracle import lucid_oracle as O

    torch.manual_seed(3)
    model = torch.nn.Sequential(Q.QuantStub(), torch.nn.ConvTranspose2d(8, 12, 3, stride=2, padding=1,
                                                                        output_padding=1)).cuda()
    x = torch.randn(2, 8, 9, 9, device="cuda")
    prepared = Q.prepare(model)
    prepared(x)
    qmodel = Q.convert(prepared)
    ct = qmodel[1]
    assert type(ct) is nnq.ConvTranspose2d and tuple(ct.weight_int8.shape) == (8, 12, 3, 3)
    assert list(ct.state_dict()) == ["weight_int8", "weight_scale", "weight_zero_point", "bias", "scale",
                                     "zero_point"]
    w = host(model[1].weight.detach())
    s_o, z_o = O.calculate_qparams(*O.per_channel_minmax_observe(w, ch_axis=1), True, O.QINT8)
    assert np.array_equal(host(ct.weight_scale), s_o)
    assert np.array_equal(host(ct.weight_int8), O.quantize(w, s_o, z_o, O.QINT8, ch_axis=1))
    xq = qmodel[0](x)
    y = ct(xq)
    w_dq = torch.from_numpy(O.dequantize(host(ct.weight_int8), s_o, z_o, ch_axis=1)).cuda()
    from lucid_b200 import _lib

    assert not ct._int8_ok()  # 8 input channels: the float route (the integer kernel wants multiples of 16)
    with _lib.ieee_float32():  # binary32 arithmetic, as the module's float route runs it
        y_f = torch.nn.functional.conv_transpose2d(xq.detach(), w_dq, ct.bias, 2, 1, 1)
    want = O.fake_quantize(host(y_f), float(ct.scale), float(ct.zero_point), 0, 255)
    assert np.array_equal(host(y), want)
    assert _mean_rel_err(y, model(x).detach()) < 0.08
