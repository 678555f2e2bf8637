"""Host-side behaviour of the quantized convolution modules that needs no GPU: buffer shapes as
the reference stores them (lucid/nn/quantized/conv.py:232-385 keeps a 3-D ``weight_int8`` for
Conv1d), state-dict round trips, and the convert mapping of the 1-D / 3-D layers."""

import torch

import lucid_b200.nn.quantized as nnq
from lucid_b200.quantization import _quantize


def test_conv1d_state_dict_keeps_the_reference_weight_shape():
    m = nnq.Conv1d(16, 32, 5, stride=2, padding=2, dilation=1, groups=2)
    sd = m.state_dict()
    assert sd["weight_int8"].shape == (32, 8, 5) and m.weight_int8.shape == (32, 8, 1, 5)
    assert set(sd) == {"weight_int8", "weight_scale", "weight_zero_point", "bias", "scale", "zero_point"}
    sd["weight_int8"] = torch.randint(-128, 128, (32, 8, 5), dtype=torch.int8)
    other = nnq.ConvReLU1d(16, 32, 5, stride=2, padding=2, groups=2)
    other.load_state_dict(sd)
    assert torch.equal(other.weight_int8.squeeze(2), sd["weight_int8"])
    assert m.kernel_size == (1, 5) and m.stride == (1, 2) and m.padding == (0, 2)
    assert "kernel_size=(5,)" in repr(m)


def test_conv3d_buffers_and_mapping():
    m = nnq.Conv3d(4, 8, (3, 3, 1), padding=(1, 1, 0), bias=False)
    assert m.weight_int8.shape == (8, 4, 3, 3, 1) and m.bias is None
    mapping = _quantize._quant_mapping()
    for float_cls, q_cls in ((torch.nn.Conv1d, nnq.Conv1d), (torch.nn.Conv2d, nnq.Conv2d),
                             (torch.nn.Conv3d, nnq.Conv3d)):
        assert mapping[float_cls].__self__ is q_cls
    import lucid_b200.nn.intrinsic as nni

    assert mapping[nni.ConvReLU1d].__self__ is nnq.ConvReLU1d and mapping[nni.ConvReLU3d].__self__ is nnq.ConvReLU3d
