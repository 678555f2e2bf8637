"""Trainable Conv + BatchNorm (+ ReLU) fusions for quantization-aware training
(lucid/nn/intrinsic/qat/modules.py:30-90, 211-330, 564-680; conversion :796-833).

Each forward folds the BatchNorm's running statistics and affine parameters into the
convolution weight, fake-quantizes the FOLDED weight per output channel, convolves, applies
the optional ReLU and fake-quantizes the output -- so the weight grid the model trains against
is the grid ``convert`` will bake.  BatchNorm stays a live sub-module: its parameters keep
learning and the fold is recomputed every step.  The float convolution under the fake-quantize
ops is the library's (training path); ``convert`` turns the module into the inference layer
of its rank: the integer ``nn.quantized.Conv2d`` / ``ConvReLU2d`` and ``Conv1d`` / ``ConvReLU1d``,
or ``Conv3d`` / ``ConvReLU3d`` (which keep the reference's float sequence)."""

from __future__ import annotations

import torch
import torch.nn.functional as F


def fold_conv_bn(conv_w, conv_b, bn: torch.nn.modules.batchnorm._BatchNorm):
    """``(W * g / sqrt(var + eps),  (b - mean) * g / sqrt(var + eps) + beta)``: the eval-time
    fold of lucid/nn/utils/fusion.py:100-135 (same operation order)."""
    inv_std = (bn.running_var + bn.eps).rsqrt()
    scale = bn.weight * inv_std if bn.affine else inv_std
    w = conv_w * scale.reshape((-1,) + (1,) * (conv_w.dim() - 1))
    b = conv_b if conv_b is not None else torch.zeros_like(scale)
    b = (b - bn.running_mean) * scale
    if bn.affine:
        b = b + bn.bias
    return w, b


class _ConvBnNd(torch.nn.Module):
    _RELU = False
    _RANK = 2

    def __init__(self, conv: torch.nn.Module, bn: torch.nn.Module, qconfig=None) -> None:
        super().__init__()
        if qconfig is None:
            raise ValueError(f"{type(self).__name__} requires a qconfig")
        conv_t = (torch.nn.Conv1d, torch.nn.Conv2d, torch.nn.Conv3d)[self._RANK - 1]
        bn_t = (torch.nn.BatchNorm1d, torch.nn.BatchNorm2d, torch.nn.BatchNorm3d)[self._RANK - 1]
        if not isinstance(conv, conv_t) or not isinstance(bn, bn_t):
            raise TypeError(f"{type(self).__name__} fuses {conv_t.__name__} + {bn_t.__name__}, got "
                            f"{type(conv).__name__} + {type(bn).__name__}")
        self.conv, self.bn = conv, bn
        self.relu = self._RELU
        self.qconfig = qconfig
        self.weight_fake_quant = qconfig.weight()
        self.activation_post_process = qconfig.activation()

    def _fold(self):
        return fold_conv_bn(self.conv.weight, self.conv.bias, self.bn)

    def forward(self, x):
        if self.training and self.bn.training and self.bn.track_running_stats:
            # keep the running statistics learning: one BatchNorm pass over the un-folded
            # convolution's output updates them (its result is not used)
            with torch.no_grad():
                self.bn(self.conv(x))
        weight, bias = self._fold()
        w_q = self.weight_fake_quant(weight)
        y = self.conv._conv_forward(x, w_q, bias)
        if self.relu:
            y = F.relu(y)
        return self.activation_post_process(y)

    def to_quantized(self):
        """The integer inference layer with the folded weight baked in
        (lucid/nn/intrinsic/qat/modules.py:796-833)."""
        import lucid_b200.nn.quantized as nnq
        from lucid_b200.quantization import quantize

        with torch.no_grad():
            weight, bias = self._fold()
            weight, bias = weight.detach().contiguous(), bias.detach().to(torch.float32)
            wfq = self.weight_fake_quant
            wfq(weight)  # observe the folded weight
            w_scale, w_zp = wfq.calculate_qparams()
            ch_axis = wfq.ch_axis if wfq.ch_axis is not None else 0
            dev = weight.device
            codes = quantize(weight, w_scale.to(dev), w_zp.to(dev), wfq.qdtype, ch_axis=wfq.ch_axis)
            conv = self.conv
            padding = conv.padding if not isinstance(conv.padding, str) else 0
            plain = (nnq.Conv1d, nnq.Conv2d, nnq.Conv3d)[self._RANK - 1]
            fused = (nnq.ConvReLU1d, nnq.ConvReLU2d, nnq.ConvReLU3d)[self._RANK - 1]
            if self._RANK == 1:
                codes = codes.unsqueeze(2)  # the 1-D layer keeps its kernel as 1 x k
            q = (fused if self.relu else plain)(conv.in_channels, conv.out_channels, conv.kernel_size, conv.stride, padding, conv.dilation,
                    conv.groups, bias=True)
            q.weight_int8, q.weight_scale, q.weight_zero_point = codes, w_scale.to(dev), w_zp.to(dev)
            q.weight_ch_axis = ch_axis
            q.padding_str = conv.padding if isinstance(conv.padding, str) else None
            q.padding_mode = conv.padding_mode
            q.bias = bias
            a_scale, a_zp = self.activation_post_process.calculate_qparams()
            q.scale, q.zero_point = a_scale.to(dev), a_zp.to(dev)
            q.out_qdtype = self.activation_post_process.qdtype
        return q


class ConvBn1d(_ConvBnNd):
    _RANK = 1


class ConvBn2d(_ConvBnNd):
    _RANK = 2


class ConvBn3d(_ConvBnNd):
    _RANK = 3


class _WithReLU:
    """The fused-ReLU forms take the reference's ``(conv, bn, relu=True, qconfig=None)``
    (lucid/nn/intrinsic/qat/modules.py:553-561)."""

    _RELU = True

    def __init__(self, conv, bn, relu: bool = True, qconfig=None) -> None:
        super().__init__(conv, bn, qconfig=qconfig)
        self.relu = bool(relu)


class ConvBnReLU1d(_WithReLU, ConvBn1d):
    pass


class ConvBnReLU2d(_WithReLU, ConvBn2d):
    pass


class ConvBnReLU3d(_WithReLU, ConvBn3d):
    pass


def convbnrelu2d_to_quantized(mod: _ConvBnNd):
    """Rank-generic bake of a trained ``ConvBn*`` module into its inference layer
    (lucid/nn/intrinsic/qat/modules.py:796-837)."""
    return mod.to_quantized()
