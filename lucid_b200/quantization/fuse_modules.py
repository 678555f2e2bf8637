"""``fuse_modules`` / ``fuse_modules_qat``: collapse Conv/BN/ReLU (or Linear/ReLU) runs before
quantization (lucid/quantization/fuse_modules.py:62-186, 219-330).

Given groups of dotted module names, the first member of each run becomes the fused module and
the rest become ``Identity`` (the model's own ``forward`` still routes through them).  BatchNorm
is folded into the preceding convolution's weight at eval time; a trailing ReLU is absorbed into
an intrinsic container so that the activation observer sees the post-ReLU range -- and so that
``convert`` produces ONE integer kernel (convolution, bias, ReLU, requantisation) for the run.
Without the fold a model with BatchNorm cannot reach the integer convolution at all."""

from __future__ import annotations

import copy

import torch

_CONV_TYPES = (torch.nn.Conv1d, torch.nn.Conv2d, torch.nn.Conv3d)
_BN_TYPES = (torch.nn.BatchNorm1d, torch.nn.BatchNorm2d, torch.nn.BatchNorm3d)


def _rank(conv: torch.nn.Module) -> int:
    return conv.weight.dim() - 2


def _check_pair(who: str, conv: torch.nn.Module, bn: torch.nn.Module) -> None:
    """A convolution folds with the BatchNorm of its own rank only."""
    if not isinstance(conv, _CONV_TYPES) or not isinstance(bn, _BN_TYPES[_rank(conv) - 1]):
        raise TypeError(f"{who}: unsupported pair {type(conv).__name__}, {type(bn).__name__}")


def _get_module(root: torch.nn.Module, dotted: str) -> torch.nn.Module:
    mod = root
    for part in dotted.split("."):
        mod = getattr(mod, part)
    return mod


def _set_module(root: torch.nn.Module, dotted: str, value: torch.nn.Module) -> None:
    """Assign through ``_modules`` so that the child keeps its position (``Sequential`` order)."""
    parts = dotted.split(".")
    parent = root
    for part in parts[:-1]:
        parent = getattr(parent, part)
    if parts[-1] in parent._modules:
        parent._modules[parts[-1]] = value
    else:
        setattr(parent, parts[-1], value)


def fuse_conv_bn_eval(conv: torch.nn.Module, bn: torch.nn.Module) -> torch.nn.Module:
    """A copy of ``conv`` computing ``bn(conv(x))`` at eval time
    (lucid/nn/utils/fusion.py:100-135): ``W' = W * g / sqrt(var + eps)``,
    ``b' = (b - mean) * g / sqrt(var + eps) + beta``."""
    from ..nn.intrinsic.qat import fold_conv_bn

    _check_pair("fuse_conv_bn_eval", conv, bn)
    fused = copy.deepcopy(conv)
    with torch.no_grad():
        w, b = fold_conv_bn(conv.weight.detach(), None if conv.bias is None else conv.bias.detach(), bn)
    fused.weight = torch.nn.Parameter(w)
    fused.bias = torch.nn.Parameter(b)
    return fused


def _conv_relu(conv):
    import torch.ao.nn.intrinsic as nni

    return (nni.ConvReLU1d, nni.ConvReLU2d, nni.ConvReLU3d)[_rank(conv) - 1](conv, torch.nn.ReLU())


def _fuse_run(mods):
    import torch.ao.nn.intrinsic as nni

    ids = [torch.nn.Identity() for _ in range(len(mods) - 1)]
    first, rest = mods[0], list(mods[1:])
    if isinstance(first, _CONV_TYPES):
        conv = first
        if rest and isinstance(rest[0], _BN_TYPES):
            conv = fuse_conv_bn_eval(conv, rest.pop(0))
        if rest and isinstance(rest[0], torch.nn.ReLU):
            rest.pop(0)
            if not rest:
                return [_conv_relu(conv), *ids]
        elif not rest:
            return [conv, *ids]
    elif isinstance(first, torch.nn.Linear) and len(mods) == 2 and isinstance(mods[1], torch.nn.ReLU):
        return [nni.LinearReLU(first, torch.nn.ReLU()), *ids]
    raise ValueError(f"fuse_modules: unsupported fusion pattern {[type(m).__name__ for m in mods]}")


def fuse_modules(model: torch.nn.Module, modules_to_fuse, inplace: bool = False) -> torch.nn.Module:
    """Static-PTQ fusion, run on a model in eval mode before ``prepare``.  Supported runs:
    ``[Conv, BN]``, ``[Conv, BN, ReLU]``, ``[Conv, ReLU]``, ``[Linear, ReLU]``; anything else
    raises ``ValueError``."""
    model = model if inplace else copy.deepcopy(model)
    for group in modules_to_fuse:
        mods = [_get_module(model, name) for name in group]
        for name, repl in zip(group, _fuse_run(mods)):
            _set_module(model, name, repl)
    return model


def _fuse_run_qat(mods, qconfig):
    import torch.ao.nn.intrinsic as nni

    from ..nn.intrinsic import qat as nniqat

    ids = [torch.nn.Identity() for _ in range(len(mods) - 1)]
    first, rest = mods[0], list(mods[1:])
    if isinstance(first, _CONV_TYPES):
        if rest and isinstance(rest[0], _BN_TYPES):
            bn = rest.pop(0)
            relu = bool(rest and isinstance(rest[0], torch.nn.ReLU))
            if len(rest) == (1 if relu else 0):
                plain = (nniqat.ConvBn1d, nniqat.ConvBn2d, nniqat.ConvBn3d)[_rank(first) - 1]
                fused = (nniqat.ConvBnReLU1d, nniqat.ConvBnReLU2d, nniqat.ConvBnReLU3d)[_rank(first) - 1]
                return [(fused if relu else plain)(first, bn, qconfig=qconfig), *ids]
        elif len(rest) == 1 and isinstance(rest[0], torch.nn.ReLU):
            return [_conv_relu(first), *ids]
        elif not rest:
            return [first, *ids]
    elif isinstance(first, torch.nn.Linear) and len(mods) == 2 and isinstance(mods[1], torch.nn.ReLU):
        return [nni.LinearReLU(first, torch.nn.ReLU()), *ids]
    raise ValueError(f"fuse_modules_qat: unsupported pattern {[type(m).__name__ for m in mods]}")


def fuse_modules_qat(model: torch.nn.Module, modules_to_fuse, qconfig, inplace: bool = False) -> torch.nn.Module:
    """QAT fusion, run before ``prepare_qat``: ``[Conv, BN]`` / ``[Conv, BN, ReLU]`` runs become
    trainable ``ConvBn{1,2,3}d`` / ``ConvBnReLU{1,2,3}d`` modules that fold BatchNorm per forward (the
    qconfig is needed here: they fake-quantize from their first forward)."""
    model = model if inplace else copy.deepcopy(model)
    for group in modules_to_fuse:
        mods = [_get_module(model, name) for name in group]
        for name, repl in zip(group, _fuse_run_qat(mods, qconfig)):
            _set_module(model, name, repl)
    return model
