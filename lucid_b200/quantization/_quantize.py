"""Eager-mode workflows: ``prepare`` -> calibrate -> ``convert`` and ``quantize_dynamic``
(lucid/quantization/_quantize.py:204-419, 429-554, 684-699).

The float model is a ``torch.nn`` model on a CUDA device; the converted model holds the
quantized modules of ``lucid_b200.nn.quantized``, whose buffers carry the reference's
``state_dict`` names (``weight_int8`` / ``weight_scale`` / ``weight_zero_point`` / ``bias`` /
``scale`` / ``zero_point``), so a checkpoint written by either side loads into the other.
"""

from __future__ import annotations

import copy
import warnings

import torch

from ._qscheme import QDtype, qint8
from .qconfig import (
    QConfig,
    QConfigMapping,
    get_default_qat_qconfig_mapping,
    get_default_qconfig_mapping,
)


class QuantStub(torch.nn.Module):
    """Marks where float activations enter the quantized region
    (lucid/nn/quantized/modules.py:29-123): an identity under static PTQ, where a forward hook
    feeds the observer; a ``FakeQuantize`` attached as ``activation_post_process`` is applied."""

    def __init__(self, qconfig=None) -> None:
        super().__init__()
        if qconfig is not None:
            self.qconfig = qconfig

    def forward(self, x):
        from ._fake_quantize import FakeQuantize

        app = getattr(self, "activation_post_process", None)
        if isinstance(app, FakeQuantize) and torch.is_floating_point(x):
            return app(x)
        return x


class DeQuantStub(torch.nn.Module):
    """Marks where activations leave the quantized region (identity;
    lucid/nn/quantized/modules.py:126-183)."""

    def __init__(self, qconfig=None) -> None:
        super().__init__()
        if qconfig is not None:
            self.qconfig = qconfig

    def forward(self, x):
        return x


class QuantWrapper(torch.nn.Module):
    """``quant -> module -> dequant`` around a model that has no stubs of its own
    (lucid/nn/quantized/modules.py:351-424)."""

    def __init__(self, module: torch.nn.Module) -> None:
        super().__init__()
        self.quant = QuantStub()
        self.module = module
        self.dequant = DeQuantStub()

    def forward(self, x):
        return self.dequant(self.module(self.quant(x)))


def _intrinsic():
    try:
        import torch.ao.nn.intrinsic as nni

        return nni
    except Exception:  # pragma: no cover - torch always ships it
        return None


_ACTIVATIONS = (torch.nn.Sigmoid, torch.nn.Hardswish, torch.nn.Hardsigmoid, torch.nn.Tanh, torch.nn.ELU,
                torch.nn.LeakyReLU)


_CONV_TRANSPOSE = (torch.nn.ConvTranspose1d, torch.nn.ConvTranspose2d, torch.nn.ConvTranspose3d)


def _observed_types() -> tuple:
    from ..nn.quantized.functional_module import FloatFunctional

    nni = _intrinsic()
    fused = (nni.LinearReLU, nni.ConvReLU1d, nni.ConvReLU2d, nni.ConvReLU3d) if nni is not None else ()
    return (torch.nn.Linear, torch.nn.Conv1d, torch.nn.Conv2d, torch.nn.Conv3d, QuantStub, FloatFunctional) + \
        _ACTIVATIONS + _CONV_TRANSPOSE + fused


def _quant_mapping() -> dict:
    import lucid_b200.nn.quantized as nnq

    m = {
        torch.nn.Linear: nnq.Linear.from_float,
        torch.nn.Conv1d: nnq.Conv1d.from_float,
        torch.nn.Conv2d: nnq.Conv2d.from_float,
        torch.nn.Conv3d: nnq.Conv3d.from_float,
        QuantStub: nnq.Quantize.from_float,
        DeQuantStub: nnq.DeQuantize.from_float,
        torch.nn.ReLU: nnq.ReLU.from_float,
        nnq.FloatFunctional: nnq.QFunctional.from_float,
        torch.nn.ConvTranspose1d: nnq.ConvTranspose1d.from_float,
        torch.nn.ConvTranspose2d: nnq.ConvTranspose2d.from_float,
        torch.nn.ConvTranspose3d: nnq.ConvTranspose3d.from_float,
        torch.nn.Sigmoid: nnq.Sigmoid.from_float,
        torch.nn.Hardswish: nnq.Hardswish.from_float,
        torch.nn.Hardsigmoid: nnq.Hardsigmoid.from_float,
        torch.nn.Tanh: nnq.Tanh.from_float,
        torch.nn.ELU: nnq.ELU.from_float,
        torch.nn.LeakyReLU: nnq.LeakyReLU.from_float,
        torch.nn.Embedding: nnq.Embedding.from_float,
        torch.nn.EmbeddingBag: nnq.EmbeddingBag.from_float,
    }
    nni = _intrinsic()
    if nni is not None:
        m[nni.LinearReLU] = nnq.LinearReLU.from_float
        m[nni.ConvReLU1d] = nnq.ConvReLU1d.from_float
        m[nni.ConvReLU2d] = nnq.ConvReLU2d.from_float
        m[nni.ConvReLU3d] = nnq.ConvReLU3d.from_float
    from ..nn import qat as nnqat

    m[nnqat.Linear] = nnq.Linear.from_float
    m[nnqat.LinearReLU] = nnq.LinearReLU.from_float
    m[nnqat.Conv1d] = nnq.Conv1d.from_float
    m[nnqat.Conv2d] = nnq.Conv2d.from_float
    m[nnqat.Conv3d] = nnq.Conv3d.from_float
    m[nnqat.ConvReLU1d] = nnq.ConvReLU1d.from_float
    m[nnqat.ConvReLU2d] = nnq.ConvReLU2d.from_float
    m[nnqat.ConvReLU3d] = nnq.ConvReLU3d.from_float
    m[nnqat.Embedding] = nnq.Embedding.from_float
    from ..nn.intrinsic import qat as nniqat

    for cls in (nniqat.ConvBn1d, nniqat.ConvBn2d, nniqat.ConvBn3d,
                nniqat.ConvBnReLU1d, nniqat.ConvBnReLU2d, nniqat.ConvBnReLU3d):
        m[cls] = lambda mod: mod.to_quantized()
    from .. import backends

    if backends.quantized.use_mlx():  # the Linear family on the group-wise weight-only kernel
        m[torch.nn.Linear] = _mlx_linear_builder(False)
        if nni is not None:
            m[nni.LinearReLU] = _mlx_linear_builder(True)
    return m


def _mlx_weight_bits(mod) -> int:
    """Weight bit-width (4 / 8) of the group-wise route, read from the module's qconfig
    (lucid/quantization/_quantize.py:116-124)."""
    qcfg = getattr(mod, "qconfig", None)
    if qcfg is not None and hasattr(qcfg, "weight"):
        bits = getattr(getattr(qcfg.weight(), "qdtype", None), "bits", None)
        if isinstance(bits, int) and bits in (4, 8):
            return bits
    return 8


def _mlx_group_size(in_features: int):
    """Largest preferred group size (64, 128, 32) dividing ``in_features``, or None
    (lucid/quantization/_quantize.py:127-140)."""
    for gs in (64, 128, 32):
        if in_features % gs == 0:
            return gs
    return None


def _mlx_linear_builder(relu: bool):
    """``convert`` builder of the group-wise route (lucid/quantization/_quantize.py:143-165):
    weight-only codes, float activations; a layer no group size divides falls back to the
    calibrated layer."""
    import lucid_b200.nn.quantized as nnq

    fallback = nnq.LinearReLU.from_float if relu else nnq.Linear.from_float

    def build(child):
        inner = child[0] if relu else child
        gs = _mlx_group_size(inner.in_features)
        if gs is None:
            return fallback(child)
        return nnq.QuantizedLinearMLX.from_float(inner, bits=_mlx_weight_bits(child), group_size=gs, relu=relu)

    return build


def _mlx_dynamic_builder():
    """``quantize_dynamic`` builder of the group-wise route (lucid/quantization/_quantize.py:168-179)."""
    import lucid_b200.nn.quantized as nnq

    def build(child, dtype):
        gs = _mlx_group_size(child.in_features)
        if gs is None or dtype.bits not in (4, 8):
            return nnq.dynamic.Linear.from_float(child, dtype)
        return nnq.QuantizedLinearMLX.from_float(child, bits=dtype.bits, group_size=gs, relu=False)

    return build


def _make_observer_hook(obs):
    def hook(module, inputs, output):
        obs(output.detach().to(torch.float32).contiguous())
        return None

    return hook


def _as_mapping(qconfig, default) -> QConfigMapping:
    """A bare ``QConfig`` is the global tier of a mapping, ``None`` the default mapping
    (lucid/quantization/_quantize.py:195-201)."""
    if qconfig is None:
        return default()
    if isinstance(qconfig, QConfig):
        return QConfigMapping().set_global(qconfig)
    return qconfig


def prepare(model: torch.nn.Module, qconfig: QConfig | QConfigMapping | None = None, inplace: bool = False):
    """Attach an activation observer (forward hook) to every quantizable module the mapping
    gives a qconfig; nothing numeric changes.  Fused containers are observed as a unit, not
    their children (an excluded container keeps its children in float too)."""
    from ..nn.quantized.functional_module import FloatFunctional

    qmap = _as_mapping(qconfig, get_default_qconfig_mapping)
    model = model if inplace else copy.deepcopy(model)
    model.eval()
    observed = _observed_types()
    nni = _intrinsic()
    fused = (nni.LinearReLU, nni.ConvReLU1d, nni.ConvReLU2d, nni.ConvReLU3d) if nni is not None else ()
    inside_fused = set()
    n_matched = 0
    for name, mod in model.named_modules():
        if any(name.startswith(p + ".") for p in inside_fused):
            continue
        if not isinstance(mod, observed):
            continue
        if isinstance(mod, fused):
            inside_fused.add(name)
        qcfg = qmap.get_qconfig(type(mod), name)
        if qcfg is None:
            continue
        mod.qconfig = qcfg
        obs = qcfg.activation()
        mod.activation_post_process = obs
        if not isinstance(mod, FloatFunctional):  # a functional feeds its observer itself
            mod._lq_hook = mod.register_forward_hook(_make_observer_hook(obs))
        n_matched += 1
    if n_matched == 0:
        warnings.warn("prepare(): the QConfigMapping matched no quantizable modules -- convert() will "
                      "leave this model unchanged.", stacklevel=2)
    return model


def _convert_recursive(module, mapping, always) -> None:
    for name, child in list(module.named_children()):
        build = mapping.get(type(child))
        convertible = build is not None and (
            isinstance(child, always) or hasattr(child, "activation_post_process"))
        if convertible:
            hook = getattr(child, "_lq_hook", None)
            if hook is not None:
                hook.remove()
            # assign through _modules to keep the child's position (Sequential order)
            module._modules[name] = build(child)
        else:
            _convert_recursive(child, mapping, always)


def convert(model: torch.nn.Module, inplace: bool = False):
    """Swap every calibrated float module for its quantized counterpart."""
    model = model if inplace else copy.deepcopy(model)
    model.eval()
    mapping = _quant_mapping()
    # tables need no calibration (lucid/quantization/_quantize.py:416)
    always = (DeQuantStub, torch.nn.ReLU, torch.nn.Embedding, torch.nn.EmbeddingBag)
    build = mapping.get(type(model))
    if build is not None and hasattr(model, "activation_post_process"):
        return build(model)
    _convert_recursive(model, mapping, always)
    return model


def prepare_qat(model: torch.nn.Module, qconfig: QConfig | QConfigMapping | None = None, inplace: bool = False):
    """Swap every float ``Linear`` / ``Conv{1,2,3}d`` and every fused ``LinearReLU`` /
    ``ConvReLU{1,2,3}d`` container for its QAT form (weight and output each behind a
    ``FakeQuantize``) and leave the model in training mode
    (lucid/quantization/_quantize.py:557-572, 575-640)."""
    from ..nn import qat as nnqat

    qmap = _as_mapping(qconfig, get_default_qat_qconfig_mapping)
    model = model if inplace else copy.deepcopy(model)
    mapping = {torch.nn.Linear: nnqat.Linear.from_float, torch.nn.Conv1d: nnqat.Conv1d.from_float,
               torch.nn.Conv2d: nnqat.Conv2d.from_float, torch.nn.Conv3d: nnqat.Conv3d.from_float,
               torch.nn.Embedding: nnqat.Embedding.from_float}
    nni = _intrinsic()
    if nni is not None:
        mapping.update({nni.LinearReLU: nnqat.LinearReLU.from_float, nni.ConvReLU1d: nnqat.ConvReLU1d.from_float,
                        nni.ConvReLU2d: nnqat.ConvReLU2d.from_float, nni.ConvReLU3d: nnqat.ConvReLU3d.from_float})
    n_matched = 0

    from ..nn.intrinsic import qat as nniqat

    def swap(module, prefix):
        nonlocal n_matched
        for name, child in list(module.named_children()):
            full = f"{prefix}.{name}" if prefix else name
            if isinstance(child, nniqat._ConvBnNd):  # fused by fuse_modules_qat: already a QAT module
                n_matched += 1
                continue
            build = mapping.get(type(child))
            qcfg = qmap.get_qconfig(type(child), full)
            if build is not None and qcfg is not None:
                child.qconfig = qcfg
                module._modules[name] = build(child)
                n_matched += 1
            elif qcfg is not None and isinstance(child, QuantStub):
                # the entry grid is trained too: the stub fake-quantizes its input, and convert
                # bakes that grid into nn.quantized.Quantize (lucid/quantization/_quantize.py:677-679)
                child.qconfig = qcfg
                child.activation_post_process = qcfg.activation()
            else:
                swap(child, full)

    build = mapping.get(type(model))
    qcfg = qmap.get_qconfig(type(model), "")
    if build is not None and qcfg is not None:
        model.qconfig = qcfg
        model = build(model)
        n_matched += 1
    else:
        swap(model, "")
    if n_matched == 0:
        warnings.warn("prepare_qat(): the QConfigMapping matched no quantizable modules -- convert() will "
                      "leave this model unchanged.", stacklevel=2)
    model.train()
    return model


def _dynamic_mapping() -> dict:
    import lucid_b200.nn.quantized as nnq

    from .. import backends

    linear = _mlx_dynamic_builder() if backends.quantized.use_mlx() else nnq.dynamic.Linear.from_float
    return {torch.nn.Linear: linear,
            torch.nn.LSTM: nnq.dynamic.LSTM.from_float,
            torch.nn.Embedding: lambda mod, dtype: nnq.Embedding.from_float(mod),
            torch.nn.EmbeddingBag: lambda mod, dtype: nnq.EmbeddingBag.from_float(mod)}


def _swap_dynamic(module, mapping, types, dtype) -> None:
    for name, child in list(module.named_children()):
        build = mapping.get(type(child))
        if build is not None and type(child) in types:
            module._modules[name] = build(child, dtype)
        else:
            _swap_dynamic(child, mapping, types, dtype)


def quantize_dynamic(model: torch.nn.Module, qconfig_spec: set | None = None, dtype: QDtype = qint8,
                     inplace: bool = False):
    """int8 weights, activations quantized at run time; no calibration."""
    model = model if inplace else copy.deepcopy(model)
    model.eval()
    mapping = _dynamic_mapping()
    types = qconfig_spec if qconfig_spec is not None else set(mapping)
    if not any(type(m) in types for m in model.modules()):
        warnings.warn("quantize_dynamic(): no module of a targeted type "
                      f"({', '.join(sorted(t.__name__ for t in types))}) found -- the model is "
                      "returned unchanged.", stacklevel=2)
    build = mapping.get(type(model))
    if build is not None and type(model) in types:
        return build(model, dtype)
    _swap_dynamic(model, mapping, types, dtype)
    return model
