"""Generate ``reference_vectors.npz`` by EXECUTING the reference's own Python
sources for the quantization path.

The reference package cannot be imported as a whole (it needs its compiled
Apple-only engine and a newer Python), but the files on the hot path are pure
Python composites over a small tensor-op surface.  This script loads those
files unmodified from a checkout of the reference (``--reference DIR``) into a
synthetic ``lucid`` package whose tensor type is a thin NumPy float32 stand-in,
runs them on seeded inputs, and stores inputs and outputs.  The stand-in
supplies only the primitive ops (IEEE divide, ties-to-even round, compare-based
clip, truncating cast, min/max); the op ORDER, scalar promotion and module
logic all come from the reference's code.

Run where the reference checkout exists:

    python tests/golden/make_golden.py --reference <path-to-reference>

The produced ``.npz`` is committed; tests only read the ``.npz``.
"""

from __future__ import annotations

import __future__ as _fut
import argparse
import os
import sys
import types

import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------
# NumPy tensor stand-in
# --------------------------------------------------------------------------
class dtype:  # noqa: N801 - mirrors ``lucid.dtype``
    def __init__(self, name, np_dtype):
        self.name = name
        self.np = np.dtype(np_dtype)

    def __repr__(self):
        return f"lucid.{self.name}"


float32 = dtype("float32", np.float32)
float64 = dtype("float64", np.float64)
int8 = dtype("int8", np.int8)
int16 = dtype("int16", np.int16)
int32 = dtype("int32", np.int32)
int64 = dtype("int64", np.int64)
_BY_NP = {d.np: d for d in (float32, float64, int8, int16, int32, int64)}


class device:  # noqa: N801
    def __init__(self, kind="cpu"):
        self.type = kind

    def __eq__(self, other):
        return isinstance(other, device) and other.type == self.type

    def __ne__(self, other):
        return not self == other

    def __hash__(self):
        return hash(self.type)


_CPU = device("cpu")


def _cast_truncating(a, np_dtype):
    """``static_cast<int>(float)`` of an (already integral) value."""
    return a.astype(np_dtype)


class Tensor:
    def __init__(self, a, requires_grad=False):
        self.a = np.asarray(a)
        self.requires_grad = requires_grad

    # -- metadata
    @property
    def shape(self):
        return tuple(self.a.shape)

    @property
    def dtype(self):
        return _BY_NP[self.a.dtype]

    @property
    def device(self):
        return _CPU

    @property
    def ndim(self):
        return self.a.ndim

    def numpy(self):
        return self.a

    def item(self):
        return self.a.item()

    def detach(self):
        return Tensor(self.a.copy())

    def to(self, what):
        if isinstance(what, dtype):
            return Tensor(_cast_truncating(self.a, what.np))
        return self

    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = tuple(shape[0])
        return Tensor(self.a.reshape(shape))

    def min(self):
        return Tensor(self.a.min())

    def max(self):
        return Tensor(self.a.max())

    def any(self):
        return Tensor(np.asarray(self.a.any()))

    def all(self):
        return Tensor(np.asarray(self.a.all()))

    def tolist(self):
        return self.a.tolist()

    # -- scalar promotion: a Python number becomes a 0-d constant of the
    #    tensor's dtype when the tensor is floating, else float32 / int64.
    def _other(self, o):
        if isinstance(o, Tensor):
            return o.a
        if self.a.dtype.kind == "f":
            return np.asarray(o, dtype=self.a.dtype)
        if isinstance(o, float):
            return np.asarray(o, dtype=F32)
        return np.asarray(o, dtype=self.a.dtype)

    def _bin(self, o, fn, swap=False):
        b = self._other(o)
        a = self.a
        if a.dtype.kind != "f" and b.dtype.kind == "f":
            a = a.astype(b.dtype)
        r = fn(b, a) if swap else fn(a, b)
        return Tensor(r)

    def __truediv__(self, o):
        return self._bin(o, np.divide)

    def __rtruediv__(self, o):
        return self._bin(o, np.divide, swap=True)

    def __add__(self, o):
        return self._bin(o, np.add)

    __radd__ = __add__

    def __sub__(self, o):
        return self._bin(o, np.subtract)

    def __rsub__(self, o):
        return self._bin(o, np.subtract, swap=True)

    def __mul__(self, o):
        return self._bin(o, np.multiply)

    __rmul__ = __mul__

    def __ge__(self, o):
        return Tensor(self.a >= self._other(o))

    def __le__(self, o):
        return Tensor(self.a <= self._other(o))

    def __eq__(self, o):  # noqa: D105
        return Tensor(self.a == self._other(o))

    __hash__ = object.__hash__


def _t(x):
    return x.a if isinstance(x, Tensor) else x


def tensor(data, dtype=None, requires_grad=False, device=None):  # noqa: A002
    a = np.asarray(_t(data))
    if dtype is not None:
        a = a.astype(dtype.np)
    elif a.dtype.kind == "f":
        a = a.astype(F32)
    return Tensor(a, requires_grad)


def zeros(shape, dtype=float32, device=None):  # noqa: A002
    return Tensor(np.zeros(shape, dtype=dtype.np))


def ones(shape, dtype=float32, device=None):  # noqa: A002
    return Tensor(np.ones(shape, dtype=dtype.np))


def zeros_like(t):
    return Tensor(np.zeros_like(t.a))


def full_like(t, v):
    return Tensor(np.full_like(t.a, v))


def minimum(a, b):
    return Tensor(np.minimum(_t(a), _t(b)))


def maximum(a, b):
    return Tensor(np.maximum(_t(a), _t(b)))


def _abs(t):
    return Tensor(np.abs(t.a))


def _round(t):
    return Tensor(np.rint(t.a))  # ties to even


def clip(t, lo, hi):
    a = t.a
    lo = np.asarray(lo, dtype=a.dtype)
    hi = np.asarray(hi, dtype=a.dtype)
    return Tensor(np.where(a < lo, lo, np.where(a > hi, hi, a)).astype(a.dtype))


def moveaxis(t, src, dst):
    return Tensor(np.moveaxis(t.a, src, dst))


def amin(t, dim):
    return Tensor(t.a.min(axis=dim))


def amax(t, dim):
    return Tensor(t.a.max(axis=dim))


def isinf(t):
    return Tensor(np.isinf(t.a))


def cat(tensors, dim=0):
    return Tensor(np.concatenate([t.a for t in tensors], axis=dim))


def where(c, a, b):
    return Tensor(np.where(_t(c), _t(a), _t(b)))


def arange(n, device=None):
    return Tensor(np.arange(n, dtype=np.int64))


def scatter_add(out, dim, index, src):
    """Adds ``src[i]`` into ``out[index[i]]``, sources visited in order."""
    assert dim == 0
    r = out.a.copy()
    for i, d in enumerate(index.a.tolist()):
        r[d] = r[d] + src.a[i]
    return Tensor(r)


def histc(t, bins=100, min=0, max=0):  # noqa: A002
    """Stand-in for the engine's histc, which is C++ and cannot be executed here: a
    restatement of lucid/_C/ops/composite/Stats.cpp:47-91 over the counting loop of
    lucid/_C/backend/cpu/CpuBackend.h:13276-13318, written element by element."""
    lo, hi = float(min), float(max)
    flat = t.a.astype(np.float64).ravel()
    if lo == hi:
        lo, hi = float(flat.min()), float(flat.max())
        if lo == hi:
            hi = lo + 1.0
    step = (hi - lo) / float(bins)
    counts = np.zeros(bins, dtype=np.float64)
    for v in flat.tolist():
        if v < lo or v > hi:
            continue
        b = int((v - lo) / step)
        if b >= bins:
            b = bins - 1
        counts[b] += 1.0
    return Tensor(counts.astype(t.a.dtype))


# -- autograd stand-in (forward only)
class FunctionCtx:
    def save_for_backward(self, *ts):
        self.saved_tensors = ts


class Function:
    @classmethod
    def apply(cls, *args, **kwargs):
        ctx = FunctionCtx()
        out = cls.forward(ctx, *args, **kwargs)
        out._ctx = ctx
        return out


# -- nn stand-in
class Module:
    def __init__(self):
        object.__setattr__(self, "_buffers", {})

    def register_buffer(self, name, value):
        self._buffers[name] = value
        object.__setattr__(self, name, value)

    def named_buffers(self, recurse=True):
        return list(self._buffers.items())

    def parameters(self):
        return iter(())

    def __call__(self, *a, **k):
        return self.forward(*a, **k)

    def _load_from_state_dict(self, *a, **k):
        pass


class FloatLinear(Module):
    """Minimal float ``nn.Linear`` carrier for ``from_float``."""

    def __init__(self, weight, bias):
        super().__init__()
        self.weight = Tensor(weight)
        self.bias = None if bias is None else Tensor(bias)
        self.out_features, self.in_features = weight.shape


def f_linear(x, w, b=None):
    y = x.a @ w.a.T
    if b is not None:
        y = y + b.a
    return Tensor(y.astype(F32))


def f_relu(x):
    return Tensor(np.maximum(x.a, F32(0)))


# --------------------------------------------------------------------------
# Loader: execute reference files unmodified inside a synthetic package
# --------------------------------------------------------------------------
def _mod(name, is_pkg=False):
    m = types.ModuleType(name)
    if is_pkg:
        m.__path__ = []
    sys.modules[name] = m
    return m


def _load(name, path):
    with open(path, "r", encoding="utf-8") as fh:
        src = fh.read()
    m = _mod(name)
    m.__file__ = path
    # Deferred annotation evaluation (the reference targets a Python where
    # that is the default).
    code = compile(src, path, "exec", flags=_fut.annotations.compiler_flag, dont_inherit=True)
    exec(code, m.__dict__)
    return m


def install(reference_root):
    import typing

    if not hasattr(typing, "override"):
        typing.override = lambda f: f
    lucid = _mod("lucid", True)
    for k, v in dict(
        Tensor=Tensor, tensor=tensor, zeros=zeros, ones=ones, zeros_like=zeros_like,
        full_like=full_like, minimum=minimum, maximum=maximum, abs=_abs, round=_round,
        clip=clip, moveaxis=moveaxis, amin=amin, amax=amax, isinf=isinf, dtype=dtype,
        where=where, arange=arange, scatter_add=scatter_add, histc=histc, cat=cat,
        device=device, float32=float32, float64=float64, int8=int8, int16=int16,
        int32=int32, int64=int64,
    ).items():
        setattr(lucid, k, v)
    _mod("lucid._tensor", True)
    _mod("lucid._tensor.tensor").Tensor = Tensor
    ag = _mod("lucid.autograd")
    ag.Function, ag.FunctionCtx = Function, FunctionCtx
    nn = _mod("lucid.nn", True)
    nn.Module = Module
    lucid.nn = nn
    fn = _mod("lucid.nn.functional")
    fn.linear, fn.relu = f_linear, f_relu
    nn.functional = fn
    _mod("lucid.quantization", True)
    _mod("lucid.nn.quantized", True)
    _mod("lucid.nn.quantized.dynamic", True)
    q = os.path.join(reference_root, "lucid", "quantization")
    nq = os.path.join(reference_root, "lucid", "nn", "quantized")
    mods = {}
    mods["qscheme"] = _load("lucid.quantization._qscheme", os.path.join(q, "_qscheme.py"))
    mods["qparams"] = _load("lucid.quantization._qparams", os.path.join(q, "_qparams.py"))
    mods["functional"] = _load("lucid.quantization._functional", os.path.join(q, "_functional.py"))
    mods["observer"] = _load("lucid.quantization.observer", os.path.join(q, "observer.py"))
    mods["fake_quantize"] = _load("lucid.quantization._fake_quantize", os.path.join(q, "_fake_quantize.py"))
    mods["utils"] = _load("lucid.nn.quantized._utils", os.path.join(nq, "_utils.py"))
    mods["linear"] = _load("lucid.nn.quantized.linear", os.path.join(nq, "linear.py"))
    mods["dyn_linear"] = _load("lucid.nn.quantized.dynamic.linear",
                               os.path.join(nq, "dynamic", "linear.py"))
    mods["functional_module"] = _load("lucid.nn.quantized.functional_module",
                                      os.path.join(nq, "functional_module.py"))
    return mods


# --------------------------------------------------------------------------
# Cases
# --------------------------------------------------------------------------
def generate(reference_root):
    m = install(reference_root)
    S, P, Fn, O = m["qscheme"], m["qparams"], m["functional"], m["observer"]
    out = {}

    def T(a):
        return tensor(np.asarray(a, dtype=F32))

    # -- quantize / dequantize / fake_quantize, per tensor
    cases = [
        ("pt_s8", 0, (3, 16), 0.05, 0.0, S.qint8),
        ("pt_s8_b", 1, (4, 8), 0.05, 0.0, S.qint8),
        ("pt_s8_c", 2, (3, 16), 0.037, 0.0, S.qint8),
        ("pt_u8", 3, (5, 7), 0.02, 128.0, S.quint8),
        ("pt_sat", 5, (2, 10), 0.05, 0.0, S.qint8),
        ("pt_big", 6, (128, 192), None, 0.0, None),
    ]
    narrow = S.QDtype("qint8_narrow", 8, True, -127, 127, "int8")
    for name, seed, shape, s, z, qd in cases:
        x = np.random.default_rng(seed).standard_normal(shape).astype(F32)
        if name == "pt_sat":
            x = (x * F32(3.0)).astype(F32)
        if s is None:
            # absmax / 127 evaluated by the reference's tensor ops
            s_t = _abs(T(x)).max() / 127
            qd = narrow
            s_val = s_t
            out[f"{name}_scale"] = s_t.a
        else:
            s_val = s
            out[f"{name}_scale"] = np.asarray(s, dtype=np.float64)
        out[f"{name}_x"] = x
        out[f"{name}_zp"] = np.asarray(z, dtype=np.float64)
        out[f"{name}_qrange"] = np.asarray([qd.quant_min, qd.quant_max], dtype=np.int64)
        q = Fn.quantize(T(x), s_val, z, qd)
        out[f"{name}_q"] = q.a
        out[f"{name}_dq"] = Fn.dequantize(q, s_val, z).a
        fq = Fn.fake_quantize(T(x), s_val, z, qd.quant_min, qd.quant_max)
        out[f"{name}_fq"] = fq.a
        out[f"{name}_mask"] = fq._ctx.saved_tensors[0].a

    # -- exact ties: x / s lands on k + 0.5
    ks = np.arange(-300, 300, dtype=F32)
    x = ((ks + F32(0.5)) * F32(0.5)).astype(F32)
    out["ties_x"] = x
    out["ties_q"] = Fn.quantize(T(x), 0.5, 0.0, S.qint8).a
    out["ties_q_u8"] = Fn.quantize(T(x), 0.5, 3.0, S.quint8).a

    # -- per-channel (axis 0 and axis 1)
    x = np.random.default_rng(4).standard_normal((4, 8)).astype(F32)
    sc = np.array([0.02, 0.03, 0.05, 0.017], dtype=F32)
    zc = np.zeros(4, dtype=F32)
    out["pc_x"], out["pc_scale"], out["pc_zp"] = x, sc, zc
    q = Fn.quantize(T(x), T(sc), T(zc), S.qint8, ch_axis=0)
    out["pc_q"] = q.a
    out["pc_dq"] = Fn.dequantize(q, T(sc), T(zc), ch_axis=0).a
    out["pc_fq"] = Fn.fake_quantize(T(x), T(sc), T(zc), -128, 127, ch_axis=0).a
    x1 = np.random.default_rng(7).standard_normal((6, 4)).astype(F32)
    z1 = np.array([3, 120, 128, 250], dtype=F32)
    out["pc1_x"], out["pc1_zp"] = x1, z1
    q1 = Fn.quantize(T(x1), T(sc), T(z1), S.quint8, ch_axis=1)
    out["pc1_q"] = q1.a
    out["pc1_dq"] = Fn.dequantize(q1, T(sc), T(z1), ch_axis=1).a

    # -- calculate_qparams over a grid of ranges
    rng = np.random.default_rng(8)
    mins = np.concatenate([[-1.0, -2.0, -2.5, 0.0, 3.0, -0.8, 0.5, -7.0],
                           rng.standard_normal(24) * 3]).astype(F32)
    maxs = np.concatenate([[3.0, 6.0, 2.0, 0.0, 3.0, 0.5, 4.0, -1.0],
                           mins[8:] + np.abs(rng.standard_normal(24)) * 5]).astype(F32)
    out["qp_min"], out["qp_max"] = mins, maxs
    for sname, scheme in (("aff", S.per_tensor_affine), ("sym", S.per_tensor_symmetric)):
        for dname, qd in (("s8", S.qint8), ("u8", S.quint8), ("s4", S.qint4)):
            # vector form (per-channel path) and scalar form must agree
            s_v, z_v = P.calculate_qparams(T(mins), T(maxs), scheme, qd)
            out[f"qp_{sname}_{dname}_scale"] = s_v.a
            out[f"qp_{sname}_{dname}_zp"] = z_v.a
            s_s = [P.calculate_qparams(float(a), float(b), scheme, qd)[0].a
                   for a, b in zip(mins, maxs)]
            out[f"qp_{sname}_{dname}_scale_scalar"] = np.asarray(s_s, dtype=F32)

    # -- observers
    obs = O.MinMaxObserver()
    xa = np.random.default_rng(9).standard_normal((8, 33)).astype(F32)
    xb = (np.random.default_rng(10).standard_normal((3, 5)) * 2).astype(F32)
    obs(T(xa))
    obs(T(xb))
    out["obs_xa"], out["obs_xb"] = xa, xb
    out["obs_min"], out["obs_max"] = obs.min_val.a, obs.max_val.a
    s_o, z_o = obs.calculate_qparams()
    out["obs_scale"], out["obs_zp"] = s_o.a, z_o.a
    pobs = O.PerChannelMinMaxObserver(ch_axis=0)
    pobs(T(xa))
    out["pobs_min"], out["pobs_max"] = pobs.min_val.a, pobs.max_val.a
    s_p, z_p = pobs.calculate_qparams()
    out["pobs_scale"], out["pobs_zp"] = s_p.a, z_p.a

    # -- moving-average observers (three batches each)
    batches = [(np.random.default_rng(30 + i).standard_normal((6, 40)) * (1.0 + 0.7 * i)).astype(F32)
               for i in range(3)]
    ma = O.MovingAverageMinMaxObserver(averaging_constant=0.05)
    mac = O.MovingAveragePerChannelMinMaxObserver(ch_axis=0, averaging_constant=0.05)
    for i, xb_ in enumerate(batches):
        out[f"ma_x{i}"] = xb_
        ma(T(xb_))
        mac(T(xb_))
        out[f"ma_min{i}"], out[f"ma_max{i}"] = ma.min_val.a, ma.max_val.a
        out[f"mac_min{i}"], out[f"mac_max{i}"] = mac.min_val.a, mac.max_val.a
    s_m, z_m = ma.calculate_qparams()
    out["ma_scale"], out["ma_zp"] = s_m.a, z_m.a
    s_m, z_m = mac.calculate_qparams()
    out["mac_scale"], out["mac_zp"] = s_m.a, z_m.a

    # -- histogram observer: range growth (re-binning), a batch inside the range, a constant
    #    first batch (the empty-range rule of histc), rectified data, a symmetric signed grid
    def run_hist(tag, xs, bins, **kw):
        h = O.HistogramObserver(bins=bins, **kw)
        for i, xb_ in enumerate(xs):
            out[f"{tag}_x{i}"] = xb_
            h(T(xb_))
            out[f"{tag}_hist{i}"] = h.histogram.a
            out[f"{tag}_range{i}"] = np.asarray([h.min_val.a, h.max_val.a], dtype=np.float64)
        out[f"{tag}_clip"] = np.asarray(h._search_clip_range(), dtype=np.float64)
        s_h, z_h = h.calculate_qparams()
        out[f"{tag}_scale"], out[f"{tag}_zp"] = s_h.a, z_h.a

    g = np.random.default_rng(40)
    grow = [g.standard_normal(3000).astype(F32), (g.standard_normal(2500) * 2.5).astype(F32),
            (g.standard_normal(2000) * 0.5).astype(F32), (g.standard_normal((7, 300)) * 4 + 1).astype(F32)]
    run_hist("hg", grow, 2048)
    run_hist("hs", grow[:3], 128, qscheme=S.per_tensor_symmetric, qdtype=S.qint8)
    const = [np.full(37, 0.75, dtype=F32), g.standard_normal(1500).astype(F32)]
    run_hist("hc", const, 256)
    relu = [np.maximum(g.standard_normal(4000), 0).astype(F32),
            np.maximum(g.standard_normal(4000) * 1.5, 0).astype(F32)]
    run_hist("hr", relu, 2048)
    # heavy tails: the clip search has something to cut
    tails = [np.concatenate([g.standard_normal(20000), [40.0, -35.0]]).astype(F32)]
    run_hist("ht", tails, 2048)

    # -- FakeQuantize module: moving-average activations over three batches, a frozen observer,
    #    fake-quant switched off; per-channel symmetric weights
    FQ = m["fake_quantize"].FakeQuantize
    fq = FQ(observer=O.MovingAverageMinMaxObserver, averaging_constant=0.1)
    g = np.random.default_rng(60)
    for i in range(3):
        xb_ = (g.standard_normal((5, 24)) * (1 + i)).astype(F32)
        out[f"fqm_x{i}"] = xb_
        out[f"fqm_y{i}"] = fq(T(xb_)).a
        out[f"fqm_qp{i}"] = np.asarray([fq.scale.a, fq.zero_point.a], dtype=F32)
    fq.disable_observer()
    wide = (g.standard_normal((5, 24)) * 9).astype(F32)
    out["fqm_xwide"], out["fqm_ywide"] = wide, fq(T(wide)).a
    out["fqm_qpwide"] = np.asarray([fq.scale.a, fq.zero_point.a], dtype=F32)
    wfq = FQ(observer=O.PerChannelMinMaxObserver, ch_axis=0, qscheme=S.per_channel_symmetric, qdtype=S.qint8)
    wt = (g.standard_normal((6, 20)) * 0.05).astype(F32)
    out["fqm_w"], out["fqm_wy"] = wt, wfq(T(wt)).a
    out["fqm_wscale"], out["fqm_wzp"] = wfq.scale.a, wfq.zero_point.a

    # -- QFunctional: every merge on one grid; operands are fake-quantized tensors on their own
    #    grids (what the producing layers hand over) and one raw float pair
    g = np.random.default_rng(50)
    xa_ = (g.standard_normal((6, 50)) * 1.3).astype(F32)
    ya_ = (g.standard_normal((6, 50)) * 0.8).astype(F32)
    out["qf_xraw"], out["qf_yraw"] = xa_, ya_
    xq = Fn.quantize(T(xa_), 0.04, 120.0, S.quint8)
    yq = Fn.quantize(T(ya_), 0.025, 0.0, S.qint8)
    out["qf_xq"], out["qf_yq"] = xq.a, yq.a
    xf, yf_ = Fn.dequantize(xq, 0.04, 120.0), Fn.dequantize(yq, 0.025, 0.0)
    for tag_, (sc_, zp_, qd_) in {"u8": (0.05, 110.0, S.quint8), "s8": (0.03, -5.0, S.qint8)}.items():
        qf = m["functional_module"].QFunctional(tensor(sc_), tensor(zp_), qd_)
        out[f"qf_{tag_}_grid"] = np.asarray([sc_, zp_, qd_.quant_min, qd_.quant_max], dtype=np.float64)
        out[f"qf_{tag_}_add"] = qf.add(xf, yf_).a
        out[f"qf_{tag_}_mul"] = qf.mul(xf, yf_).a
        out[f"qf_{tag_}_add_relu"] = qf.add_relu(xf, yf_).a
        out[f"qf_{tag_}_add_scalar"] = qf.add_scalar(xf, 0.75).a
        out[f"qf_{tag_}_mul_scalar"] = qf.mul_scalar(xf, -1.5).a
        out[f"qf_{tag_}_cat"] = qf.cat([xf, yf_], dim=1).a
        out[f"qf_{tag_}_add_raw"] = qf.add(T(xa_), T(ya_)).a

    # -- dynamic Linear: from_float + forward (float GEMM = NumPy f32 matmul)
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((32, 64)) * 0.02).astype(F32)
    b = (rng.standard_normal(32) * 0.01).astype(F32)
    xin = rng.standard_normal((16, 64)).astype(F32)
    dl = m["dyn_linear"].Linear.from_float(FloatLinear(w, b))
    out["dyn_w"], out["dyn_b"], out["dyn_x"] = w, b, xin
    out["dyn_wq"] = dl.weight_int8.a
    out["dyn_ws"] = dl.weight_scale.a
    out["dyn_wz"] = dl.weight_zero_point.a
    out["dyn_y"] = dl(T(xin)).a
    xs, xz = P.calculate_qparams(T(xin).min(), T(xin).max(), S.per_tensor_affine, S.quint8)
    out["dyn_xs"], out["dyn_xz"] = xs.a, xz.a
    out["dyn_xq"] = Fn.quantize(T(xin), xs, xz, S.quint8).a

    # -- static quantized Linear.forward with installed buffers
    ql = m["linear"].Linear(64, 32)
    ql.register_buffer("weight_int8", dl.weight_int8)
    ql.register_buffer("weight_scale", dl.weight_scale)
    ql.register_buffer("weight_zero_point", dl.weight_zero_point)
    ql.register_buffer("bias", tensor(b))
    yf = f_linear(T(xin), T(w), T(b)).a
    os_, oz_ = P.calculate_qparams(float(yf.min()), float(yf.max()), S.per_tensor_affine, S.quint8)
    ql.register_buffer("scale", os_)
    ql.register_buffer("zero_point", oz_)
    out["ql_os"], out["ql_oz"] = os_.a, oz_.a
    out["ql_y"] = ql(T(xin)).a
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                  "reference_vectors.npz"))
    a = ap.parse_args()
    data = generate(a.reference)
    np.savez_compressed(a.out, **data)
    print(f"wrote {a.out}: {len(data)} arrays, "
          f"{os.path.getsize(a.out) / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
