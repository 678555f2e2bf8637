"""Quantized embedding tables (lucid/nn/quantized/sparse.py:28-340): per-row int8 codes,
looked up and decoded in one kernel (the reference decodes the whole table per call)."""

from __future__ import annotations

import torch

from ... import _lib
from ...quantization import PerChannelMinMaxObserver, per_channel_symmetric, qint8, quantize
from ._utils import quantize_weight

_MODES = {"sum": 0, "mean": 1, "max": 2}


def _quantize_table(mod):
    if getattr(mod, "qconfig", None) is None:
        obs = PerChannelMinMaxObserver(ch_axis=0, qscheme=per_channel_symmetric, qdtype=qint8)
        w = mod.weight.detach()
        obs(w)
        scale, zero_point = obs.calculate_qparams()
        return quantize(w, scale, zero_point, qint8, ch_axis=0), scale, zero_point
    codes, scale, zero_point, _ = quantize_weight(mod)
    return codes, scale, zero_point


def _index_tensor(x, what):
    _lib.require_cuda(x, what)
    if x.dtype not in (torch.int32, torch.int64):
        raise _lib.DtypeMismatch(f"{what} must be int32 or int64, got {x.dtype}")
    return x.contiguous()


class _QuantizedTable(torch.nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx=None) -> None:
        super().__init__()
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.padding_idx = padding_idx
        self.register_buffer("weight_int8", torch.zeros((num_embeddings, embedding_dim), dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(num_embeddings))
        self.register_buffer("weight_zero_point", torch.zeros(num_embeddings))

    def _lookup(self, idx, offsets, include_last, mode, out):
        w = self.weight_int8
        dev = w.device
        n_bags = 0 if offsets is None else offsets.numel()
        status = _lib.status_word(dev) if offsets is None else None
        with torch.cuda.device(dev):
            _lib.check(_lib.load().lq_embedding_s8(
                _lib.ptr(w), _lib.ptr(self.weight_scale), _lib.ptr(self.weight_zero_point),
                self.num_embeddings, self.embedding_dim, _lib.ptr(idx), 64 if idx.dtype == torch.int64 else 32,
                idx.numel(), _lib.ptr(offsets), n_bags, int(include_last), mode,
                -1 if self.padding_idx is None else int(self.padding_idx), _lib.ptr(out),
                _lib.code_of(out.dtype), _lib.ptr(status), _lib.stream_ptr(dev)))
        return out

    def _install(self, codes, scale, zero_point):
        self.weight_int8, self.weight_scale, self.weight_zero_point = codes, scale, zero_point
        return self


class Embedding(_QuantizedTable):
    """``out[..., :] = dequantize(table)[x[...]]``; rows equal to ``padding_idx`` are zeros.
    An index outside the table leaves a zero row and sets the device status word
    (``lucid_b200._lib.check_device_status``); nothing is synchronised in ``forward``."""

    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx=None,
                 out_dtype: torch.dtype = torch.float32) -> None:
        super().__init__(num_embeddings, embedding_dim, padding_idx)
        self.out_dtype = out_dtype

    def forward(self, x):
        idx = _index_tensor(x, "indices")
        out = torch.empty(tuple(idx.shape) + (self.embedding_dim,), dtype=self.out_dtype, device=idx.device)
        return self._lookup(idx, None, False, 0, out)

    def extra_repr(self) -> str:
        return f"{self.num_embeddings}, {self.embedding_dim}, padding_idx={self.padding_idx}, qdtype=qint8"

    @classmethod
    def from_float(cls, mod) -> "Embedding":
        q = cls(mod.num_embeddings, mod.embedding_dim, padding_idx=mod.padding_idx)
        return q._install(*_quantize_table(mod))


class EmbeddingBag(_QuantizedTable):
    """Pooled lookup: 2-D ``x`` (one bag per row) or 1-D ``x`` with ``offsets``."""

    def __init__(self, num_embeddings: int, embedding_dim: int, mode: str = "mean", padding_idx=None,
                 include_last_offset: bool = False) -> None:
        super().__init__(num_embeddings, embedding_dim, padding_idx)
        if mode not in _MODES:
            raise ValueError(f"embedding_bag: mode must be one of {sorted(_MODES)}, got {mode!r}")
        self.mode = mode
        self.include_last_offset = include_last_offset

    def forward(self, x, offsets=None):
        idx = _index_tensor(x, "indices")
        include_last = False
        if idx.dim() == 2:
            rows, length = idx.shape
            offsets = torch.arange(0, rows * length, length, device=idx.device, dtype=idx.dtype)
            idx = idx.reshape(-1)
        else:
            if offsets is None:
                raise ValueError("embedding_bag: offsets required for 1-D input")
            offsets = _index_tensor(offsets, "offsets").to(idx.dtype)
            include_last = self.include_last_offset
        out = torch.empty((offsets.numel(), self.embedding_dim), dtype=torch.float32, device=idx.device)
        return self._lookup(idx, offsets, include_last, _MODES[self.mode], out)

    def extra_repr(self) -> str:
        return f"{self.num_embeddings}, {self.embedding_dim}, mode={self.mode}, qdtype=qint8"

    @classmethod
    def from_float(cls, mod) -> "EmbeddingBag":
        q = cls(mod.num_embeddings, mod.embedding_dim, mode=getattr(mod, "mode", "mean"),
                padding_idx=getattr(mod, "padding_idx", None),
                include_last_offset=getattr(mod, "include_last_offset", False))
        return q._install(*_quantize_table(mod))
