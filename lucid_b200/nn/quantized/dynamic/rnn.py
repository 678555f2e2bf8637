"""Dynamically (weight-only) quantized ``LSTM`` (lucid/nn/quantized/dynamic/rnn.py:27-111).

As in the reference, the recurrent weight matrices are stored as per-row symmetric int8
(``weight_ih_l*_int8`` / ``weight_hh_l*_int8`` with ``*_scale``), biases stay float, and the
forward runs the FLOAT recurrence on the dequantized weights: activations are not quantized
inside the cell, so the result is the float LSTM's on the decoded weights.  The reference decodes
every weight on every call; here the decoded copy is cached until the codes change.  Per time
step the cell is one float GEMM against the recurrent weight (library GEMM) and one fused
gate kernel (``lq_lstm_cell_f32``); the input projection of all time steps is one GEMM.
Packed sequences go through the library's LSTM routine on the same decoded weights."""

from __future__ import annotations

import torch

from .... import _lib
from ....quantization import PerChannelMinMaxObserver, QDtype, dequantize, per_channel_symmetric, qint8, quantize


class LSTM(torch.nn.Module):
    def __init__(self, input_size, hidden_size: int | None = None, num_layers: int = 1, bias: bool = True,
                 batch_first: bool = False, bidirectional: bool = False) -> None:
        super().__init__()
        if isinstance(input_size, torch.nn.LSTM):
            # the reference's constructor takes the float layer as a configuration "shell"
            # (lucid/nn/quantized/dynamic/rnn.py:54-64); the buffers are filled by from_float
            shell = input_size
            if getattr(shell, "proj_size", 0):
                raise NotImplementedError("dynamic LSTM: proj_size is not supported")
            input_size, hidden_size, num_layers = shell.input_size, shell.hidden_size, shell.num_layers
            bias, batch_first, bidirectional = shell.bias, shell.batch_first, shell.bidirectional
        elif hidden_size is None:
            raise TypeError("dynamic LSTM: hidden_size is required")
        self.input_size, self.hidden_size, self.num_layers = input_size, hidden_size, num_layers
        self.bias, self.batch_first, self.bidirectional = bias, batch_first, bidirectional
        self._weight_names: list[str] = []
        self._bias_names: list[str] = []
        dirs = 2 if bidirectional else 1
        for layer in range(num_layers):
            for d in range(dirs):
                sfx = f"_l{layer}" + ("_reverse" if d == 1 else "")
                in_sz = input_size if layer == 0 else hidden_size * dirs
                for name, cols in (("weight_ih" + sfx, in_sz), ("weight_hh" + sfx, hidden_size)):
                    self.register_buffer(name + "_int8", torch.zeros((4 * hidden_size, cols), dtype=torch.int8))
                    self.register_buffer(name + "_scale", torch.ones(4 * hidden_size))
                    self._weight_names.append(name)
                if bias:
                    for name in ("bias_ih" + sfx, "bias_hh" + sfx):
                        self.register_buffer(name, torch.zeros(4 * hidden_size))
                        self._bias_names.append(name)
        self._decoded: dict = {}

    # -- weights ---------------------------------------------------------------------
    def _weight(self, name: str) -> torch.Tensor:
        """Float weight decoded from the int8 buffer (``(q - 0) * scale`` per row), cached until
        the buffer is replaced or modified."""
        codes, scale = getattr(self, name + "_int8"), getattr(self, name + "_scale")
        key = (codes.data_ptr(), codes._version, scale.data_ptr(), scale._version)
        hit = self._decoded.get(name)
        if hit is None or hit[0] != key:
            w = dequantize(codes, scale, torch.zeros_like(scale), ch_axis=0)
            hit = (key, w, w.t().contiguous())
            self._decoded[name] = hit
        return hit

    # -- forward -----------------------------------------------------------------------
    def _direction(self, x: torch.Tensor, h0: torch.Tensor, c0: torch.Tensor, sfx: str, reverse: bool):
        """One layer, one direction: x (T, B, I) -> (T, B, H), h_T, c_T."""
        t_len, batch, _ = x.shape
        hid = self.hidden_size
        _, w_ih, _ = self._weight("weight_ih" + sfx)
        _, _, w_hh_t = self._weight("weight_hh" + sfx)
        xp = torch.matmul(x.reshape(t_len * batch, -1), w_ih.t())
        if self.bias:
            xp = xp + (getattr(self, "bias_ih" + sfx) + getattr(self, "bias_hh" + sfx))
        xp = xp.reshape(t_len, batch, 4 * hid)
        out = torch.empty((t_len, batch, hid), dtype=torch.float32, device=x.device)
        gates = torch.empty((batch, 4 * hid), dtype=torch.float32, device=x.device)
        h, c = h0.contiguous(), c0.contiguous().clone()
        lib, st = _lib.load(), _lib.stream_ptr(x.device)
        steps = range(t_len - 1, -1, -1) if reverse else range(t_len)
        with torch.cuda.device(x.device):
            for t in steps:
                torch.addmm(xp[t], h, w_hh_t, out=gates)
                _lib.check(lib.lq_lstm_cell_f32(_lib.ptr(gates), 4 * hid, _lib.ptr(c), _lib.ptr(out[t]), hid,
                                                _lib.ptr(c), batch, hid, st))
                h = out[t]
        return out, h, c

    def forward(self, x, hx=None):
        with _lib.ieee_float32():
            return self._forward(x, hx)

    def _forward(self, x, hx):
        if isinstance(x, torch.nn.utils.rnn.PackedSequence):
            return self._forward_packed(x, hx)
        _lib.require_cuda(x, "input")
        if x.dim() not in (2, 3):
            raise _lib.ShapeMismatch(f"LSTM input must be 2-D or 3-D, got {tuple(x.shape)}")
        unbatched = x.dim() == 2
        seq = x.unsqueeze(1) if unbatched else (x.transpose(0, 1) if self.batch_first else x)
        seq = seq.to(torch.float32).contiguous()
        t_len, batch, feat = seq.shape
        if feat != self.input_size:
            raise _lib.ShapeMismatch(f"LSTM input has {feat} features, expected {self.input_size}")
        dirs = 2 if self.bidirectional else 1
        if hx is None:
            h0 = torch.zeros((self.num_layers * dirs, batch, self.hidden_size), device=x.device)
            c0 = torch.zeros_like(h0)
        else:
            h0, c0 = (t.unsqueeze(1) if unbatched else t for t in hx)
            h0, c0 = h0.to(torch.float32), c0.to(torch.float32)
        h_n, c_n = [], []
        layer_in = seq
        for layer in range(self.num_layers):
            outs = []
            for d in range(dirs):
                sfx = f"_l{layer}" + ("_reverse" if d == 1 else "")
                o, h, c = self._direction(layer_in, h0[layer * dirs + d], c0[layer * dirs + d], sfx, d == 1)
                outs.append(o)
                h_n.append(h)
                c_n.append(c)
            layer_in = outs[0] if dirs == 1 else torch.cat(outs, dim=2)
        out = layer_in
        h_n, c_n = torch.stack(h_n), torch.stack(c_n)
        if unbatched:
            return out.squeeze(1), (h_n.squeeze(1), c_n.squeeze(1))
        return (out.transpose(0, 1) if self.batch_first else out), (h_n, c_n)

    def _forward_packed(self, packed, hx):
        """Packed input: the library's LSTM routine on the decoded weights."""
        params, dirs = [], 2 if self.bidirectional else 1
        for layer in range(self.num_layers):
            for d in range(dirs):
                sfx = f"_l{layer}" + ("_reverse" if d == 1 else "")
                params += [self._weight("weight_ih" + sfx)[1], self._weight("weight_hh" + sfx)[1]]
                if self.bias:
                    params += [getattr(self, "bias_ih" + sfx), getattr(self, "bias_hh" + sfx)]
        batch = int(packed.batch_sizes[0])
        dev = packed.data.device
        if hx is None:
            z = torch.zeros((self.num_layers * dirs, batch, self.hidden_size), device=dev)
            hx = (z, z.clone())
        elif packed.sorted_indices is not None:
            hx = tuple(t.index_select(1, packed.sorted_indices) for t in hx)
        out, h, c = torch._VF.lstm(packed.data.to(torch.float32), packed.batch_sizes, hx, params, self.bias,
                                   self.num_layers, 0.0, False, self.bidirectional)
        if packed.unsorted_indices is not None:
            h, c = h.index_select(1, packed.unsorted_indices), c.index_select(1, packed.unsorted_indices)
        return torch.nn.utils.rnn.PackedSequence(out, packed.batch_sizes, packed.sorted_indices,
                                                 packed.unsorted_indices), (h, c)

    # -- construction --------------------------------------------------------------------
    @classmethod
    def from_float(cls, mod: torch.nn.Module, dtype: QDtype = qint8) -> "LSTM":
        """Quantize a float ``nn.LSTM``'s recurrent weights per row (symmetric)."""
        if not isinstance(mod, torch.nn.LSTM):
            raise TypeError(f"dynamic LSTM.from_float expects an nn.LSTM, got {type(mod).__name__}")
        if getattr(mod, "proj_size", 0):
            raise NotImplementedError("dynamic LSTM: proj_size is not supported")
        q = cls(mod.input_size, mod.hidden_size, mod.num_layers, mod.bias, mod.batch_first, mod.bidirectional)
        for name, param in mod.named_parameters():
            p = param.detach()
            if name.startswith("weight"):
                obs = PerChannelMinMaxObserver(ch_axis=0, qscheme=per_channel_symmetric, qdtype=dtype)
                obs(p)
                scale, zero_point = obs.calculate_qparams()
                setattr(q, name + "_int8", quantize(p, scale, zero_point, dtype, ch_axis=0))
                setattr(q, name + "_scale", scale)
            else:
                setattr(q, name, p.to(torch.float32))
        return q

    def extra_repr(self) -> str:
        return (f"{self.input_size}, {self.hidden_size}, num_layers={self.num_layers}, "
                f"bidirectional={self.bidirectional}, dynamic=True")
