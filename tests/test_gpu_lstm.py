"""Weight-only quantized LSTM (lucid/nn/quantized/dynamic/rnn.py:27-111): int8 per-row weights,
float recurrence on the decoded weights.  The oracle is the float LSTM of the library run on the
decoded weights -- exactly what the reference's shell does -- compared within float tolerance
(the float GEMMs differ in summation order; the gate math goes through exp / tanh)."""

import numpy as np
import pytest
import torch

from oracle import lucid_oracle as O

pytestmark = pytest.mark.gpu

import lucid_b200.nn.quantized as nnq  # noqa: E402
import lucid_b200.quantization as Q  # noqa: E402
from gpu_util import host  # noqa: E402
from lucid_b200 import _lib  # noqa: E402


def _decoded_shell(lstm, qlstm):
    """A float nn.LSTM holding the weights decoded from the quantized module's buffers."""
    import copy

    shell = copy.deepcopy(lstm)
    with torch.no_grad():
        for name, p in shell.named_parameters():
            if name.startswith("weight"):
                p.copy_(getattr(qlstm, name + "_int8").float() * getattr(qlstm, name + "_scale")[:, None])
    return shell


@pytest.mark.parametrize("layers,bidir,batch_first", [(1, False, False), (2, True, True), (2, False, True)])
def test_dynamic_lstm_matches_float_lstm_on_decoded_weights(layers, bidir, batch_first):
    torch.manual_seed(layers * 7 + bidir)
    lstm = torch.nn.LSTM(48, 64, num_layers=layers, bidirectional=bidir, batch_first=batch_first).cuda()
    q = nnq.dynamic.LSTM.from_float(lstm)
    # weight codes / scales are the per-row symmetric encode of the reference
    w = host(lstm.weight_hh_l0.detach())
    wq, ws, _ = O.quantize_weight_per_channel(w)
    assert np.array_equal(host(q.weight_hh_l0_int8), wq) and np.array_equal(host(q.weight_hh_l0_scale), ws)
    assert "weight_ih_l0_int8" in q.state_dict() and "bias_hh_l0" in q.state_dict()
    assert not any(k.startswith("weight") and not (k.endswith("_int8") or k.endswith("_scale")) for k in q.state_dict())
    x = torch.randn(5, 9, 48, device="cuda") if batch_first else torch.randn(9, 5, 48, device="cuda")
    dirs = 2 if bidir else 1
    h0 = torch.randn(layers * dirs, 5, 64, device="cuda") * 0.1
    c0 = torch.randn(layers * dirs, 5, 64, device="cuda") * 0.1
    shell = _decoded_shell(lstm, q)
    with torch.no_grad(), _lib.ieee_float32():
        y_ref, (h_ref, c_ref) = shell(x, (h0, c0))
        y0_ref, _ = shell(x)
    y, (h, c) = q(x, (h0, c0))
    y0, _ = q(x)
    _lib.check_device_status(torch.device("cuda", torch.cuda.current_device()))
    assert y.shape == y_ref.shape and h.shape == h_ref.shape
    for got, ref in ((y, y_ref), (h, h_ref), (c, c_ref), (y0, y0_ref)):
        assert float((got - ref).abs().max()) < 2e-5


def test_dynamic_lstm_packed_unbatched_and_workflow():
    torch.manual_seed(3)
    model = torch.nn.Sequential(torch.nn.LSTM(32, 32, batch_first=True)).cuda()
    qmodel = Q.quantize_dynamic(model)
    q = qmodel[0]
    assert type(q) is nnq.dynamic.LSTM and q.weight_ih_l0_int8.dtype == torch.int8
    shell = _decoded_shell(model[0], q)
    x = torch.randn(7, 32, device="cuda")  # unbatched (T, I)
    with torch.no_grad(), _lib.ieee_float32():
        y_ref, _ = shell(x)
    y, _ = q(x)
    assert y.shape == (7, 32) and float((y - y_ref).abs().max()) < 2e-5
    seqs = torch.randn(3, 6, 32, device="cuda")
    packed = torch.nn.utils.rnn.pack_padded_sequence(seqs, [6, 4, 2], batch_first=True)
    with torch.no_grad(), _lib.ieee_float32():
        p_ref, (hp_ref, _) = shell(packed)
    p, (hp, _) = q(packed)
    assert float((p.data - p_ref.data).abs().max()) < 2e-5 and float((hp - hp_ref).abs().max()) < 2e-5
    # the decoded weight is cached until the codes change
    w1 = q._weight("weight_hh_l0")[1]
    assert q._weight("weight_hh_l0")[1] is w1
    q.weight_hh_l0_int8.zero_()
    assert q._weight("weight_hh_l0")[1] is not w1 and float(q._weight("weight_hh_l0")[1].abs().max()) == 0.0
    with pytest.raises(TypeError):
        nnq.dynamic.LSTM.from_float(torch.nn.GRU(8, 8))
