"""The reference's literal forward goldens (flashlight/fl/test/nn/ModuleTest.cpp: EmbeddingFwd,
LinearFwd, LogSoftmaxFwd, RNNFwd / LSTMFwd / GRUFwd) against the CUDA path through the C ABI.
The vectors come from tests/golden/reference_module_goldens.npz (written from a checkout of the
project by tests/golden/make_reference_goldens.py, and checked against a fresh parse by
tests/test_oracle_pins.py wherever a checkout is present), so these tests need no checkout."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import flref as R

pytestmark = pytest.mark.gpu
GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_module_goldens.npz")


def _literals(test, count):
    return [torch.from_numpy(GOLDEN[f"{test}_{i}"]) for i in range(count)]


def _grab(test):
    L_, H, I, B, T, n = (int(v) for v in GOLDEN[f"{test}_dims"])
    sin, sw = (float(v) for v in GOLDEN[f"{test}_scales"])
    return dict(L=L_, H=H, I=I, B=B, T=T, n=n, sin=sin, sw=sw, vals=GOLDEN[f"{test}_vals"])


@pytest.fixture(scope="module")
def fx():
    from flashlight_b200 import functions
    return functions


def test_embedding_linear_logsoftmax_goldens(fx):
    table, ids, want = _literals("EmbeddingFwd", 3)
    got = fx.embedding(table.float().cuda(), ids.to(torch.int32).cuda())
    assert torch.equal(got.cpu().double().reshape(want.shape), want)
    w, x, want, bias, want_b = _literals("LinearFwd", 5)
    from flashlight_b200 import _lib as L
    for mode in (L.MATH_STRICT_F32, L.MATH_F32X3):
        y = fx.linear(x.float().cuda(), w.float().cuda(), None, math_mode=mode)
        assert (y.cpu().double() - want).abs().max() < 1e-4
        yb = fx.linear(x.float().cuda(), w.float().cuda(), bias.float().cuda(), math_mode=mode)
        assert (yb.cpu().double() - want_b).abs().max() < 1e-4
    x, want0, want1 = _literals("LogSoftmaxFwd", 3)
    assert (fx.log_softmax(x.float().cuda()).cpu().double() - want0).abs().max() < 1e-4
    got1 = fx.log_softmax(x.t().contiguous().float().cuda()).cpu().double().t()
    assert (got1 - want1).abs().max() < 1e-4


@pytest.mark.parametrize("test,mode", [("RNNFwd", R.RNN_RELU), ("LSTMFwd", R.RNN_LSTM),
                                       ("GRUFwd", R.RNN_GRU)])
def test_rnn_forward_goldens(test, mode):
    from flashlight_b200 import _lib as L
    from flashlight_b200.extension import B200AutogradExtension
    c = _grab(test)
    w = (torch.arange(1, c["n"] + 1, dtype=torch.float64) * c["sw"]).float().cuda()
    x = (torch.arange(1, c["I"] * c["B"] * c["T"] + 1, dtype=torch.float64) * c["sin"]).reshape(
        c["T"], c["B"], c["I"]).float().cuda()
    ext = B200AutogradExtension(math_mode=L.MATH_STRICT_F32)
    y, _, _ = ext.rnn(x, None, None, w, c["H"], c["L"], mode, False, 0.0, None)
    got = y.cpu().double().numpy().reshape(-1)
    assert abs(got - c["vals"]).max() < 1e-4
