"""The reference's literal forward goldens (flashlight/fl/test/nn/ModuleTest.cpp: EmbeddingFwd,
LinearFwd, LogSoftmaxFwd, RNNFwd / LSTMFwd / GRUFwd) against the CUDA path through the C ABI.
The vectors are parsed from the flashlight checkout at test time and never copied, so these
tests run where both a GPU and the checkout are present; elsewhere the CUDA path is compared
with the oracle, which tests/test_oracle_pins.py pins on the same vectors."""
import pytest
import torch

from oracle import flref as R
from tests.test_oracle_pins import _grab, _literals, _module_tests

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fx():
    from flashlight_b200 import functions
    return functions


def test_embedding_linear_logsoftmax_goldens(fx, reference_root):
    src = _module_tests(reference_root)
    table, ids, want = _literals(src, "EmbeddingFwd")[:3]
    got = fx.embedding(table.float().cuda(), ids.to(torch.int32).cuda())
    assert torch.equal(got.cpu().double().reshape(want.shape), want)
    w, x, want, bias, want_b = _literals(src, "LinearFwd")[:5]
    from flashlight_b200 import _lib as L
    for mode in (L.MATH_STRICT_F32, L.MATH_F32X3):
        y = fx.linear(x.float().cuda(), w.float().cuda(), None, math_mode=mode)
        assert (y.cpu().double() - want).abs().max() < 1e-4
        yb = fx.linear(x.float().cuda(), w.float().cuda(), bias.float().cuda(), math_mode=mode)
        assert (yb.cpu().double() - want_b).abs().max() < 1e-4
    x, want0, want1 = _literals(src, "LogSoftmaxFwd")[:3]
    assert (fx.log_softmax(x.float().cuda()).cpu().double() - want0).abs().max() < 1e-4
    got1 = fx.log_softmax(x.t().contiguous().float().cuda()).cpu().double().t()
    assert (got1 - want1).abs().max() < 1e-4


@pytest.mark.parametrize("test,mode", [("RNNFwd", R.RNN_RELU), ("LSTMFwd", R.RNN_LSTM),
                                       ("GRUFwd", R.RNN_GRU)])
def test_rnn_forward_goldens(reference_root, test, mode):
    from flashlight_b200 import _lib as L
    from flashlight_b200.extension import B200AutogradExtension
    c = _grab(_module_tests(reference_root), test)
    w = (torch.arange(1, c["n"] + 1, dtype=torch.float64) * c["sw"]).float().cuda()
    x = (torch.arange(1, c["I"] * c["B"] * c["T"] + 1, dtype=torch.float64) * c["sin"]).reshape(
        c["T"], c["B"], c["I"]).float().cuda()
    ext = B200AutogradExtension(math_mode=L.MATH_STRICT_F32)
    y, _, _ = ext.rnn(x, None, None, w, c["H"], c["L"], mode, False, 0.0, None)
    got = y.cpu().double().numpy().reshape(-1)
    assert abs(got - c["vals"]).max() < 1e-4
