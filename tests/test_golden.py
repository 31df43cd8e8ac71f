"""Committed golden vectors (tests/golden/*.npz, written by tests/golden/make_golden.py).
CPU: the oracle still reproduces them.  GPU: the CUDA path matches them through the C ABI."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import flref as R
from tests.parity import STRICT_TOL, assert_close

GOLD = Path(__file__).resolve().parent / "golden"


def load(name):
    z = np.load(GOLD / f"{name}.npz")
    return {k: torch.from_numpy(np.asarray(z[k])) for k in z.files}


def test_oracle_reproduces_the_fixtures():
    c = load("conv")
    args = tuple(int(v) for v in c["args"])
    assert_close(R.conv2d(c["x"], c["w"], c["b"], *args), c["y"], 1e-12, "conv")
    assert_close(R.conv2d_backward_data(c["gy"], c["x"].shape, c["w"], *args), c["gx"], 1e-12, "gx")
    p = load("pool")
    geo = tuple(int(v) for v in p["geo"])
    assert_close(R.pool2d_backward(p["gy"], p["x"], *geo, R.POOL_MAX), p["gx"], 1e-12, "pool gx")
    b = load("batchnorm")
    gx, gg, gb = R.batchnorm_backward(b["gy"], b["x"], b["g"], [2], 1e-5)
    assert_close(gx, b["gx"], 1e-12, "bn gx")
    r = load("rnn_lstm")
    I, H, L_, B, T = (int(v) for v in r["dims"])
    y, _, _ = R.rnn(r["x"], r["hx"], r["cx"], r["w"], H, L_, R.RNN_LSTM, True)
    assert_close(y, r["y"], 1e-12, "rnn y")
    lo = load("loss")
    loss, denom = R.categorical_cross_entropy(R.log_softmax(lo["x"]), lo["t"], R.REDUCE_MEAN, -1)
    assert_close(loss, lo["loss"], 1e-12, "loss")
    assert denom == int(lo["denom"])


@pytest.mark.gpu
def test_cuda_path_matches_the_fixtures():
    from flashlight_b200 import _lib as L
    from flashlight_b200 import functions as F
    from flashlight_b200.extension import AutogradPayload, B200AutogradExtension, RNNGradData
    ext = B200AutogradExtension(math_mode=L.MATH_STRICT_F32)
    f = lambda t: t.float().cuda()

    c = load("conv")
    args = tuple(int(v) for v in c["args"])
    assert_close(ext.conv2d(f(c["x"]), f(c["w"]), f(c["b"]), *args), c["y"], STRICT_TOL, "conv y")
    assert_close(ext.conv2dBackwardData(f(c["gy"]), f(c["x"]), f(c["w"]), *args), c["gx"],
                 STRICT_TOL, "conv gx")
    gw, gb = ext.conv2dBackwardFilterBias(f(c["gy"]), f(c["x"]), f(c["w"]), f(c["b"]), *args)
    assert_close(gw, c["gw"], STRICT_TOL, "conv gw")
    assert_close(gb, c["gb"], STRICT_TOL, "conv gb")

    p = load("pool")
    geo = tuple(int(v) for v in p["geo"])
    payload = AutogradPayload()
    y = ext.pool2d(f(p["x"]), *geo, L.POOL_MAX, payload)
    assert_close(y, p["y"], 1e-6, "pool y")
    assert torch.equal(payload.data.argmax.cpu(), p["argmax"])
    assert_close(ext.pool2dBackward(f(p["gy"]), f(p["x"]), y, *geo, L.POOL_MAX, payload), p["gx"],
                 1e-6, "pool gx")
    ya = ext.pool2d(f(p["x"]), *geo, L.POOL_AVG_EXCLUDE_PAD, None)
    assert_close(ya, p["y_avg"], 1e-5, "avg pool y")
    assert_close(ext.pool2dBackward(f(p["gy"]), f(p["x"]), ya, *geo, L.POOL_AVG_EXCLUDE_PAD, None),
                 p["gx_avg"], 1e-5, "avg pool gx")

    b = load("batchnorm")
    rm, rv = torch.zeros(6).cuda(), torch.ones(6).cuda()
    y, sm, sv = ext.batchnorm(f(b["x"]), f(b["g"]), f(b["b"]), rm, rv, [2], True, 0.1, 1e-5)
    assert_close(y, b["y"], STRICT_TOL, "bn y")
    assert_close(sm, b["mean"], STRICT_TOL, "bn mean")
    assert_close(sv, b["invstd"], STRICT_TOL, "bn invstd")
    assert_close(rm, b["rm"], STRICT_TOL, "bn running mean")
    assert_close(rv, b["rv"], STRICT_TOL, "bn running var")
    gx, gg, gb = ext.batchnormBackward(f(b["gy"]), sm, sv, f(b["x"]), f(b["g"]), [2], True, 1e-5)
    assert_close(gx, b["gx"], STRICT_TOL, "bn gx")
    assert_close(gg, b["gg"], STRICT_TOL, "bn dgamma")
    assert_close(gb, b["gb"], STRICT_TOL, "bn dbeta")

    r = load("rnn_lstm")
    I, H, L_, B, T = (int(v) for v in r["dims"])
    payload = AutogradPayload()
    y, hy, cy = ext.rnn(f(r["x"]), f(r["hx"]), f(r["cx"]), f(r["w"]), H, L_, L.RNN_LSTM, True, 0.0,
                        payload)
    assert_close(y, r["y"], STRICT_TOL, "rnn y")
    assert_close(hy, r["hy"], STRICT_TOL, "rnn hy")
    assert_close(cy, r["cy"], STRICT_TOL, "rnn cy")
    dx, dhx, dcx, dw = ext.rnnBackward(f(r["x"]), f(r["hx"]), f(r["cx"]), f(r["w"]),
                                       RNNGradData(f(r["gy"]), None, None), y, L_, H, L.RNN_LSTM,
                                       True, 0.0, payload)
    assert_close(dx, r["dx"], STRICT_TOL, "rnn dx")
    assert_close(dhx, r["dhx"], STRICT_TOL, "rnn dhx")
    assert_close(dcx, r["dcx"], STRICT_TOL, "rnn dcx")
    assert_close(dw, r["dw"], STRICT_TOL, "rnn dw")

    lo = load("loss")
    lp = F.log_softmax(f(lo["x"]))
    assert_close(lp, lo["lp"], STRICT_TOL, "logSoftmax")
    loss, state = F.categorical_cross_entropy(lp, lo["t"].cuda(), L.REDUCE_MEAN, -1)
    assert_close(loss, lo["loss"], STRICT_TOL, "CE loss")
    gx = F.log_softmax_cross_entropy_backward(lp, torch.ones(1).cuda(), state)
    assert_close(gx, lo["gx"], STRICT_TOL, "fused gradient")
