"""The persistent LSTM / GRU recurrence (one kernel for all time steps of a layer and direction, the
recurrent weights resident in shared memory, a grid-wide barrier per step) against the fp64
oracle and against the one-kernel-per-step path, and the bounded wait of its barrier."""
import ctypes as C
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from oracle import flref as R
from tests.parity import assert_close_scaled, randn

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def L():
    from flashlight_b200 import _lib
    if not _lib.lib.flb200_has_tensor_core_path():
        pytest.fail("tensor-core path unavailable on this device")
    return _lib


@pytest.mark.parametrize("dims", [
    (40, 256, 1, 8, 7, False),     # one CTA per cluster
    (48, 512, 2, 7, 9, True),      # clusters of 2, ragged batch, two layers, both directions
    (80, 1024, 1, 32, 12, True),   # the biLSTM workload's hidden size and batch: 128 CTAs
])
@pytest.mark.parametrize("with_state", [False, True])
def test_persistent_lstm_matches_oracle(L, dims, with_state):
    from flashlight_b200.extension import AutogradPayload, B200AutogradExtension, RNNGradData
    I, H, layers, B, T, bidir = dims
    dirs = 2 if bidir else 1
    ext = B200AutogradExtension(math_mode=L.MATH_TF32)
    n = R.rnn_num_params(I, H, layers, R.RNN_LSTM, bidir)
    w = randn(n, seed=40) * (0.5 / H ** 0.5)
    x = randn(T, B, I, seed=41)
    hx = randn(layers * dirs, B, H, seed=42) * 0.5 if with_state else None
    cx = randn(layers * dirs, B, H, seed=43) * 0.5 if with_state else None
    dev = lambda t: None if t is None else t.cuda()
    f64 = lambda t: None if t is None else t.double()
    payload = AutogradPayload()
    before = L.kernel_launches()
    y, hy, cy = ext.rnn(x.cuda(), dev(hx), dev(cx), w.cuda(), H, layers, R.RNN_LSTM, bidir, 0.0,
                        payload)
    torch.cuda.synchronize()
    launches = L.kernel_launches() - before
    # not one kernel per time step: a handful per (layer, direction)
    assert launches <= 8 * layers * dirs, f"{launches} launches for {T} steps"
    wy, why, wcy = R.rnn(x.double(), f64(hx), f64(cx), w.double(), H, layers, R.RNN_LSTM, bidir)
    assert_close_scaled(y, wy, 5e-3, "persistent lstm y")
    assert_close_scaled(hy, why, 5e-3, "persistent lstm hy")
    assert_close_scaled(cy, wcy, 5e-3, "persistent lstm cy")
    gy = randn(T, B, dirs * H, seed=44)
    dx, dhx, dcx, dw = ext.rnnBackward(x.cuda(), dev(hx), dev(cx), w.cuda(),
                                       RNNGradData(gy.cuda(), None, None), y, layers, H,
                                       R.RNN_LSTM, bidir, 0.0, payload)
    wdx, wdhx, wdcx, wdw = R.rnn_backward(x.double(), f64(hx), f64(cx), w.double(), H, layers,
                                          R.RNN_LSTM, bidir, gy.double(), None, None)
    assert_close_scaled(dx, wdx, 5e-3, "persistent lstm dx")
    assert_close_scaled(dw, wdw, 5e-3, "persistent lstm dw")
    if with_state:
        assert_close_scaled(dhx, wdhx, 5e-3, "persistent lstm dhx")
        assert_close_scaled(dcx, wdcx, 5e-3, "persistent lstm dcx")


@pytest.mark.parametrize("dims", [
    (40, 256, 1, 8, 7, False),     # forward: one CTA per cluster; backward: 6 CTAs, 43 units each
    (48, 512, 2, 7, 9, True),      # clusters of 2, ragged batch, two layers, both directions
    (80, 1024, 1, 32, 12, True),   # 128 CTAs forward, 96 backward
])
@pytest.mark.parametrize("with_state", [False, True])
@pytest.mark.parametrize("mode", [R.RNN_GRU, R.RNN_TANH, R.RNN_RELU])
def test_persistent_other_cells_match_oracle(L, dims, with_state, mode):
    """The GRU (three gates; q = U_n h + b_hn kept for the gradient; two gate-gradient tensors,
    the recurrent side's with dn * r) and the plain tanh / relu cells (one gate) on the same
    persistent kernels.  The relu cell is discontinuous: a TF32 rounding difference flips the
    mask of a few pre-activations near zero, hence its root-mean-square gradient bound."""
    from flashlight_b200.extension import AutogradPayload, B200AutogradExtension, RNNGradData
    I, H, layers, B, T, bidir = dims
    dirs = 2 if bidir else 1
    ext = B200AutogradExtension(math_mode=L.MATH_TF32)
    n = R.rnn_num_params(I, H, layers, mode, bidir)
    w = randn(n, seed=50) * (0.5 / H ** 0.5)
    x = randn(T, B, I, seed=51)
    hx = randn(layers * dirs, B, H, seed=52) * 0.5 if with_state else None
    dev = lambda t: None if t is None else t.cuda()
    f64 = lambda t: None if t is None else t.double()
    payload = AutogradPayload()
    before = L.kernel_launches()
    y, hy, _ = ext.rnn(x.cuda(), dev(hx), None, w.cuda(), H, layers, mode, bidir, 0.0, payload)
    torch.cuda.synchronize()
    launches = L.kernel_launches() - before
    assert launches <= 8 * layers * dirs, f"{launches} launches for {T} steps"
    wy, why, _ = R.rnn(x.double(), f64(hx), None, w.double(), H, layers, mode, bidir)
    assert_close_scaled(y, wy, 5e-3, "persistent cell y")
    assert_close_scaled(hy, why, 5e-3, "persistent cell hy")
    gy = randn(T, B, dirs * H, seed=54)
    ghy = randn(layers * dirs, B, H, seed=55) if with_state else None
    before = L.kernel_launches()
    dx, dhx, _, dw = ext.rnnBackward(x.cuda(), dev(hx), None, w.cuda(),
                                     RNNGradData(gy.cuda(), dev(ghy), None), y, layers, H,
                                     mode, bidir, 0.0, payload)
    torch.cuda.synchronize()
    launches = L.kernel_launches() - before
    assert launches <= 40 * layers * dirs, f"{launches} backward launches for {T} steps"
    wdx, wdhx, _, wdw = R.rnn_backward(x.double(), f64(hx), None, w.double(), H, layers,
                                       mode, bidir, gy.double(), f64(ghy), None)
    if mode == R.RNN_RELU:
        pairs = [(dx, wdx, "dx"), (dw, wdw, "dw")] + ([(dhx, wdhx, "dhx")] if with_state else [])
        for got, want, what in pairs:
            d = got.double().cpu() - want
            rms = float(d.pow(2).mean().sqrt() / want.pow(2).mean().sqrt())
            assert rms <= 0.15, f"persistent relu cell {what}: rms error {rms:.3e}"
        return
    assert_close_scaled(dx, wdx, 5e-3, "persistent cell dx")
    assert_close_scaled(dw, wdw, 5e-3, "persistent cell dw")
    if with_state:
        assert_close_scaled(dhx, wdhx, 5e-3, "persistent cell dhx")


def test_persistent_equals_per_step_path(L):
    """Same arithmetic, same order: the persistent kernel reproduces the per-step kernels bit
    for bit (the other path is selected in a child process, the switch is read once)."""
    code = r"""
import sys, torch
sys.path.insert(0, %r)
from flashlight_b200 import _lib as L
from flashlight_b200.extension import AutogradPayload, B200AutogradExtension
from oracle import flref as R
from tests.parity import randn
ext = B200AutogradExtension(math_mode=L.MATH_TF32)
I, H, layers, B, T = 48, 512, 2, 7, 9
w = randn(R.rnn_num_params(I, H, layers, R.RNN_LSTM, True), seed=40) * (0.5 / H ** 0.5)
x = randn(T, B, I, seed=41)
y, hy, cy = ext.rnn(x.cuda(), None, None, w.cuda(), H, layers, R.RNN_LSTM, True, 0.0, AutogradPayload())
torch.save([y.cpu(), hy.cpu(), cy.cpu()], sys.argv[1])
""" % str(ROOT)
    outs = []
    for flag in ("1", "0"):
        path = f"/tmp/flb200_rnn_persistent_{flag}.pt"
        env = dict(os.environ, FLB200_RNN_PERSISTENT=flag)
        res = subprocess.run([sys.executable, "-c", code, path], env=env, capture_output=True,
                             text=True, timeout=600)
        assert res.returncode == 0, res.stderr[-2000:]
        outs.append(torch.load(path))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_barrier_wait_is_bounded(L):
    """One thread block never arrives at the per-step grid barrier: the others give up after
    the budget, the kernel ends by itself, the status flag reads FLB200_TIMEOUT once and the
    context stays usable."""
    nbytes = L.lib.flb200_selftest_bounded_wait_workspace_bytes()
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert L.lib.flb200_tc_poll_status(stream) == L.OK
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = L.lib.flb200_selftest_bounded_wait(5.0, ws.data_ptr(), nbytes, stream)
    t1.record()
    assert rc == L.OK, L.lib.flb200_last_error()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 500.0, "the kernel did not end within its wait budget"
    assert L.lib.flb200_tc_poll_status(stream) == L.TIMEOUT
    assert b"gave up" in L.lib.flb200_last_error()
    assert L.lib.flb200_tc_poll_status(stream) == L.OK  # cleared
    # the context is intact: ordinary work still runs
    a = torch.ones(1024, device="cuda")
    assert float((a + a).sum()) == 2048.0
