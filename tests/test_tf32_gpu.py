"""TF32 (tcgen05 tensor-core) mode against the fp64 oracle.  Bound: relative error
relative to the tensor scale (tests/parity.py scaled_err) <= 2e-3 — fp32 operands are read with a 10-bit mantissa (2^-11 relative
rounding each) and accumulated in fp32; strict mode keeps the 1e-4 bound."""
import ctypes as C

import pytest
import torch

from oracle import flref as R
from tests.parity import TF32_SCALED_TOL, assert_close, assert_close_scaled, randn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    from flashlight_b200 import _lib
    if not _lib.lib.flb200_has_tensor_core_path():
        pytest.fail("tensor-core path unavailable on this device: TF32 mode cannot be tested")
    return _lib


@pytest.fixture(scope="module")
def fx():
    from flashlight_b200 import functions
    return functions


def tc_delta(L, fn):
    before = L.lib.flb200_tc_kernel_launches()
    out = fn()
    torch.cuda.synchronize()
    L.check(L.lib.flb200_tc_poll_status(torch.cuda.current_stream().cuda_stream))
    return out, L.lib.flb200_tc_kernel_launches() - before


# (m, n, k): full tiles, ragged tiles, K tails, skinny shapes that take the swapped orientation
MNK = [(128, 128, 32), (128, 128, 256), (256, 384, 512), (200, 136, 100), (129, 65, 33),
       (1000, 64, 72), (32, 4096, 1024), (4096, 32, 1024), (512, 520, 4100), (64, 64, 8192)]


@pytest.mark.parametrize("mnk", MNK)
@pytest.mark.parametrize("a_mn_major", [False, True])
@pytest.mark.parametrize("b_mn_major", [False, True])
def test_matmul_tf32_all_majors(L, fx, mnk, a_mn_major, b_mn_major):
    m, n, k = mnk
    pad = lambda v: (v + 3) // 4 * 4  # leading dimensions must be multiples of 16 bytes
    if a_mn_major:
        a_store = randn(k, pad(m), seed=1)          # A(i,kk) at kk*ld + i
        a_view, a_str = a_store[:, :m].t(), (1, pad(m))
    else:
        a_store = randn(m, pad(k), seed=1)          # A(i,kk) at i*ld + kk
        a_view, a_str = a_store[:, :k], (pad(k), 1)
    if b_mn_major:
        b_store = randn(k, pad(n), seed=2)          # B(kk,j) at kk*ld + j
        b_view, b_str = b_store[:, :n], (pad(n), 1)
    else:
        b_store = randn(n, pad(k), seed=2)          # B(kk,j) at j*ld + kk
        b_view, b_str = b_store[:, :k].t(), (1, pad(k))
    want = a_view.double() @ b_view.double()
    c, launched = tc_delta(L, lambda: fx.matmul(a_store.cuda(), b_store.cuda(), m=m, n=n, k=k,
                                                a_strides=a_str, b_strides=b_str,
                                                math_mode=L.MATH_TF32))
    assert launched >= 1, "TF32 matmul did not run on the tensor-core kernel"
    assert_close_scaled(c, want, TF32_SCALED_TOL, f"matmul {mnk} a_mn={a_mn_major} b_mn={b_mn_major}")


def test_matmul_tf32_batched_alpha_beta(L, fx):
    a = randn(3, 160, 96, seed=3)
    b = randn(3, 96, 200, seed=4)
    c0 = randn(3, 160, 200, seed=5)
    c = c0.clone().cuda()
    _, launched = tc_delta(L, lambda: fx.matmul(
        a.cuda(), b.cuda(), c, m=160, n=200, k=96, a_strides=(96, 1), b_strides=(200, 1),
        c_strides=(200, 1), batch=3, batch_strides=(160 * 96, 96 * 200, 160 * 200), alpha=0.5,
        beta=2.0, math_mode=L.MATH_TF32))
    assert launched >= 1
    assert_close_scaled(c, 0.5 * a.double() @ b.double() + 2.0 * c0.double(), TF32_SCALED_TOL, "batched matmul")


def test_matmul_tf32_unaligned_layout_falls_back_to_fp32_kernel(L, fx):
    """A leading dimension that is not a multiple of 16 bytes cannot be described to TMA: the
    call still succeeds (fp32 kernel) and meets the strict bound."""
    a = randn(70, 33, seed=6)
    b = randn(33, 50, seed=7)
    c, launched = tc_delta(L, lambda: fx.matmul(a.cuda(), b.cuda(), m=70, n=50, k=33,
                                                a_strides=(33, 1), b_strides=(50, 1),
                                                math_mode=L.MATH_TF32))
    assert launched == 0
    assert_close(c, a.double() @ b.double(), 1e-4, "fallback matmul")


@pytest.mark.parametrize("dims", [(1024, 3136, 64), (1000, 2048, 256), (768, 3072, 512),
                                  (32000, 768, 128), (30, 1024, 2000)])
def test_linear_tf32(L, fx, dims):
    O, I, cols = dims
    x = randn(cols, I, seed=8)
    w = randn(I, O, seed=9) * (1.0 / I ** 0.5)
    b = randn(O, seed=10)
    y, launched = tc_delta(L, lambda: fx.linear(x.cuda(), w.cuda(), b.cuda(), math_mode=L.MATH_TF32))
    assert_close_scaled(y, R.linear(x.double(), w.double(), b.double()), TF32_SCALED_TOL, "linear forward")
    gy = randn(cols, O, seed=11)
    (gx, gw, gb), launched2 = tc_delta(L, lambda: fx.linear_backward(
        x.cuda(), w.cuda(), gy.cuda(), True, math_mode=L.MATH_TF32))
    wx, ww, wb = R.linear_backward(x.double(), w.double(), gy.double(), True)
    assert_close_scaled(gx, wx, TF32_SCALED_TOL, "linear dx")
    assert_close_scaled(gw, ww, TF32_SCALED_TOL, "linear dW")
    assert_close(gb, wb, 1e-4, "linear db")
    if O % 4 == 0 and I % 4 == 0:
        assert launched >= 1 and launched2 >= 2


def test_split_k_is_deterministic_tf32(L, fx):
    a = randn(128, 16384, seed=12)
    b = randn(16384, 128, seed=13)
    run = lambda: fx.matmul(a.cuda(), b.cuda(), m=128, n=128, k=16384, a_strides=(16384, 1),
                            b_strides=(128, 1), math_mode=L.MATH_TF32)
    c1, _ = tc_delta(L, run)
    c2, _ = tc_delta(L, run)
    assert torch.equal(c1, c2)
    assert_close_scaled(c1, a.double() @ b.double(), TF32_SCALED_TOL, "split-K matmul")


# ------------------------------------------------------------- convolution
# N, C, H, W, Cout, kH, kW, sx, sy, px, py, dx, dy, groups, expect tensor-core kernel
TF32_CONV_CASES = [
    (2, 64, 16, 16, 256, 1, 1, 1, 1, 0, 0, 1, 1, 1, True),    # direct 1x1, expand
    (3, 256, 14, 14, 64, 1, 1, 1, 1, 0, 0, 1, 1, 1, True),    # direct 1x1, reduce, 196 pixels
    (2, 128, 28, 28, 128, 1, 1, 1, 1, 0, 0, 1, 1, 1, True),   # direct 1x1
    (8, 256, 16, 16, 256, 1, 1, 1, 1, 0, 0, 1, 1, 1, True),   # direct 1x1 big enough for CTA pairs: forward (planes MN-major), backward filter (64 K blocks)
    (3, 288, 12, 12, 320, 1, 1, 1, 1, 0, 0, 1, 1, 1, True),   # pairs with a phantom half tile and a ragged column block
    (4, 512, 7, 7, 128, 1, 1, 1, 1, 0, 0, 1, 1, 1, True),     # 1x1 on 49-pixel planes: general route
    (2, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1, 1, 1, 1, True),     # 3x3
    (2, 128, 14, 14, 128, 3, 3, 2, 2, 1, 1, 1, 1, 1, True),   # 3x3 stride 2
    (2, 32, 15, 13, 32, 3, 3, 2, 2, 1, 1, 1, 1, 1, True),     # 3x3 stride 2, odd extents: one launch per parity class
    (3, 256, 16, 16, 256, 3, 3, 2, 2, 1, 1, 1, 1, 1, True),   # 3x3 stride 2 on CTA pairs: the classes share a launch
    (2, 256, 14, 14, 512, 1, 1, 2, 2, 0, 0, 1, 1, 1, True),   # 1x1 stride 2 downsample
    (2, 32, 9, 11, 48, 1, 1, 3, 2, 0, 0, 1, 1, 1, True),      # 1x1, strides (3, 2), odd extents
    (2, 3, 32, 32, 64, 7, 7, 2, 2, 3, 3, 1, 1, 1, True),      # stem: K = 147 (padded filter rows)
    (4, 1, 28, 28, 32, 5, 5, 1, 1, 2, 2, 1, 1, 1, True),      # MNIST conv1: K = 25
    (3, 3, 37, 45, 24, 3, 3, 1, 2, 1, 0, 1, 1, 1, True),      # few channels, ragged, mixed stride
    (2, 4, 20, 19, 40, 5, 8, 2, 1, 0, 3, 1, 2, 1, True),      # 4 channels, 8-wide filter rows, dilated rows
    (2, 2, 12, 200, 16, 2, 3, 1, 1, 1, 1, 1, 1, 1, True),     # few channels, rows wider than one patch
    (2, 80, 1, 100, 96, 1, 13, 1, 1, 6, 0, 1, 1, 1, True),    # conv-ASR time convolution
    (3, 48, 1, 50, 48, 1, 13, 1, 1, 6, 0, 1, 1, 1, True),     # 48 channels: half-filled 32-channel groups
    (3, 16, 1, 50, 48, 1, 13, 1, 1, 6, 0, 1, 1, 1, True),     # 16 channels
    (7, 8, 9, 10, 6, 3, 4, 1, 1, 2, 1, 1, 1, 1, True),        # reference test shape, ragged pixels
    (2, 8, 9, 10, 6, 3, 4, 1, 1, 2, 1, 2, 1, 1, True),        # dilation
    (2, 8, 9, 10, 6, 3, 4, 1, 1, 2, 1, 1, 1, 2, False),       # groups: fp32 kernel
]


@pytest.mark.parametrize("case", TF32_CONV_CASES)
def test_conv2d_tf32(L, case):
    from flashlight_b200.extension import B200AutogradExtension
    N, Cin, H, W, Cout, kH, kW, sx, sy, px, py, dx, dy, groups, expect_tc = case
    ext = B200AutogradExtension(math_mode=L.MATH_TF32)
    x = randn(N, Cin, H, W, seed=21)
    w = randn(Cout, Cin // groups, kH, kW, seed=22) * (1.0 / (Cin // groups * kH * kW) ** 0.5)
    b = randn(Cout, seed=23)
    args = (sx, sy, px, py, dx, dy, groups)
    y, n1 = tc_delta(L, lambda: ext.conv2d(x.cuda(), w.cuda(), b.cuda(), *args))
    want = R.conv2d(x.double(), w.double(), b.double(), *args)
    assert tuple(y.shape) == tuple(want.shape)
    assert_close_scaled(y, want, TF32_SCALED_TOL, "conv forward")
    gy = randn(*want.shape, seed=24)
    gx, n2 = tc_delta(L, lambda: ext.conv2dBackwardData(gy.cuda(), x.cuda(), w.cuda(), *args))
    assert_close_scaled(gx, R.conv2d_backward_data(gy.double(), x.shape, w.double(), *args),
                        TF32_SCALED_TOL, "conv backward data")
    (gw, gb), n3 = tc_delta(L, lambda: ext.conv2dBackwardFilterBias(gy.cuda(), x.cuda(), w.cuda(),
                                                                    b.cuda(), *args))
    wgw, wgb = R.conv2d_backward_filter_bias(gy.double(), x.double(), w.shape, True, *args)
    assert_close_scaled(gw, wgw, TF32_SCALED_TOL, "conv backward filter")
    assert_close(gb, wgb, 1e-4, "conv backward bias")
    if expect_tc:
        assert n1 >= 1 and n2 >= 1 and n3 >= 1, (n1, n2, n3)
    else:
        assert n1 == 0 and n2 == 0 and n3 == 0


@pytest.mark.parametrize("which", ["x", "w", "gy"])
@pytest.mark.parametrize("case", [(2, 64, 16, 16, 256, 1, 1, 0), (2, 64, 14, 14, 64, 3, 1, 1)])
def test_conv2d_tf32_unaligned_operand_runs_on_fp32_kernel(L, case, which):
    """The tensor-core routes hand their operands to TMA and use 16-byte vectors on the scratch:
    a tensor that starts 4 bytes off a 16-byte boundary (an offset view) must never reach them.
    The call still succeeds, on the fp32 kernel, and meets the strict bound."""
    from flashlight_b200.extension import B200AutogradExtension
    N, Cin, H, W, Cout, k, s, p = case
    ext = B200AutogradExtension(math_mode=L.MATH_TF32, cache_layouts=False)

    def off_by_4(t):  # same values, storage starting one float past an aligned address
        buf = torch.empty(t.numel() + 1, dtype=t.dtype, device="cuda")
        view = buf[1:].view(t.shape)
        view.copy_(t)
        assert view.data_ptr() % 16 == 4
        return view

    x = randn(N, Cin, H, W, seed=51)
    w = randn(Cout, Cin, k, k, seed=52) * (1.0 / (Cin * k * k) ** 0.5)
    args = (s, s, p, p, 1, 1, 1)
    want = R.conv2d(x.double(), w.double(), None, *args)
    gy = randn(*want.shape, seed=53)
    xd = off_by_4(x) if which == "x" else x.cuda()
    wd = off_by_4(w) if which == "w" else w.cuda()
    gyd = off_by_4(gy) if which == "gy" else gy.cuda()
    def check(got, wanted, op_uses, what):
        # the passes that read the offset tensor run in fp32 (strict bound); the third pass
        # still takes the tensor-core route (TF32 bound)
        if which in op_uses:
            assert_close(got, wanted, 1e-4, what + " on an offset view")
        else:
            assert_close_scaled(got, wanted, TF32_SCALED_TOL, what)

    y, n1 = tc_delta(L, lambda: ext.conv2d(xd, wd, None, *args))
    check(y, want, ("x", "w"), "conv forward")
    gx, n2 = tc_delta(L, lambda: ext.conv2dBackwardData(gyd, xd, wd, *args))
    check(gx, R.conv2d_backward_data(gy.double(), x.shape, w.double(), *args), ("gy", "w"),
          "conv backward data")
    (gw, _), n3 = tc_delta(L, lambda: ext.conv2dBackwardFilterBias(gyd, xd, wd, None, *args))
    wgw, _ = R.conv2d_backward_filter_bias(gy.double(), x.double(), w.shape, False, *args)
    check(gw, wgw, ("gy", "x"), "conv backward filter")
    uses = {"x": (n1, n3), "w": (n1, n2), "gy": (n2, n3)}[which]
    assert uses == (0, 0), f"an unaligned {which} reached a tensor-core kernel: {uses}"


@pytest.mark.parametrize("dims", [
    (80, 128, 2, 32, 6),    # per-step contraction + cell kernel
    (80, 256, 2, 32, 5),    # fused LSTM step, one CTA per cluster
    (48, 512, 2, 7, 4),     # fused step, clusters of 2, ragged batch
    (40, 1024, 1, 32, 3),   # fused step, clusters of 4 (the biLSTM workload's hidden size)
])
def test_rnn_tf32(L, dims):
    """The recurrent and input GEMMs of the RNN run on the tensor-core kernels in TF32 mode."""
    from flashlight_b200.extension import AutogradPayload, B200AutogradExtension, RNNGradData
    ext = B200AutogradExtension(math_mode=L.MATH_TF32)
    I, H, L_, B, T = dims
    n = R.rnn_num_params(I, H, L_, R.RNN_LSTM, True)
    w = randn(n, seed=40) * (0.5 / H ** 0.5)
    x = randn(T, B, I, seed=41)
    payload = AutogradPayload()
    (y, hy, cy), launched = tc_delta(L, lambda: ext.rnn(x.cuda(), None, None, w.cuda(), H, L_,
                                                         R.RNN_LSTM, True, 0.0, payload))
    wy, why, wcy = R.rnn(x.double(), None, None, w.double(), H, L_, R.RNN_LSTM, True)
    assert launched >= 1
    assert_close_scaled(y, wy, 5e-3, "rnn y (tf32)")
    gy = randn(T, B, 2 * H, seed=44)
    dx, _, _, dw = ext.rnnBackward(x.cuda(), None, None, w.cuda(), RNNGradData(gy.cuda(), None, None),
                                   y, L_, H, R.RNN_LSTM, True, 0.0, payload)
    wdx, _, _, wdw = R.rnn_backward(x.double(), None, None, w.double(), H, L_, R.RNN_LSTM, True,
                                    gy.double(), None, None)
    assert_close_scaled(dx, wdx, 5e-3, "rnn dx (tf32)")
    assert_close_scaled(dw, wdw, 5e-3, "rnn dw (tf32)")


@pytest.mark.parametrize("mode", [R.RNN_RELU, R.RNN_TANH, R.RNN_GRU])
@pytest.mark.parametrize("dims", [(40, 128, 2, 8, 6, True), (24, 256, 1, 32, 5, False)])
def test_rnn_tf32_other_cells(L, mode, dims):
    """RELU / TANH / GRU cells in TF32 mode: the input and recurrent contractions run on the
    tensor-core kernels; same bound as the LSTM case.  The RELU cell is discontinuous: a TF32
    rounding difference flips the mask of a few pre-activations that are almost zero, which the
    backward pass turns into larger differences, hence its root-mean-square gradient bound."""
    from flashlight_b200.extension import AutogradPayload, B200AutogradExtension, RNNGradData
    ext = B200AutogradExtension(math_mode=L.MATH_TF32)
    I, H, L_, B, T, bidir = dims
    dirs = 2 if bidir else 1
    n = R.rnn_num_params(I, H, L_, mode, bidir)
    w = randn(n, seed=45) * (0.5 / H ** 0.5)
    x = randn(T, B, I, seed=46)
    hx = randn(L_ * dirs, B, H, seed=47) * 0.5
    payload = AutogradPayload()
    (y, hy, _), launched = tc_delta(L, lambda: ext.rnn(x.cuda(), hx.cuda(), None, w.cuda(), H, L_,
                                                       mode, bidir, 0.0, payload))
    wy, why, _ = R.rnn(x.double(), hx.double(), None, w.double(), H, L_, mode, bidir)
    assert launched >= 1
    assert_close_scaled(y, wy, 5e-3, "rnn y (tf32)")
    assert_close_scaled(hy, why, 5e-3, "rnn hy (tf32)")
    gy = randn(T, B, dirs * H, seed=48)
    dx, dhx, _, dw = ext.rnnBackward(x.cuda(), hx.cuda(), None, w.cuda(),
                                     RNNGradData(gy.cuda(), None, None), y, L_, H, mode, bidir, 0.0,
                                     payload)
    wdx, wdhx, _, wdw = R.rnn_backward(x.double(), hx.double(), None, w.double(), H, L_, mode, bidir,
                                       gy.double(), None, None)
    if mode == R.RNN_RELU:
        # A flipped mask changes a whole column of the gradient, so no element-wise bound holds
        # (the strict mode, tested elsewhere, is exact to 1e-6); what TF32 must still deliver is
        # the same gradient in the root-mean-square sense.
        for got, want, what in ((dx, wdx, "dx"), (dhx, wdhx, "dhx"), (dw, wdw, "dw")):
            d = got.double().cpu() - want
            rms = float(d.pow(2).mean().sqrt() / want.pow(2).mean().sqrt())
            assert rms <= 0.15, f"relu rnn {what} (tf32): rms error {rms:.3e}"
        return
    assert_close_scaled(dx, wdx, 5e-3, "rnn dx (tf32)")
    assert_close_scaled(dhx, wdhx, 5e-3, "rnn dhx (tf32)")
    assert_close_scaled(dw, wdw, 5e-3, "rnn dw (tf32)")


# ------------------------------------------------------------- layout cache
@pytest.mark.parametrize("case", [
    (2, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1, 1, 1, 1),     # channels-last patch route
    (2, 128, 14, 14, 128, 3, 3, 2, 2, 1, 1, 1, 1, 1),   # strided
    (2, 3, 32, 32, 64, 7, 7, 2, 2, 3, 3, 1, 1, 1),      # row-window route (caches x only)
    (2, 64, 16, 16, 256, 1, 1, 1, 1, 0, 0, 1, 1, 1),    # direct 1x1: nothing to cache
])
def test_conv2d_layout_cache(L, case):
    """With a payload the backward-filter pass reuses the channels-last copies made by the
    forward and backward-data passes; results are bit-identical to the uncached calls, and a
    copy is never reused for a different tensor."""
    from flashlight_b200.extension import AutogradPayload, B200AutogradExtension
    N, Cin, H, W, Cout, kH, kW, sx, sy, px, py, dx, dy, groups = case
    plain = B200AutogradExtension(math_mode=L.MATH_TF32, cache_layouts=False)
    cached = B200AutogradExtension(math_mode=L.MATH_TF32, cache_layouts=True)
    x = randn(N, Cin, H, W, seed=31).cuda()
    w = (randn(Cout, Cin, kH, kW, seed=32) * (1.0 / (Cin * kH * kW) ** 0.5)).cuda()
    args = (sx, sy, px, py, dx, dy, groups)
    y0 = plain.conv2d(x, w, None, *args)
    gy = randn(*y0.shape, seed=33).cuda()
    gx0 = plain.conv2dBackwardData(gy, x, w, *args)
    gw0, _ = plain.conv2dBackwardFilterBias(gy, x, w, None, *args)

    payload = AutogradPayload()
    before = L.kernel_launches()
    y1 = cached.conv2d(x, w, None, *args, payload)
    gx1 = cached.conv2dBackwardData(gy, x, w, *args, None, payload)
    gw1, _ = cached.conv2dBackwardFilterBias(gy, x, w, None, *args, None, None, payload)
    with_cache = L.kernel_launches() - before
    before = L.kernel_launches()
    plain.conv2d(x, w, None, *args)
    plain.conv2dBackwardData(gy, x, w, *args)
    plain.conv2dBackwardFilterBias(gy, x, w, None, *args)
    without = L.kernel_launches() - before
    assert torch.equal(y0, y1) and torch.equal(gx0, gx1) and torch.equal(gw0, gw1)
    keeps = L.lib.flb200_conv2d_cache_bytes(
        C.byref(cached._conv_desc(x, w, *args)), 0) > 0
    assert (with_cache < without) == keeps, (with_cache, without)

    # a second backward pass with another grad_y must not see the first one's copy
    gy2 = randn(*y0.shape, seed=34).cuda()
    gx2 = cached.conv2dBackwardData(gy2, x, w, *args, None, payload)
    gy3 = randn(*y0.shape, seed=35).cuda()
    gw3, _ = cached.conv2dBackwardFilterBias(gy3, x, w, None, *args, None, None, payload)
    want3, _ = plain.conv2dBackwardFilterBias(gy3, x, w, None, *args)
    assert torch.equal(gx2, plain.conv2dBackwardData(gy2, x, w, *args))
    assert torch.equal(gw3, want3)
    # ... nor a changed x (in-place update bumps the version counter)
    x.mul_(0.5)
    gw4, _ = cached.conv2dBackwardFilterBias(gy3, x, w, None, *args, None, None, payload)
    want4, _ = plain.conv2dBackwardFilterBias(gy3, x, w, None, *args)
    assert torch.equal(gw4, want4)


# ------------------------------------------------------------- bf16 contraction
BF16_CASES = [
    # m, n, k, batch, a transposed (m contiguous), b transposed (n contiguous)
    (256, 128, 512, 1, False, False),
    (200, 72, 136, 1, False, False),     # ragged tiles, K not a multiple of the 64-element stage
    (256, 256, 64, 1, True, False),      # A with the m index contiguous
    (192, 320, 256, 1, False, True),     # B with the n index contiguous
    (128, 128, 4096, 1, True, True),     # both, long K (split-K)
    (96, 64, 128, 6, False, True),       # batched (attention-sized)
    (24, 512, 768, 1, False, False),     # few rows: operands swap sides
    (24, 16, 24, 12, False, True),       # attention context at a toy size: n below one 64-column box
    (16, 24, 40, 5, True, True),
]


@pytest.mark.parametrize("case", BF16_CASES)
def test_matmul_bf16(L, case):
    """bf16 operands and result, fp32 accumulation in tensor memory.  Bound: 1e-2 of the result's
    largest magnitude (the result is rounded to 8 mantissa bits; inputs are exact in bf16)."""
    from flashlight_b200 import functions as F
    m, n, k, batch, ta, tb = case
    a = randn(batch, k, m, seed=41) if ta else randn(batch, m, k, seed=41)
    b = randn(batch, n, k, seed=42) if not tb else randn(batch, k, n, seed=42)
    ab, bb = a.to(torch.bfloat16), b.to(torch.bfloat16)
    A64 = (ab.double().transpose(1, 2) if ta else ab.double())
    B64 = (bb.double().transpose(1, 2) if not tb else bb.double())
    want = A64 @ B64
    a_str = (1, m) if ta else (k, 1)
    b_str = (n, 1) if tb else (1, k)      # strides of B viewed as (k, n)
    before = L.lib.flb200_tc_kernel_launches()
    got = F.matmul(ab.cuda(), bb.cuda(), m=m, n=n, k=k, a_strides=a_str, b_strides=b_str,
                   batch=batch, batch_strides=(m * k, n * k, 0))
    assert got.dtype == torch.bfloat16
    assert L.lib.flb200_tc_kernel_launches() > before
    assert_close_scaled(got.float().reshape(want.shape), want, 1e-2, "bf16 matmul")
    assert L.lib.flb200_tc_poll_status(None) == 0  # no bounded wait ran out


# ------------------------------------------------------------- run-time mode selection
def test_conv_gradients_pick_a_tensor_core_mode(L):
    """createBenchmarkOptions(): with benchmark mode on, a strict-mode extension's convolution
    gradients try all three modes and settle on a tensor-core one for a tensor-core-sized layer;
    with it off they stay strict."""
    from flashlight_b200.extension import B200AutogradExtension, DynamicBenchmark
    ext = B200AutogradExtension(math_mode=L.MATH_STRICT_F32)
    x = randn(32, 128, 28, 28, seed=70).cuda()
    w = (randn(128, 128, 3, 3, seed=71) * 0.03).cuda()
    gy = randn(32, 128, 28, 28, seed=72).cuda()
    args = (1, 1, 1, 1, 1, 1, 1)
    want_gx = R.conv2d_backward_data(gy.double().cpu(), x.shape, w.double().cpu(), *args)
    want_gw, _ = R.conv2d_backward_filter_bias(gy.double().cpu(), x.double().cpu(), w.shape, False, *args)
    db, fb = ext.createBenchmarkOptions(), ext.createBenchmarkOptions()
    _, launched = tc_delta(L, lambda: ext.conv2dBackwardData(gy, x, w, *args, db, None))
    assert launched == 0 and db.counts == [0, 0, 0]            # benchmark mode is off
    DynamicBenchmark.setBenchmarkMode(True)
    try:
        for _ in range(30):
            gx = ext.conv2dBackwardData(gy, x, w, *args, db, None)
            gw, _ = ext.conv2dBackwardFilterBias(gy, x, w, None, *args, fb, None, None)
            assert_close_scaled(gx, want_gx, 2e-3, "tuned backward data")
            assert_close_scaled(gw, want_gw, 2e-3, "tuned backward filter")
        for b in (db, fb):
            assert b.timingsComplete() and b.counts == [10, 10, 10]
            assert b.currentOption() in (L.MATH_TF32, L.MATH_F32X3)
            assert b.times[0] > min(b.times[1], b.times[2])
        _, launched = tc_delta(L, lambda: ext.conv2dBackwardData(gy, x, w, *args, db, None))
        assert launched >= 1                                     # now on the tensor cores
    finally:
        DynamicBenchmark.setBenchmarkMode(False)


# ------------------------------------------------------------- Linear + bias + GELU
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-3), (torch.bfloat16, 1.6e-2)])
@pytest.mark.parametrize("dims", [(96, 64, 200), (768, 3072, 512), (256, 160, 33)])
@pytest.mark.parametrize("gelu", [False, True])
def test_linear_bias_activation_fused(L, fx, dtype, tol, dims, gelu):
    """flb200_linear_bias_act_forward: bias and gelu applied in the contraction's epilogue, the
    pre-activation kept; against fp64 (the bf16 case from bf16-rounded operands), and the tape
    operator's gradients against autograd of the same chain."""
    from flashlight_b200 import autograd as A
    I, O, rows = dims
    x = randn(rows, I, seed=120).to(dtype)
    w = (randn(I, O, seed=121) * (1.0 / I ** 0.5)).to(dtype)
    b = randn(O, seed=122)
    out = fx.linear_bias_act(x.cuda(), w.cuda(), b.cuda(), gelu, math_mode=L.MATH_TF32)
    z = x.double() @ w.double() + b.double()
    want = torch.nn.functional.gelu(z, approximate="tanh") if gelu else z
    if out is None:
        # few rows: the contraction runs transposed (C^T = B^T A^T), where nothing is fused;
        # the tape operator below then takes the operators one by one
        assert rows < 64
    else:
        y, pre = out
        assert y.dtype == dtype
        assert_close_scaled(y.float(), want, tol, "linear + bias (+ gelu)")
        if gelu:
            assert_close_scaled(pre.float(), z, tol, "pre-activation")
        else:
            assert pre is None
    # the tape operator: fused forward, chain gradient
    prev = A.extension().math_mode
    A.set_math_mode(L.MATH_TF32)
    try:
        xv, wv, bv = (A.Variable(t.cuda(), True) for t in (x, w, b))
        gy = randn(rows, O, seed=123).to(dtype)
        A.linear(xv, wv, bv, gelu=gelu).backward(gy.cuda())
    finally:
        A.set_math_mode(prev)
    xr, wr, br = (t.double().requires_grad_(True) for t in (x, w, b))
    zz = xr @ wr + br
    (torch.nn.functional.gelu(zz, approximate="tanh") if gelu else zz).backward(gy.double())
    assert_close_scaled(xv.grad.float(), xr.grad, 2 * tol, "linear dx")
    assert_close_scaled(wv.grad.float(), wr.grad, 2 * tol, "linear dw")
    assert_close_scaled(bv.grad.float(), br.grad, 2 * tol, "linear db")


def test_linear_bias_activation_declines_gracefully(L, fx):
    x, w, b = randn(8, 16, seed=124).cuda(), randn(16, 24, seed=125).cuda(), randn(24, seed=126).cuda()
    assert fx.linear_bias_act(x, w, b, True, math_mode=L.MATH_TF32) is None      # O % 32 != 0
    x2, w2, b2 = randn(8, 16, seed=127).cuda(), randn(16, 32, seed=128).cuda(), randn(32, seed=129).cuda()
    assert fx.linear_bias_act(x2, w2, b2, True, math_mode=L.MATH_STRICT_F32) is None  # fp32 FMA mode
