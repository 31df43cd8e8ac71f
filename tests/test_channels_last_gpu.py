"""Channels-last storage (FLB200_LAYOUT_NHWC): the same operators on tensors stored
[N][H][W][C], against the same fp64 oracle.  A torch tensor in channels_last memory format keeps
its logical (N, C, H, W) indexing, so results compare element for element with the oracle's.
Bounds as in the fl-order tests: strict fp32 1e-4 (tests/parity.py rel_err), TF32 2e-3 of the
tensor's scale; integer payloads and layouts exactly."""
import pytest
import torch

from oracle import cpu_workloads as CW
from oracle import flref as R
from tests.parity import STRICT_TOL, TF32_SCALED_TOL, assert_close, assert_close_scaled, randn

pytestmark = pytest.mark.gpu
CL = torch.channels_last


@pytest.fixture(scope="module")
def L():
    from flashlight_b200 import _lib
    if not _lib.lib.flb200_has_tensor_core_path():
        pytest.fail("tensor-core path unavailable on this device")
    return _lib


def cl(t):
    """Device copy stored channels-last."""
    return t.cuda().contiguous(memory_format=CL)


def is_cl(t):
    from flashlight_b200.extension import is_channels_last
    return is_channels_last(t)


# N, C, H, W, Cout, kH, kW, sx, sy, px, py, dx, dy: every route the ResNet / MNIST layers take
CL_CONV_CASES = [
    (2, 64, 16, 16, 256, 1, 1, 1, 1, 0, 0, 1, 1),    # 1x1 expand: plain GEMM over the pixels
    (3, 256, 14, 14, 64, 1, 1, 1, 1, 0, 0, 1, 1),    # 1x1 reduce
    (4, 512, 7, 7, 128, 1, 1, 1, 1, 0, 0, 1, 1),     # 49-pixel planes: no padded patch rows
    (8, 256, 16, 16, 256, 1, 1, 1, 1, 0, 0, 1, 1),   # big enough for CTA pairs
    (3, 288, 12, 12, 320, 1, 1, 1, 1, 0, 0, 1, 1),   # ragged column block, K tail
    (2, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1, 1, 1),     # 3x3
    (2, 128, 14, 14, 128, 3, 3, 2, 2, 1, 1, 1, 1),   # 3x3 stride 2
    (2, 32, 15, 13, 32, 3, 3, 2, 2, 1, 1, 1, 1),     # odd extents: one launch per parity class
    (3, 256, 16, 16, 256, 3, 3, 2, 2, 1, 1, 1, 1),   # stride 2 on CTA pairs, classes share a launch
    (2, 256, 14, 14, 512, 1, 1, 2, 2, 0, 0, 1, 1),   # 1x1 stride 2 downsample (cell fill)
    (2, 32, 9, 11, 48, 1, 1, 3, 2, 0, 0, 1, 1),      # strides (3, 2): fp32 kernel in every mode
    (2, 20, 9, 10, 24, 3, 4, 1, 1, 2, 1, 2, 1),      # dilation, ragged
    (2, 6, 9, 10, 10, 3, 3, 1, 1, 1, 1, 1, 1),       # channels not a multiple of 4: fp32 kernel
]


@pytest.mark.parametrize("mode", ["strict", "tf32", "f32x3"])
@pytest.mark.parametrize("case", CL_CONV_CASES)
def test_conv2d_channels_last(L, case, mode):
    from flashlight_b200.extension import B200AutogradExtension
    N, Cin, H, W, Cout, kH, kW, sx, sy, px, py, dx, dy = case
    ext = B200AutogradExtension(math_mode=L.MATH_BY_NAME[mode])
    x = randn(N, Cin, H, W, seed=61)
    w = randn(Cout, Cin, kH, kW, seed=62) * (1.0 / (Cin * kH * kW) ** 0.5)
    b = randn(Cout, seed=63)
    args = (sx, sy, px, py, dx, dy, 1)
    if mode == "tf32":
        check = lambda got, want, what: assert_close_scaled(got, want, TF32_SCALED_TOL, what)
    elif mode == "f32x3":
        check = lambda got, want, what: assert_close_scaled(got, want, 2e-5, what)
    else:
        check = lambda got, want, what: assert_close(got, want, STRICT_TOL, what)
    before = L.lib.flb200_tc_kernel_launches()
    y = ext.conv2d(cl(x), w.cuda(), b.cuda(), *args)
    want = R.conv2d(x.double(), w.double(), b.double(), *args)
    assert tuple(y.shape) == tuple(want.shape) and (is_cl(y) or y.is_contiguous())
    assert y.is_contiguous(memory_format=CL)
    check(y, want, "conv forward")
    gy = randn(*want.shape, seed=64)
    gx = ext.conv2dBackwardData(cl(gy), cl(x), w.cuda(), *args)
    assert gx.is_contiguous(memory_format=CL)
    check(gx, R.conv2d_backward_data(gy.double(), x.shape, w.double(), *args), "conv backward data")
    gw, gb = ext.conv2dBackwardFilterBias(cl(gy), cl(x), w.cuda(), b.cuda(), *args)
    wgw, wgb = R.conv2d_backward_filter_bias(gy.double(), x.double(), w.shape, True, *args)
    assert gw.is_contiguous()  # parameters keep the reference's layout
    check(gw, wgw, "conv backward filter")
    assert_close(gb, wgb, STRICT_TOL, "conv backward bias")
    torch.cuda.synchronize()
    tc = L.lib.flb200_tc_kernel_launches() - before
    expect_tc = mode != "strict" and Cin % 4 == 0 and Cout % 4 == 0 and Cin >= 16 and max(sx, sy) <= 2
    assert (tc >= 3) == expect_tc, (tc, expect_tc)


@pytest.mark.parametrize("mode", ["strict", "tf32"])
@pytest.mark.parametrize("case", [(2, 3, 32, 32, 64, 7, 7, 2, 2, 3, 3), (4, 1, 28, 28, 32, 5, 5, 1, 1, 2, 2),
                                  (3, 3, 37, 45, 24, 3, 3, 1, 2, 1, 0)])
def test_first_convolution_fl_order_in_channels_last_out(L, case, mode):
    """A network's first convolution: x in fl's order, y and grad_y channels-last."""
    from flashlight_b200.extension import B200AutogradExtension
    N, Cin, H, W, Cout, kH, kW, sx, sy, px, py = case
    ext = B200AutogradExtension(math_mode=L.MATH_BY_NAME[mode])
    x = randn(N, Cin, H, W, seed=65)
    w = randn(Cout, Cin, kH, kW, seed=66) * (1.0 / (Cin * kH * kW) ** 0.5)
    args = (sx, sy, px, py, 1, 1, 1)
    check = (lambda g, wnt, what: assert_close_scaled(g, wnt, TF32_SCALED_TOL, what)) if mode == "tf32" \
        else (lambda g, wnt, what: assert_close(g, wnt, STRICT_TOL, what))
    before = L.lib.flb200_tc_kernel_launches()
    y = ext.conv2d(x.cuda(), w.cuda(), None, *args, channels_last_out=True)
    want = R.conv2d(x.double(), w.double(), None, *args)
    assert is_cl(y)
    check(y, want, "first conv forward")
    gy = randn(*want.shape, seed=67)
    gw, _ = ext.conv2dBackwardFilterBias(cl(gy), x.cuda(), w.cuda(), None, *args)
    wgw, _ = R.conv2d_backward_filter_bias(gy.double(), x.double(), w.shape, False, *args)
    check(gw, wgw, "first conv backward filter")
    gx = ext.conv2dBackwardData(cl(gy), x.cuda(), w.cuda(), *args)
    assert gx.is_contiguous()
    check(gx, R.conv2d_backward_data(gy.double(), x.shape, w.double(), *args), "first conv backward data")
    torch.cuda.synchronize()
    if mode == "tf32":
        assert L.lib.flb200_tc_kernel_launches() - before >= 2


POOL_GEOS = [(2, 2, 2, 2, 0, 0), (3, 3, 2, 2, 1, 1), (3, 2, 1, 2, 1, 0), (7, 7, 1, 1, 0, 0),
             (3, 3, 2, 2, 0, 0), (2, 2, 2, 2, 1, 1)]  # the last two: the 2 x 2 cell kernels' other paddings


@pytest.mark.parametrize("mode", [R.POOL_MAX, R.POOL_AVG_INCLUDE_PAD, R.POOL_AVG_EXCLUDE_PAD])
@pytest.mark.parametrize("geo", POOL_GEOS)
@pytest.mark.parametrize("with_payload", [True, False])
@pytest.mark.parametrize("channels", [8, 5])
def test_pool2d_channels_last(L, mode, geo, with_payload, channels):
    from flashlight_b200.extension import AutogradPayload, B200AutogradExtension
    ext = B200AutogradExtension(math_mode=L.MATH_STRICT_F32)
    wx, wy, sx, sy, px, py = geo
    x = randn(3, channels, 14, 13, seed=71)
    payload = AutogradPayload() if with_payload else None
    y = ext.pool2d(cl(x), wx, wy, sx, sy, px, py, mode, payload)
    want = R.pool2d(x.double(), wx, wy, sx, sy, px, py, mode)
    assert tuple(y.shape) == tuple(want.shape) and y.is_contiguous(memory_format=CL)
    assert_close(y, want, 1e-5, "pool forward")
    gy = randn(*want.shape, seed=72)
    gx = ext.pool2dBackward(cl(gy), cl(x), y, wx, wy, sx, sy, px, py, mode, payload)
    assert gx.is_contiguous(memory_format=CL)
    assert_close(gx, R.pool2d_backward(gy.double(), x.double(), wx, wy, sx, sy, px, py, mode), 1e-5,
                 "pool backward")
    if mode == R.POOL_MAX and with_payload:
        _, arg = R.pool2d_naive(x.numpy(), wx, wy, sx, sy, px, py, mode)
        assert torch.equal(payload.data.argmax.cpu(), torch.from_numpy(arg))


def test_max_pool_ties_after_relu_channels_last(L):
    from flashlight_b200.extension import AutogradPayload, B200AutogradExtension
    ext = B200AutogradExtension(math_mode=L.MATH_STRICT_F32)
    x = torch.relu(randn(2, 8, 12, 12, seed=73))  # many all-zero windows
    gy = randn(*R.pool2d(x, 3, 3, 2, 2, 1, 1, R.POOL_MAX).shape, seed=74)
    want = R.pool2d_backward(gy.double(), x.double(), 3, 3, 2, 2, 1, 1, R.POOL_MAX)
    for payload in (AutogradPayload(), None):
        y = ext.pool2d(cl(x), 3, 3, 2, 2, 1, 1, R.POOL_MAX, payload)
        gx = ext.pool2dBackward(cl(gy), cl(x), y, 3, 3, 2, 2, 1, 1, R.POOL_MAX, payload)
        assert_close(gx, want, 1e-6, "max pool gradient routing")


BN_SHAPES = [(8, 64, 28, 28), (4, 256, 7, 7), (3, 12, 6, 7), (2, 6, 5, 3), (16, 2048, 2, 2)]


@pytest.mark.parametrize("shape", BN_SHAPES)
@pytest.mark.parametrize("affine", [True, False])
def test_batchnorm_channels_last(L, shape, affine):
    from flashlight_b200.extension import B200AutogradExtension
    ext = B200AutogradExtension(math_mode=L.MATH_STRICT_F32)
    ch = shape[1]
    x = randn(*shape, seed=81) * 1.7 + 0.4
    w = (randn(ch, seed=82).abs() + 0.5) if affine else None
    b = randn(ch, seed=83) if affine else None
    rm, rv = randn(ch, seed=84) * 0.1, randn(ch, seed=85).abs() + 0.5
    rm_d, rv_d = rm.cuda(), rv.cuda()
    dev = lambda t: None if t is None else t.cuda()
    f64 = lambda t: None if t is None else t.double()
    y, sm, sv = ext.batchnorm(cl(x), dev(w), dev(b), rm_d, rv_d, [2], True, 0.1, 1e-5)
    wy, wm, wi, wrm, wrv = R.batchnorm(x.double(), f64(w), f64(b), rm.double(), rv.double(), [2],
                                       True, 0.1, 1e-5)
    assert y.is_contiguous(memory_format=CL)
    assert_close(y, wy, STRICT_TOL, "bn y")
    assert_close(sm, wm, STRICT_TOL, "bn save_mean")
    assert_close(sv, wi, STRICT_TOL, "bn save_invstd")
    assert_close(rm_d, wrm, STRICT_TOL, "bn running mean")
    assert_close(rv_d, wrv, STRICT_TOL, "bn running var")
    gy = randn(*shape, seed=86)
    gx, gw, gb = ext.batchnormBackward(cl(gy), sm, sv, cl(x), dev(w), [2], True, 1e-5)
    wgx, wgw, wgb = R.batchnorm_backward(gy.double(), x.double(), f64(w), [2], 1e-5)
    assert gx.is_contiguous(memory_format=CL)
    assert_close(gx, wgx, STRICT_TOL, "bn dx")
    assert_close(gw, wgw, STRICT_TOL, "bn dgamma")
    assert_close(gb, wgb, STRICT_TOL, "bn dbeta")
    # relu(batchnorm(x)) as one operator and its gradient, against the chain of operators
    y1, sm1, sv1 = ext.batchnorm(cl(x), dev(w), dev(b), None, None, [2], True, 0.0, 1e-5, relu=True)
    assert_close(y1, torch.relu(wy), STRICT_TOL, "bn+relu y")
    masked = gy.double() * (wy > 0)
    gx1, gw1, gb1 = ext.batchnormReluBackward(cl(gy), sm1, sv1, cl(x), dev(w), dev(b), [2], True, 1e-5)
    w1gx, w1gw, w1gb = R.batchnorm_backward(masked, x.double(), f64(w), [2], 1e-5)
    assert_close(gx1, w1gx, STRICT_TOL, "bn+relu dx")
    assert_close(gw1, w1gw, STRICT_TOL, "bn+relu dgamma")
    assert_close(gb1, w1gb, STRICT_TOL, "bn+relu dbeta")


@pytest.mark.parametrize("shape", [(8, 64, 28, 28), (4, 256, 7, 7), (2, 2048, 3, 3)])
def test_batchnorm_add_relu_channels_last(L, shape):
    """The residual block's tail on channels-last tensors, against the chain of operators."""
    from flashlight_b200.extension import B200AutogradExtension
    ext = B200AutogradExtension(math_mode=L.MATH_STRICT_F32)
    ch = shape[1]
    x = randn(*shape, seed=91) * 1.7 + 0.4
    s = randn(*shape, seed=92)
    w, b = randn(ch, seed=93).abs() + 0.5, randn(ch, seed=94)
    assert ext.batchnormAddReluSupported(cl(x), cl(s), [2])
    y, mask, sm, sv = ext.batchnormAddRelu(cl(x), cl(s), w.cuda(), b.cuda(), None, None, [2], True,
                                           0.0, 1e-5)
    wy, _, _, _, _ = R.batchnorm(x.double(), w.double(), b.double(), None, None, [2], True, 0.0, 1e-5)
    z = wy + s.double()
    assert_close(y, torch.relu(z), STRICT_TOL, "tail y")
    ga, gb_ = randn(*shape, seed=95), randn(*shape, seed=96)
    for second in (gb_, None):
        gz, gx, gw, gbias = ext.batchnormAddReluBackward(
            mask, cl(ga), cl(second) if second is not None else None, sm, sv, cl(x), w.cuda(), [2],
            True, 1e-5)
        tot = ga.double() + (second.double() if second is not None else 0.0)
        want_gz = tot * (y.detach().cpu().double() > 0)
        assert gz.is_contiguous(memory_format=CL)
        assert_close(gz, want_gz, 1e-6, "tail shortcut gradient")
        wgx, wgw, wgb = R.batchnorm_backward(want_gz, x.double(), w.double(), [2], 1e-5)
        assert_close(gx, wgx, STRICT_TOL, "tail dx")
        assert_close(gw, wgw, STRICT_TOL, "tail dgamma")
        assert_close(gbias, wgb, STRICT_TOL, "tail dbeta")
    assert not ext.batchnormAddReluSupported(cl(randn(2, 12, 4, 4, seed=1)), cl(randn(2, 12, 4, 4, seed=2)), [2])


def test_elementwise_needs_equal_layouts(L):
    from flashlight_b200 import functions as F
    a, b = randn(2, 8, 4, 4, seed=1), randn(2, 8, 4, 4, seed=2)
    assert_close(F.add(cl(a), cl(b)), a.double() + b.double(), 1e-6, "add")
    with pytest.raises(ValueError):
        F.add(cl(a), b.cuda())


@pytest.mark.parametrize("mode,loss_tol,grad_tol", [("strict", 1e-4, 1e-3), ("tf32", 2e-3, 0.15)])
@pytest.mark.parametrize("channels_last", [True, False])
def test_resnet_step_both_layouts(L, mode, loss_tol, grad_tol, channels_last):
    """One scaled-down ResNet step with the activations channels-last and in fl's order: same
    loss and gradients (against the CPU restatement), and no layout-copy kernel when
    channels-last."""
    from flashlight_b200 import autograd as A
    from flashlight_b200 import workloads
    A.set_math_mode(L.MATH_BY_NAME[mode])
    try:
        model = workloads.resnet50(seed=7, blocks=(1, 1, 1), classes=10, width=16,
                                   channels_last=channels_last)
        g = torch.Generator().manual_seed(11)
        x = torch.randn(4, 3, 112, 112, generator=g)
        t = torch.randint(0, 10, (4,), generator=g, dtype=torch.int32)
        loss = model.loss(x.cuda(), t.cuda())
        loss.backward()
        params = [p.tensor.detach().cpu().double() for p in model.parameters()]
        want_loss, want_grads = CW.resnet50_step(params, x.double(), t, blocks=(1, 1, 1))
        got = float(loss.tensor.cpu())
        assert abs(got - float(want_loss)) <= loss_tol * max(1.0, abs(float(want_loss)))
        for i, (p, wg) in enumerate(zip(model.parameters(), want_grads)):
            gg = p.grad.detach().cpu().double().reshape(wg.shape)
            if mode == "strict":
                err = float((gg - wg).abs().max()) / (float(wg.abs().max()) or 1.0)
            else:
                err = float((gg - wg).norm()) / (float(wg.norm()) or 1.0)
            assert err <= grad_tol, f"parameter {i} {tuple(wg.shape)}: gradient error {err:.3e}"
    finally:
        A.set_math_mode(L.MATH_STRICT_F32)


# ------------------------------------------------------------- statistics in the conv epilogue
@pytest.mark.parametrize("case", [
    (8, 64, 14, 14, 256, 1, 1, 0),      # channels-last 1 x 1 (GEMM route), expand
    (5, 256, 7, 7, 64, 1, 1, 0),        # ragged last row tile
    (8, 64, 14, 14, 64, 3, 1, 1),       # patch route
    (6, 128, 15, 15, 128, 3, 2, 1),     # strided, patches that overhang the image
    (4, 3, 32, 32, 64, 7, 2, 3),        # first layer: row-window route, fl-order input
    (33, 128, 7, 7, 512, 1, 1, 0),      # wide output on CTA pairs, odd tile count
])
def test_conv_forward_statistics_match_the_output(case):
    """flb200_conv2d_forward_stats: the column sums of the matrix written in the epilogue are the
    per-channel sums of the tensor the same call wrote, and the batch-norm built on them equals the stand-alone one."""
    from flashlight_b200 import _lib as L
    from flashlight_b200.extension import B200AutogradExtension
    N, Cc, H, W, Co, k, s, p = case
    ext = B200AutogradExtension(math_mode=L.MATH_TF32)
    x = randn(N, Cc, H, W, seed=110).cuda()
    first = Cc <= 4
    if not first:
        x = x.contiguous(memory_format=torch.channels_last)
    w = (randn(Co, Cc, k, k, seed=111) * (1.0 / (Cc * k * k) ** 0.5)).cuda()
    args = (s, s, p, p, 1, 1, 1)
    sums = []
    y = ext.conv2d(x, w, None, *args, None, channels_last_out=True if first else None, stats_out=sums)
    assert len(sums) == 1
    matrix, groups = sums[0]
    assert matrix.numel() >= groups * 2 * Co
    totals = matrix[:groups * 2 * Co].view(groups, 2 * Co).double().sum(0)
    y_plain = ext.conv2d(x, w, None, *args, None, channels_last_out=True if first else None)
    assert torch.equal(y, y_plain)                       # same kernels, same result
    want_s = y.double().sum(dim=(0, 2, 3))
    want_q = (y.double() ** 2).sum(dim=(0, 2, 3))
    assert_close_scaled(totals[:Co], want_s, 2e-6, "sum of y")
    assert_close_scaled(totals[Co:], want_q, 2e-6, "sum of y^2")
    # batch-norm (+ relu) from the totals against the one that takes its own statistics
    g, b = (randn(Co, seed=112) * 0.3 + 1.0).cuda(), randn(Co, seed=113).cuda()
    rm0, rv0 = torch.zeros(Co).cuda(), torch.ones(Co).cuda()
    rm1, rv1 = rm0.clone(), rv0.clone()
    o0, m0, v0 = ext.batchnorm(y, g, b, rm0, rv0, [2], True, 0.1, 1e-5, relu=True)
    o1, m1, v1 = ext.batchnorm(y, g, b, rm1, rv1, [2], True, 0.1, 1e-5, relu=True,
                               conv_stats=sums[0])
    assert_close_scaled(m1, m0, 2e-5, "mean from sums")  # means are ~1e-2 of the values summed
    assert_close_scaled(v1, v0, 2e-5, "inverse std from sums")
    assert_close_scaled(rv1, rv0, 2e-5, "running variance from sums")
    assert_close_scaled(o1, o0, 5e-5, "batch-norm + relu from sums")
    if Co % 8 == 0:
        short = randn(*y.shape, seed=114).cuda().contiguous(memory_format=torch.channels_last)
        a0 = ext.batchnormAddRelu(y, short, g, b, None, None, [2], True, 0.1, 1e-5)
        a1 = ext.batchnormAddRelu(y, short, g, b, None, None, [2], True, 0.1, 1e-5,
                                  conv_stats=sums[0])
        assert_close_scaled(a1[0], a0[0], 5e-5, "batch-norm + add + relu from sums")


def test_conv_statistics_are_declined_where_not_built():
    from flashlight_b200 import _lib as L
    from flashlight_b200.extension import B200AutogradExtension
    x = randn(2, 32, 8, 8, seed=115).cuda()
    w = randn(48, 32, 3, 3, seed=116).cuda()
    for ext, xin in ((B200AutogradExtension(math_mode=L.MATH_TF32), x),                       # fl order
                     (B200AutogradExtension(math_mode=L.MATH_STRICT_F32),
                      x.contiguous(memory_format=torch.channels_last)),                        # fp32 FMA
                     (B200AutogradExtension(math_mode=L.MATH_TF32),
                      x.contiguous(memory_format=torch.channels_last))):                       # Cout % 32
        sums = []
        y = ext.conv2d(xin, w, None, 1, 1, 1, 1, 1, 1, 1, None, stats_out=sums)
        assert sums == [] and y.shape == (2, 48, 8, 8)
