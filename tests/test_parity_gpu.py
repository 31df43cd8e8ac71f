"""Parity of the CUDA path (through the C ABI) against the CPU oracle on seeded inputs.
Strict-fp32 mode: relative error (tests/parity.py) <= 1e-4 against the fp64 oracle."""
import pytest
import torch

from oracle import flref as R
from tests.parity import STRICT_TOL, assert_close, randint, randn, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fx():
    from flashlight_b200 import functions
    return functions


@pytest.fixture(scope="module")
def ext():
    from flashlight_b200 import _lib as L
    from flashlight_b200.extension import B200AutogradExtension
    return B200AutogradExtension(math_mode=L.MATH_STRICT_F32)


def dev(t):
    return None if t is None else t.cuda()


def f64(t):
    return None if t is None else t.double()


# ------------------------------------------------------------------ eltwise
@pytest.mark.parametrize("n", [1, 7, 4096, 1000003])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 5e-5), (torch.float16, 2e-3),
                                       (torch.bfloat16, 1.6e-2)])
def test_eltwise_gradfuncs(fx, n, dtype, tol):
    x = randn(n, seed=1, dtype=dtype)
    gy = randn(n, seed=2, dtype=dtype)
    xd, gd = x.cuda(), gy.cuda()
    x64, g64 = x.double(), gy.double()
    assert_close(fx.relu(xd), R.relu(x64), tol, "relu")
    assert_close(fx.relu_backward(xd, gd), R.relu_backward(x64, g64), tol, "relu_backward")
    assert_close(fx.gelu(xd), R.gelu(x64), tol, "gelu")
    assert_close(fx.gelu_backward(xd, gd), R.gelu_backward(x64, g64), tol, "gelu_backward")
    y = torch.tanh(x64).to(dtype)
    assert_close(fx.tanh(xd), torch.tanh(x64), tol, "tanh")
    assert_close(fx.tanh_backward(y.cuda(), gd), R.tanh_backward(y.double(), g64), tol, "tanh_backward")
    mask = (randn(n, seed=3) > 0).to(dtype)
    assert_close(fx.dropout_apply(gd, mask.cuda(), 0.5), R.dropout_apply(g64, mask.double(), 0.5),
                 tol, "dropout")
    assert_close(fx.add(xd, gd), x64 + g64, tol, "add")


def test_eltwise_unaligned_pointers_and_inplace(fx):
    base = randn(10001, seed=4).cuda()
    gbase = randn(10001, seed=5).cuda()
    x, g = base[1:], gbase[1:]  # 4-byte aligned only: takes the scalar kernels
    want = R.relu_backward(x.cpu().double(), g.cpu().double())
    assert_close(fx.relu_backward(x, g), want, 1e-6, "unaligned inputs")
    out = torch.empty(10001, device="cuda")[1:]
    from flashlight_b200 import _lib as L
    L.check(L.lib.flb200_relu_backward(x.data_ptr(), g.data_ptr(), out.data_ptr(), x.numel(), L.F32,
                                       torch.cuda.current_stream().cuda_stream))
    assert_close(out, want, 1e-6, "unaligned pointers")
    a = randn(5000, seed=6).cuda()
    b = randn(5000, seed=7).cuda()
    want = a.cpu().double() + b.cpu().double()
    fx.add(a, b, out=a)
    assert_close(a, want, 1e-6, "in-place add")


def test_relu_propagates_nan_and_handles_negative_zero(fx):
    x = torch.tensor([float("nan"), -0.0, 0.0, -1.0, 2.0], device="cuda")
    y = fx.relu(x).cpu()
    assert torch.isnan(y[0]) and y[1] == 0 and y[2] == 0 and y[3] == 0 and y[4] == 2
    g = fx.relu_backward(x, torch.ones_like(x)).cpu()
    assert g.tolist() == [0.0, 0.0, 0.0, 0.0, 1.0]


# -------------------------------------------------- channel sum / bias add
GEOS = [(8, 64, 3136), (4, 16, 49), (1, 16, 102400), (1000, 30, 1), (7, 33, 1), (3, 5, 7),
        (2, 3, 1026), (16, 2048, 49), (1, 300, 768), (5000, 1, 1), (1, 1, 5)]


@pytest.mark.parametrize("geo", GEOS)
def test_channel_sum_and_bias_add(fx, geo):
    outer, ch, inner = geo
    x = randn(outer, ch, inner, seed=8)
    want = x.double().sum(dim=(0, 2))
    assert_close(fx.channel_sum(x.cuda(), outer, ch, inner), want, STRICT_TOL, f"channel_sum {geo}")
    b = randn(ch, seed=9)
    got = fx.channel_bias_add(x.cuda(), b.cuda(), outer, ch, inner)
    assert_close(got, x.double() + b.double()[None, :, None], 1e-6, f"bias_add {geo}")


# ---------------------------------------------------------------- batchnorm
BN_CASES = [
    # torch shape, fl axes
    ((8, 64, 28, 28), [2]),        # ResNet-style spatial
    ((4, 256, 7, 7), [2]),         # inner = 49 (not a multiple of 4)
    ((3, 5, 6, 7), [2]),           # tiny, ragged
    ((2, 384, 768), [1, 2]),       # LayerNorm over fl axis 0 (transformer)
    ((4, 64, 1, 3000), [3]),       # fl [T,1,C,B] 'LN 0 1 2' -> axes {3}: few long channels
    ((16, 6, 5, 7), [0, 1, 2]),    # per-activation
    ((6, 4, 5, 3), [0, 1, 2, 3]),  # everything is a feature, outer = 1
    ((64, 10), [1]),               # fl [10, 64]: axis 1 -> 64 channels... of inner 10
]


@pytest.mark.parametrize("shape,axes", BN_CASES)
@pytest.mark.parametrize("affine", [True, False])
def test_batchnorm_forward_backward(ext, shape, axes, affine):
    x = randn(*shape, seed=10) * 1.7 + 0.4
    outer, ch, inner = R.batchnorm_geometry(tuple(reversed(shape)), axes)
    w = (randn(ch, seed=11).abs() + 0.5) if affine else None
    b = randn(ch, seed=12) if affine else None
    rm, rv = randn(ch, seed=13) * 0.1, randn(ch, seed=14).abs() + 0.5
    rm_d, rv_d = rm.cuda(), rv.cuda()
    y, sm, sv = ext.batchnorm(x.cuda(), dev(w), dev(b), rm_d, rv_d, axes, True, 0.1, 1e-5)
    wy, wm, wi, wrm, wrv = R.batchnorm(x.double(), f64(w), f64(b), rm.double(), rv.double(), axes,
                                       True, 0.1, 1e-5)
    assert_close(y, wy, STRICT_TOL, "bn y")
    assert_close(sm, wm, STRICT_TOL, "bn save_mean")
    assert_close(sv, wi, STRICT_TOL, "bn save_invstd")
    assert_close(rm_d, wrm, STRICT_TOL, "bn running_mean")
    if outer * inner > 1:
        assert_close(rv_d, wrv, STRICT_TOL, "bn running_var")
    gy = randn(*shape, seed=15)
    dx, dg, db = ext.batchnormBackward(gy.cuda(), sm, sv, x.cuda(), dev(w), axes, True, 1e-5)
    wdx, wdg, wdb = R.batchnorm_backward(gy.double(), x.double(), f64(w), axes, 1e-5)
    assert_close(dx, wdx, STRICT_TOL, "bn dx")
    assert_close(dg, wdg, STRICT_TOL, "bn dgamma")
    assert_close(db, wdb, STRICT_TOL, "bn dbeta")
    # inference path with the running statistics
    yi, _, _ = ext.batchnorm(x.cuda(), dev(w), dev(b), rm.cuda(), rv.cuda(), axes, False, 0.0, 1e-5)
    wyi, *_ = R.batchnorm(x.double(), f64(w), f64(b), rm.double(), rv.double(), axes, False, 0.0, 1e-5)
    assert_close(yi, wyi, STRICT_TOL, "bn inference")


@pytest.mark.parametrize("shape,axes", BN_CASES)
@pytest.mark.parametrize("affine", [True, False])
def test_batchnorm_relu_fused(ext, fx, shape, axes, affine):
    """relu(batchnorm(x)) as one operator: the output equals the relu kernel applied to the plain
    operator's output bit for bit, statistics are the plain operator's, and the gradients equal
    the plain batchnorm gradient of the relu-masked dy (the oracle's chain) — the predicate is
    rebuilt from x, nothing else is saved."""
    x = randn(*shape, seed=10) * 1.7 + 0.4
    ch = R.batchnorm_geometry(tuple(reversed(shape)), axes)[1]
    w = (randn(ch, seed=11).abs() + 0.5) if affine else None
    b = randn(ch, seed=12) if affine else None
    xd = x.cuda()
    y0, sm0, sv0 = ext.batchnorm(xd, dev(w), dev(b), None, None, axes, True, 0.0, 1e-5)
    y1, sm1, sv1 = ext.batchnorm(xd, dev(w), dev(b), None, None, axes, True, 0.0, 1e-5, relu=True)
    assert torch.equal(sm0, sm1) and torch.equal(sv0, sv1)
    assert torch.equal(y1, fx.relu(y0))
    gy = randn(*shape, seed=15).cuda()
    masked = fx.relu_backward(y0, gy)
    dx0, dg0, db0 = ext.batchnormBackward(masked, sm0, sv0, xd, dev(w), axes, True, 1e-5)
    dx1, dg1, db1 = ext.batchnormReluBackward(gy, sm1, sv1, xd, dev(w), dev(b), axes, True, 1e-5)
    assert torch.equal(dx0, dx1) and torch.equal(dg0, dg1) and torch.equal(db0, db1)
    # and against the fp64 oracle's chain batchnorm -> relu
    wy, *_ = R.batchnorm(x.double(), f64(w), f64(b), None, None, axes, True, 0.0, 1e-5)
    assert_close(y1, R.relu(wy), STRICT_TOL, "bn+relu y")
    # a predicate that flips between fp32 and fp64 at |y| ~ 1e-7 moves dx by one element's dy
    # over the channel size, far below the bound
    wdx, wdg, wdb = R.batchnorm_backward(R.relu_backward(wy, gy.cpu().double()), x.double(), f64(w),
                                         axes, 1e-5)
    assert_close(dx1, wdx, STRICT_TOL, "bn+relu dx")
    assert_close(dg1, wdg, STRICT_TOL, "bn+relu dgamma")
    assert_close(db1, wdb, STRICT_TOL, "bn+relu dbeta")


@pytest.mark.parametrize("shape", [(8, 64, 28, 28), (4, 32, 4, 6), (2, 16, 8, 8), (4, 32, 14, 14),
                                   (3, 8, 2, 6), (4, 16, 7, 7), (2, 5, 3, 5)])
def test_batchnorm_add_relu_fused(ext, fx, shape):
    """relu(batchnorm(x) + shortcut) in one apply pass: output and mask bit for bit equal to the
    batchnorm operator followed by the fused add + relu kernel; unsupported row lengths are
    reported so that the caller runs the operators one by one."""
    x = randn(*shape, seed=10) * 1.7 + 0.4
    s = randn(*shape, seed=17)
    ch = shape[1]
    w, b = randn(ch, seed=11).abs() + 0.5, randn(ch, seed=12)
    xd, sd = x.cuda(), s.cuda()
    assert ext.batchnormAddReluSupported(xd, sd, [2])
    y0, sm0, sv0 = ext.batchnorm(xd, w.cuda(), b.cuda(), None, None, [2], True, 0.0, 1e-5)
    want_y, want_mask = fx.add_relu_with_mask(y0, sd)
    y1, mask1, sm1, sv1 = ext.batchnormAddRelu(xd, sd, w.cuda(), b.cuda(), None, None, [2], True,
                                               0.0, 1e-5)
    assert torch.equal(y1, want_y)
    if (shape[2] * shape[3]) % 8 == 0:   # one mask byte per 8 elements: the relu kernels' layout
        assert torch.equal(mask1, want_mask)
    elif (shape[2] * shape[3]) % 4 == 0:  # one byte per 4 elements, private to the fused pair
        assert mask1.numel() == (x.numel() + 3) // 4
    else:                                 # one byte per element
        assert mask1.numel() == x.numel()
    assert torch.equal(sm0, sm1) and torch.equal(sv0, sv1)
    flat = randn(6, 4, seed=3).cuda()        # per-activation layout: run operator by operator
    assert not ext.batchnormAddReluSupported(flat, flat, [0])
    # gradient: the join's relu gradient formed inside the first batch-norm pass
    ga, gb = randn(*shape, seed=18).cuda(), randn(*shape, seed=19).cuda()
    for second in (gb, None):
        gz0 = fx.relu_backward_mask_sum(want_mask, ga, second) if second is not None else \
            fx.relu_backward_mask(want_mask, ga)
        dx0, dg0, db0 = ext.batchnormBackward(gz0, sm0, sv0, xd, w.cuda(), [2], True, 1e-5)
        gz1, dx1, dg1, db1 = ext.batchnormAddReluBackward(mask1, ga, second, sm1, sv1, xd, w.cuda(),
                                                          [2], True, 1e-5)
        assert torch.equal(gz0, gz1)
        assert_close(dx1, dx0.cpu().double(), 1e-5, "block tail dx")
        assert_close(dg1, dg0.cpu().double(), 1e-5, "block tail dgamma")
        assert_close(db1, db0.cpu().double(), 1e-5, "block tail dbeta")


def test_tape_batchnorm_add_relu_matches_operator_chain():
    """The tape's fused block tail gives the gradients of relu(add(batchnorm(x), s))."""
    from flashlight_b200 import autograd as A
    from flashlight_b200.autograd import Variable

    def run(fused, shape):
        x = Variable((randn(*shape, seed=81) * 1.3 + 0.2).cuda(), True)
        s = Variable(randn(*shape, seed=82).cuda(), True)
        w = Variable((randn(shape[1], seed=83).abs() + 0.5).cuda(), True)
        b = Variable(randn(shape[1], seed=84).cuda(), True)
        if fused:
            y = A.batchnorm_add_relu(x, s, w, b, None, None, [2], True, 0.0, 1e-5)
        else:
            y = A.relu(A.add(A.batchnorm(x, w, b, None, None, [2], True, 0.0, 1e-5), s))
        z = A.add(A.tanh(y), A.gelu(y))
        z.backward(randn(*shape, seed=85).cuda())
        return [t.clone() for t in (y.tensor, x.grad, s.grad, w.grad, b.grad)]

    for shape in [(4, 16, 8, 8), (2, 8, 6, 6), (2, 8, 7, 7)]:  # mask bytes per 8 / 4 / 1 elements
        got, want = run(True, shape), run(False, shape)
        assert torch.equal(got[0], want[0])   # y
        assert torch.equal(got[2], want[2])   # shortcut gradient: mask ? ga + gb : 0
        # the fused first pass sums the channel in a different order than the generic one
        for g, w, what in zip(got[1::2][:1] + got[3:], want[1::2][:1] + want[3:], ("dx", "dgamma", "dbeta")):
            assert_close(g, w.cpu().double(), 1e-5, f"fused block tail {what}")


def test_batchnorm_large_mean_is_well_conditioned(ext):
    x = randn(8, 32, 14, 14, seed=16) * 0.05 + 100.0
    y, sm, sv = ext.batchnorm(x.cuda(), None, None, None, None, [2], True, 0.0, 1e-5)
    wy, wm, wi, _, _ = R.batchnorm(x.double(), None, None, None, None, [2], True, 0.0, 1e-5)
    assert_close(sm, wm, 1e-6, "mean")
    assert_close(sv, wi, 1e-3, "invstd")
    assert_close(y, wy, 2e-3, "y")


def test_batchnorm_errors(ext):
    x = randn(2, 3, 4, 5, seed=1).cuda()
    with pytest.raises(ValueError):
        ext.batchnorm(x, None, None, None, None, [0, 2], True, 0.0, 1e-5)
    with pytest.raises(ValueError):
        ext.batchnorm(x, torch.ones(7, device="cuda"), None, None, None, [2], True, 0.0, 1e-5)
    with pytest.raises(RuntimeError):
        ext.batchnormBackward(x, None, None, x, None, [2], False, 1e-5)


@pytest.mark.parametrize("rows,feat", [(4096, 768), (37, 20), (5, 3), (2000, 1024)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, STRICT_TOL), (torch.bfloat16, 1.6e-2)])
def test_layernorm_affine(fx, rows, feat, dtype, tol):
    """The affine part of fl::LayerNorm (y = xhat * gamma + beta over rows of features) and its
    gradient chain as kernels; fp32 parameters with fp32 or bf16 activations."""
    xh = randn(rows, feat, seed=41, dtype=dtype)
    w, b = randn(feat, seed=42) + 1.5, randn(feat, seed=43)
    gy = randn(rows, feat, seed=44, dtype=dtype)
    y = fx.layernorm_affine(xh.cuda(), w.cuda(), b.cuda())
    assert y.dtype == dtype
    assert_close(y, xh.double() * w.double() + b.double(), tol, "layernorm affine y")
    gx, gw, gb = fx.layernorm_affine_backward(gy.cuda(), xh.cuda(), w.cuda())
    assert gw.dtype == torch.float32 and gb.dtype == torch.float32
    assert_close(gx, gy.double() * w.double(), tol, "layernorm affine dx")
    assert_close(gw, (gy.double() * xh.double()).sum(0), STRICT_TOL, "layernorm affine dgamma")
    assert_close(gb, gy.double().sum(0), STRICT_TOL, "layernorm affine dbeta")
    # only the input gradient / only the parameter gradients
    gx2, gw2, gb2 = fx.layernorm_affine_backward(gy.cuda(), xh.cuda(), w.cuda(), True, False)
    assert gw2 is None and gb2 is None and torch.equal(gx2, gx)
    gx3, gw3, _ = fx.layernorm_affine_backward(gy.cuda(), xh.cuda(), w.cuda(), False, True)
    assert gx3 is None and torch.equal(gw3, gw)


@pytest.mark.parametrize("rows,feat", [(7, 5), (33, 96), (64, 768), (5, 2048), (3, 1000)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, STRICT_TOL), (torch.bfloat16, 1.6e-2)])
@pytest.mark.parametrize("affine", [True, False])
def test_layernorm_fused(fx, rows, feat, dtype, tol, affine):
    """fl::LayerNorm over the last dimension as one operator (flb200_layernorm_forward /
    _backward) against the fp64 restatement of the reference's chain (oracle layer_norm) and its
    autograd gradient."""
    from tests.parity import assert_close_scaled
    x = (randn(rows, feat, seed=50) * 1.7 + 0.4).to(dtype)
    w = (randn(feat, seed=51) * 0.5 + 1.0) if affine else None
    b = randn(feat, seed=52) if affine else None
    gy = randn(rows, feat, seed=53).to(dtype)
    xr = x.double().requires_grad_(True)
    wr = w.double().requires_grad_(True) if affine else None
    br = b.double().requires_grad_(True) if affine else None
    want = R.layer_norm(xr, [0], 1e-5, wr, br)
    want.backward(gy.double())
    y, xhat, invstd = fx.layernorm(x.cuda(), w.cuda() if affine else None,
                                   b.cuda() if affine else None, 1e-5)
    assert y.dtype == dtype and invstd.dtype == torch.float32
    check = assert_close if dtype == torch.float32 else assert_close_scaled
    check(y.float() if dtype != torch.float32 else y, want.detach(), tol, "layernorm y")
    gx, gw, gb = fx.layernorm_backward(gy.cuda(), xhat, w.cuda() if affine else None, invstd,
                                       True, affine)
    check(gx.float() if dtype != torch.float32 else gx, xr.grad, tol, "layernorm dx")
    if affine:
        ptol = STRICT_TOL if dtype == torch.float32 else 1.6e-2
        assert_close_scaled(gw, wr.grad, ptol, "layernorm dgamma")
        assert_close_scaled(gb, br.grad, ptol, "layernorm dbeta")


def test_layernorm_fused_rejects_long_rows():
    from flashlight_b200 import _lib as L
    assert L.lib.flb200_layernorm_forward(None, None, None, None, None, None, None, 4, 4096, 1e-5,
                                          L.F32, None) == L.INVALID_ARG
    assert L.lib.flb200_layernorm_forward(None, None, None, None, None, None, None, 0, 16, 1e-5,
                                          L.F32, None) == L.OK


# ------------------------------------------------------------------- pool2d
POOL_GEOS = [(2, 2, 2, 2, 0, 0), (3, 3, 2, 2, 1, 1), (3, 2, 1, 2, 1, 0), (7, 7, 1, 1, 0, 0),
             (2, 2, 1, 1, 0, 0)]


@pytest.mark.parametrize("mode", [R.POOL_MAX, R.POOL_AVG_INCLUDE_PAD, R.POOL_AVG_EXCLUDE_PAD])
@pytest.mark.parametrize("geo", POOL_GEOS)
@pytest.mark.parametrize("with_payload", [True, False])
def test_pool2d(ext, mode, geo, with_payload):
    from flashlight_b200.extension import AutogradPayload
    wx, wy, sx, sy, px, py = geo
    x = randn(3, 5, 14, 13, seed=17)
    payload = AutogradPayload() if with_payload else None
    y = ext.pool2d(x.cuda(), wx, wy, sx, sy, px, py, mode, payload)
    want = R.pool2d(x.double(), wx, wy, sx, sy, px, py, mode)
    assert tuple(y.shape) == tuple(want.shape)
    assert_close(y, want, 1e-5, "pool forward")
    gy = randn(*want.shape, seed=18)
    gx = ext.pool2dBackward(gy.cuda(), x.cuda(), y, wx, wy, sx, sy, px, py, mode, payload)
    wgx = R.pool2d_backward(gy.double(), x.double(), wx, wy, sx, sy, px, py, mode)
    assert_close(gx, wgx, 1e-5, "pool backward")
    if mode == R.POOL_MAX and with_payload:
        _, arg = R.pool2d_naive(x.numpy(), wx, wy, sx, sy, px, py, mode)
        assert torch.equal(payload.data.argmax.cpu(), torch.from_numpy(arg))


@pytest.mark.parametrize("mode", [R.POOL_AVG_INCLUDE_PAD, R.POOL_AVG_EXCLUDE_PAD])
def test_large_average_window(ext, mode):
    """A 16x16 average window has 256 elements: more than the one-byte argmax payload of max
    pooling can index, but averages need no argmax and the reference backends accept them."""
    x = randn(2, 3, 20, 18, seed=29)
    y = ext.pool2d(x.cuda(), 16, 16, 2, 2, 1, 1, mode, None)
    want = R.pool2d(x.double(), 16, 16, 2, 2, 1, 1, mode)
    assert tuple(y.shape) == tuple(want.shape)
    assert_close(y, want, 5e-5, "16x16 average pool")  # fp32 sum of 256 values
    gy = randn(*want.shape, seed=30)
    gx = ext.pool2dBackward(gy.cuda(), x.cuda(), y, 16, 16, 2, 2, 1, 1, mode, None)
    assert_close(gx, R.pool2d_backward(gy.double(), x.double(), 16, 16, 2, 2, 1, 1, mode), 5e-5,
                 "16x16 average pool gradient")
    with pytest.raises(Exception):
        ext.pool2d(x.cuda(), 16, 16, 2, 2, 1, 1, R.POOL_MAX, None)


@pytest.mark.parametrize("mode", [R.POOL_AVG_INCLUDE_PAD, R.POOL_AVG_EXCLUDE_PAD])
def test_global_average_pool(ext, mode):
    """The ResNet head: one 7x7 window over an unpadded 7x7 plane (the gradient has a kernel of
    its own: every pixel receives dy / 49)."""
    x = randn(5, 11, 7, 7, seed=27)
    y = ext.pool2d(x.cuda(), 7, 7, 1, 1, 0, 0, mode, None)
    want = R.pool2d(x.double(), 7, 7, 1, 1, 0, 0, mode)
    assert tuple(y.shape) == (5, 11, 1, 1)
    assert_close(y, want, 1e-5, "global average pool")
    gy = randn(5, 11, 1, 1, seed=28)
    gx = ext.pool2dBackward(gy.cuda(), x.cuda(), y, 7, 7, 1, 1, 0, 0, mode, None)
    assert_close(gx, R.pool2d_backward(gy.double(), x.double(), 7, 7, 1, 1, 0, 0, mode), 1e-6,
                 "global average pool gradient")
    assert torch.equal(gx.cpu(), (gy / 49.0).expand(5, 11, 7, 7))


@pytest.mark.parametrize("geo", [(2, 2, 2, 2, 0, 0), (3, 3, 2, 2, 1, 1)])
def test_max_pool_ties_after_relu(ext, geo):
    """Half the activations are exactly zero after ReLU: ties must resolve like the oracle."""
    from flashlight_b200.extension import AutogradPayload
    wx, wy, sx, sy, px, py = geo
    x = torch.clamp_min(randn(2, 4, 12, 12, seed=19) - 0.8, 0)
    x[0, 0] = 0
    gy = randn(*R.pool2d(x, wx, wy, sx, sy, px, py, R.POOL_MAX).shape, seed=20)
    want = R.pool2d_backward(gy.double(), x.double(), wx, wy, sx, sy, px, py, R.POOL_MAX)
    for payload in (AutogradPayload(), None):
        y = ext.pool2d(x.cuda(), wx, wy, sx, sy, px, py, R.POOL_MAX, payload)
        gx = ext.pool2dBackward(gy.cuda(), x.cuda(), y, wx, wy, sx, sy, px, py, R.POOL_MAX, payload)
        # a mis-routed tie would show as an O(1) error; fp32 sums of up to four terms do not
        assert_close(gx, want, 1e-6, "max pool gradient routing")


# ------------------------------------------------------------------- conv2d
CONV_CASES = [
    # N, C, H, W, Cout, kH, kW, sx, sy, px, py, dx, dy, groups
    (7, 8, 9, 10, 6, 3, 4, 1, 1, 2, 1, 1, 1, 1),    # shape of AutogradConv2DTest.cpp:21-74
    (2, 8, 9, 10, 6, 3, 4, 1, 1, 2, 1, 1, 1, 2),    # groups (AutogradConv2DTest.cpp:137-162)
    (2, 8, 9, 10, 6, 3, 4, 1, 1, 2, 1, 2, 1, 1),    # dilation dx=2 (AutogradConv2DTest.cpp:164-213)
    (4, 1, 28, 28, 32, 5, 5, 1, 1, 2, 2, 1, 1, 1),  # MNIST conv1
    (4, 32, 14, 14, 64, 5, 5, 1, 1, 2, 2, 1, 1, 1),  # MNIST conv2
    (2, 3, 32, 32, 64, 7, 7, 2, 2, 3, 3, 1, 1, 1),  # ResNet stem (reduced image)
    (2, 64, 14, 14, 256, 1, 1, 1, 1, 0, 0, 1, 1, 1),  # bottleneck expand
    (2, 256, 14, 14, 64, 1, 1, 1, 1, 0, 0, 1, 1, 1),  # bottleneck reduce
    (2, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1, 1, 1, 1),  # bottleneck 3x3
    (2, 128, 14, 14, 128, 3, 3, 2, 2, 1, 1, 1, 1, 1),  # stride-2 3x3
    (2, 256, 14, 14, 512, 1, 1, 2, 2, 0, 0, 1, 1, 1),  # stride-2 1x1 downsample
    (2, 512, 7, 7, 2048, 1, 1, 1, 1, 0, 0, 1, 1, 1),  # 7x7 plane (49 pixels)
    (2, 80, 1, 100, 96, 1, 13, 1, 1, 6, 0, 1, 1, 1),  # conv-ASR time convolution (kW=13, kH=1)
    (1, 5, 6, 7, 3, 2, 3, 3, 2, 0, 1, 1, 2, 1),      # ragged everything
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv2d_strict(ext, case):
    N, Cin, H, W, Cout, kH, kW, sx, sy, px, py, dx, dy, groups = case
    x = randn(N, Cin, H, W, seed=21)
    w = randn(Cout, Cin // groups, kH, kW, seed=22) * (1.0 / (Cin // groups * kH * kW) ** 0.5)
    b = randn(Cout, seed=23)
    args = (sx, sy, px, py, dx, dy, groups)
    y = ext.conv2d(x.cuda(), w.cuda(), b.cuda(), *args)
    want = R.conv2d(x.double(), w.double(), b.double(), *args)
    assert tuple(y.shape) == tuple(want.shape)
    assert_close(y, want, STRICT_TOL, "conv forward")
    y_nb = ext.conv2d(x.cuda(), w.cuda(), None, *args)
    assert_close(y_nb, R.conv2d(x.double(), w.double(), None, *args), STRICT_TOL, "conv forward, no bias")
    gy = randn(*want.shape, seed=24)
    gx = ext.conv2dBackwardData(gy.cuda(), x.cuda(), w.cuda(), *args)
    assert_close(gx, R.conv2d_backward_data(gy.double(), x.shape, w.double(), *args), STRICT_TOL,
                 "conv backward data")
    gw, gb = ext.conv2dBackwardFilterBias(gy.cuda(), x.cuda(), w.cuda(), b.cuda(), *args)
    wgw, wgb = R.conv2d_backward_filter_bias(gy.double(), x.double(), w.shape, True, *args)
    assert_close(gw, wgw, STRICT_TOL, "conv backward filter")
    assert_close(gb, wgb, STRICT_TOL, "conv backward bias")
    gw2, gb2 = ext.conv2dBackwardFilterBias(gy.cuda(), x.cuda(), w.cuda(), None, *args)
    assert gb2 is None
    assert torch.equal(gw2, gw), "filter gradient must not depend on the bias argument (deterministic)"


def test_conv2d_backward_filter_split_k_is_deterministic(ext):
    """Large K (batch * pixels) takes the split-K path; two runs must agree bit for bit."""
    x = randn(16, 16, 28, 28, seed=25)
    gy = randn(16, 32, 28, 28, seed=26)
    w = randn(32, 16, 3, 3, seed=27)
    args = (1, 1, 1, 1, 1, 1, 1)
    a, _ = ext.conv2dBackwardFilterBias(gy.cuda(), x.cuda(), w.cuda(), None, *args)
    b, _ = ext.conv2dBackwardFilterBias(gy.cuda(), x.cuda(), w.cuda(), None, *args)
    assert torch.equal(a, b)
    wgw, _ = R.conv2d_backward_filter_bias(gy.double(), x.double(), w.shape, False, *args)
    assert_close(a, wgw, STRICT_TOL, "split-K filter gradient")


# ------------------------------------------------------------------- linear
@pytest.mark.parametrize("dims", [(10, 1024, 64), (1024, 3136, 64), (30, 1024, 200), (1000, 2048, 16),
                                  (7, 5, 3), (768, 768, 96), (130, 70, 257)])
def test_linear(fx, dims):
    from flashlight_b200 import _lib as L
    O, I, cols = dims
    x = randn(cols, I, seed=28)
    w = randn(I, O, seed=29) * (1.0 / I ** 0.5)
    b = randn(O, seed=30)
    y = fx.linear(x.cuda(), w.cuda(), b.cuda(), math_mode=L.MATH_STRICT_F32)
    assert_close(y, R.linear(x.double(), w.double(), b.double()), STRICT_TOL, "linear forward")
    gy = randn(cols, O, seed=31)
    gx, gw, gb = fx.linear_backward(x.cuda(), w.cuda(), gy.cuda(), True, math_mode=L.MATH_STRICT_F32)
    wx, ww, wb = R.linear_backward(x.double(), w.double(), gy.double(), True)
    assert_close(gx, wx, STRICT_TOL, "linear dx")
    assert_close(gw, ww, STRICT_TOL, "linear dW")
    assert_close(gb, wb, STRICT_TOL, "linear db")


def test_matmul_strided_batched_alpha_beta(fx):
    from flashlight_b200 import _lib as L
    a = randn(3, 37, 53, seed=32)   # batch, m, k
    b = randn(3, 29, 53, seed=33)   # batch, n, k  (B read transposed)
    c0 = randn(3, 37, 29, seed=34)
    c = c0.clone().cuda()
    fx.matmul(a.cuda(), b.cuda(), c, m=37, n=29, k=53, a_strides=(53, 1), b_strides=(1, 53),
              c_strides=(29, 1), batch=3, batch_strides=(37 * 53, 29 * 53, 37 * 29), alpha=0.5,
              beta=2.0, math_mode=L.MATH_STRICT_F32)
    want = 0.5 * a.double() @ b.double().transpose(1, 2) + 2.0 * c0.double()
    assert_close(c, want, STRICT_TOL, "matmul")


# ------------------------------------------------------- logSoftmax and CE
@pytest.mark.parametrize("C_,X", [(10, 64), (30, 1000), (1000, 37), (32000, 9), (1, 5), (1025, 3)])
def test_log_softmax_and_cross_entropy(fx, C_, X):
    x = randn(X, C_, seed=35) * 3
    y = fx.log_softmax(x.cuda())
    wy = R.log_softmax(x.double())
    assert_close(y, wy, STRICT_TOL, "logSoftmax")
    gy = randn(X, C_, seed=36)
    assert_close(fx.log_softmax_backward(y, gy.cuda()), R.log_softmax_backward(wy, gy.double()),
                 STRICT_TOL, "logSoftmax backward")
    t = randint(0, C_, X, seed=37)
    if X > 2:
        t[1] = -1  # ignored
    for red in (R.REDUCE_NONE, R.REDUCE_MEAN, R.REDUCE_SUM):
        loss, state = fx.categorical_cross_entropy(y, t.cuda(), red, -1)
        fx.check_targets(state)
        wl, denom = R.categorical_cross_entropy(wy, t, red, -1)
        assert_close(loss, wl, STRICT_TOL, f"CE loss red={red}")
        assert int(state.count[0].item()) == denom
        gl = randn(*wl.shape, seed=38).abs() + 0.1
        g = fx.categorical_cross_entropy_backward(gl.cuda(), state, C_, y)
        wg = R.categorical_cross_entropy_backward(gl.double(), wy.shape, t, red, -1, torch.float64)
        assert_close(g, wg, 1e-6, f"CE backward red={red}")
        fused = fx.log_softmax_cross_entropy_backward(y, gl.cuda(), state)
        assert_close(fused, R.log_softmax_backward(wy, wg), STRICT_TOL, f"fused backward red={red}")


def test_cross_entropy_rejects_out_of_range_target(fx):
    y = fx.log_softmax(randn(4, 5, seed=39).cuda())
    t = torch.tensor([0, 1, 5, 2], dtype=torch.int32).cuda()
    _, state = fx.categorical_cross_entropy(y, t)
    with pytest.raises(ValueError, match="out of valid range"):
        fx.check_targets(state)


# ---------------------------------------------------------------------- rnn
RNN_CASES = [
    # I, H, L, B, T, bidirectional
    (2, 2, 2, 2, 3, True),     # flashlight/fl/test/autograd/AutogradRnnTest.cpp:24-157
    (4, 3, 2, 5, 6, False),    # flashlight/fl/test/nn/ModuleTest.cpp:436-480
    (5, 16, 2, 3, 7, True),
    (80, 64, 3, 4, 9, True),   # the biLSTM workload, scaled down
]


@pytest.mark.parametrize("mode", [R.RNN_RELU, R.RNN_TANH, R.RNN_LSTM, R.RNN_GRU])
@pytest.mark.parametrize("case", RNN_CASES)
@pytest.mark.parametrize("with_state", [False, True])
def test_rnn_forward_backward(ext, mode, case, with_state):
    from flashlight_b200.extension import AutogradPayload, RNNGradData
    I, H, L_, B, T, bi = case
    dirs = 2 if bi else 1
    n = R.rnn_num_params(I, H, L_, mode, bi)
    # recurrent gain kept below one so that fp32 rounding is not amplified through time
    w = randn(n, seed=40) * (0.5 / H ** 0.5)
    x = randn(T, B, I, seed=41)
    hx = randn(L_ * dirs, B, H, seed=42) * 0.5 if with_state else None
    cx = randn(L_ * dirs, B, H, seed=43) * 0.5 if (with_state and mode == R.RNN_LSTM) else None
    payload = AutogradPayload()
    y, hy, cy = ext.rnn(x.cuda(), dev(hx), dev(cx), w.cuda(), H, L_, mode, bi, 0.0, payload)
    wy, why, wcy = R.rnn(x.double(), f64(hx), f64(cx), w.double(), H, L_, mode, bi)
    assert_close(y, wy, STRICT_TOL, "rnn y")
    assert_close(hy, why, STRICT_TOL, "rnn hy")
    if mode == R.RNN_LSTM:
        assert_close(cy, wcy, STRICT_TOL, "rnn cy")
    gy = randn(T, B, H * dirs, seed=44)
    ghy = randn(L_ * dirs, B, H, seed=45) if with_state else None
    gcy = randn(L_ * dirs, B, H, seed=46) if (with_state and mode == R.RNN_LSTM) else None
    dx, dhx, dcx, dw = ext.rnnBackward(x.cuda(), dev(hx), dev(cx), w.cuda(),
                                       RNNGradData(dev(gy), dev(ghy), dev(gcy)), y, L_, H, mode, bi,
                                       0.0, payload)
    wdx, wdhx, wdcx, wdw = R.rnn_backward(x.double(), f64(hx), f64(cx), w.double(), H, L_, mode, bi,
                                          gy.double(), f64(ghy), f64(gcy))
    assert_close(dx, wdx, STRICT_TOL, "rnn dx")
    assert_close(dw, wdw, STRICT_TOL, "rnn dw")
    if with_state:
        assert_close(dhx, wdhx, STRICT_TOL, "rnn dhx")
        if mode == R.RNN_LSTM:
            assert_close(dcx, wdcx, STRICT_TOL, "rnn dcx")


@pytest.mark.parametrize("mode", [R.RNN_TANH, R.RNN_LSTM, R.RNN_GRU])
@pytest.mark.parametrize("case", [(5, 16, 2, 3, 7, True), (80, 64, 3, 4, 9, True), (6, 8, 3, 2, 5, False)])
def test_rnn_inter_layer_dropout(ext, mode, case):
    """Inter-layer dropout (backend/cudnn/RNN.cpp:83-85) with the mask supplied as data: the
    input of every layer but the first is mask * value / (1 - p), forward and backward."""
    from flashlight_b200.extension import AutogradPayload, RNNGradData
    I, H, L_, B, T, bi = case
    dirs = 2 if bi else 1
    p = 0.3
    n = R.rnn_num_params(I, H, L_, mode, bi)
    w = randn(n, seed=60) * (0.5 / H ** 0.5)
    x = randn(T, B, I, seed=61)
    hx = randn(L_ * dirs, B, H, seed=62) * 0.5
    cx = randn(L_ * dirs, B, H, seed=63) * 0.5 if mode == R.RNN_LSTM else None
    g = torch.Generator().manual_seed(64)
    mask = (torch.rand(L_ - 1, T, B, H * dirs, generator=g) >= p).float()
    payload = AutogradPayload()
    y, hy, cy = ext.rnn(x.cuda(), hx.cuda(), dev(cx), w.cuda(), H, L_, mode, bi, p, payload,
                        dropout_mask=mask.cuda())
    wy, why, wcy = R.rnn(x.double(), hx.double(), f64(cx), w.double(), H, L_, mode, bi, p, mask)
    assert_close(y, wy, STRICT_TOL, "rnn y (dropout)")
    assert_close(hy, why, STRICT_TOL, "rnn hy (dropout)")
    # and it is not the same function as without dropout
    y0, _, _ = ext.rnn(x.cuda(), hx.cuda(), dev(cx), w.cuda(), H, L_, mode, bi, 0.0, None)
    assert (y0 - y).abs().max() > 1e-3
    gy = randn(T, B, H * dirs, seed=65)
    ghy = randn(L_ * dirs, B, H, seed=66)
    dx, dhx, dcx, dw = ext.rnnBackward(x.cuda(), hx.cuda(), dev(cx), w.cuda(),
                                       RNNGradData(gy.cuda(), ghy.cuda(), None), y, L_, H, mode, bi,
                                       p, payload)
    wdx, wdhx, wdcx, wdw = R.rnn_backward(x.double(), hx.double(), f64(cx), w.double(), H, L_, mode,
                                          bi, gy.double(), ghy.double(), None, p, mask)
    assert_close(dx, wdx, STRICT_TOL, "rnn dx (dropout)")
    assert_close(dhx, wdhx, STRICT_TOL, "rnn dhx (dropout)")
    assert_close(dw, wdw, STRICT_TOL, "rnn dw (dropout)")
    if mode == R.RNN_LSTM:
        assert_close(dcx, wdcx, STRICT_TOL, "rnn dcx (dropout)")


def test_rnn_dropout_draws_its_own_mask(ext):
    """Without a supplied mask the extension draws one (kept in the payload for the backward
    pass); two calls use different parts of the random stream."""
    from flashlight_b200.extension import AutogradPayload, RNNGradData
    I, H, L_, B, T = 6, 32, 2, 4, 8
    w = randn(R.rnn_num_params(I, H, L_, R.RNN_LSTM, True), seed=67) * 0.1
    x = randn(T, B, I, seed=68)
    pa, pb = AutogradPayload(), AutogradPayload()
    ya, _, _ = ext.rnn(x.cuda(), None, None, w.cuda(), H, L_, R.RNN_LSTM, True, 0.5, pa)
    yb, _, _ = ext.rnn(x.cuda(), None, None, w.cuda(), H, L_, R.RNN_LSTM, True, 0.5, pb)
    ma, mb = pa.data.dropout_mask, pb.data.dropout_mask
    assert ma.shape == (1, T, B, 2 * H) and set(ma.unique().tolist()) <= {0.0, 1.0}
    assert 0.35 < ma.mean().item() < 0.65 and not torch.equal(ma, mb)
    assert (ya - yb).abs().max() > 1e-4
    wy, _, _ = R.rnn(x.double(), None, None, w.double(), H, L_, R.RNN_LSTM, True, 0.5, ma.cpu())
    assert_close(ya, wy, STRICT_TOL, "rnn y (own mask)")
    gy = randn(T, B, 2 * H, seed=69)
    dx, _, _, dw = ext.rnnBackward(x.cuda(), None, None, w.cuda(), RNNGradData(gy.cuda(), None, None),
                                   ya, L_, H, R.RNN_LSTM, True, 0.5, pa)
    wdx, _, _, wdw = R.rnn_backward(x.double(), None, None, w.double(), H, L_, R.RNN_LSTM, True,
                                    gy.double(), None, None, 0.5, ma.cpu())
    assert_close(dx, wdx, STRICT_TOL, "rnn dx (own mask)")
    assert_close(dw, wdw, STRICT_TOL, "rnn dw (own mask)")
    with pytest.raises(ValueError):
        ext.rnn(x.cuda(), None, None, w.cuda(), H, L_, R.RNN_LSTM, True, 1.0, None)


def test_bernoulli_mask_is_a_pure_function_of_seed_and_counter():
    from flashlight_b200.extension import bernoulli_mask
    a = bernoulli_mask((1000003,), 0.8, "cuda", seed=7, offset=100)
    b = bernoulli_mask((1000003,), 0.8, "cuda", seed=7, offset=100)
    c = bernoulli_mask((1000003,), 0.8, "cuda", seed=8, offset=100)
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert abs(a.mean().item() - 0.8) < 2e-3
    # a mask drawn in two pieces (counter advanced by the elements / 4 of the first) is the same
    d = bernoulli_mask((400,), 0.8, "cuda", seed=7, offset=100)
    e = bernoulli_mask((600,), 0.8, "cuda", seed=7, offset=200)
    assert torch.equal(torch.cat([d, e]), a[:1000])
    # neighbouring bits are not correlated
    ac = ((a[1:] - 0.8) * (a[:-1] - 0.8)).mean().item()
    assert abs(ac) < 1e-3
    h = bernoulli_mask((4096,), 0.5, "cuda", dtype=torch.bfloat16, seed=1, offset=0)
    f = bernoulli_mask((4096,), 0.5, "cuda", seed=1, offset=0)
    assert torch.equal(h.float(), f)
    assert bernoulli_mask((0,), 0.5, "cuda").numel() == 0


def test_dropout_module_with_device_masks():
    """nn.Dropout without a host generator draws its mask on the device: outputs are 0 or
    x / (1 - p), about 1 - p of them kept, the gradient passes through the same mask, eval mode
    is the identity, and the step can be captured as a CUDA graph (no host-to-device copy)."""
    from flashlight_b200 import autograd as A, nn
    m = nn.Dropout(0.25)
    x = A.Variable(torch.full((64, 1024), 2.0, device="cuda"), True)
    y = m.forward(x)
    kept = y.tensor != 0
    assert torch.allclose(y.tensor[kept], torch.full_like(y.tensor[kept], 2.0 / 0.75))
    assert abs(kept.float().mean().item() - 0.75) < 0.01
    y.backward(torch.ones_like(y.tensor))
    assert torch.equal(x.grad != 0, kept)
    assert torch.allclose(x.grad[kept], torch.full_like(x.grad[kept], 1.0 / 0.75))
    m.train(False)
    assert m.forward(x) is x
    m.train(True)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        m.forward(x)
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(g):
        z = m.forward(x)
    g.replay()
    torch.cuda.synchronize()
    assert abs((z.tensor != 0).float().mean().item() - 0.75) < 0.01


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", [
    ((2, 5, 3, 4, 64), (2, 0, 3, 1, 4)),    # packed q, k, v to heads-first
    ((3, 2, 4, 5, 64), (1, 3, 0, 2, 4)),    # and back
    ((3, 4, 7, 32), (0, 2, 1, 3)),          # head merge
    ((6, 9, 8), (1, 0, 2)),                 # three indices, the shortest run (fp32: two vectors)
    ((5, 40), (0, 1)),                      # identity
])
def test_reorder_matches_permute(fx, case, dtype):
    """flb200_reorder against torch's permute copy: bit-exact data movement."""
    shape, perm = case
    x = randn(*shape, seed=91).to(dtype).cuda()
    got = fx.reorder(x, shape, perm)
    assert got is not None and got.is_contiguous()
    assert torch.equal(got, x.permute(perm).contiguous())
    # what the kernel is not built for is declined, not mis-copied
    odd = randn(4, 6, 3, seed=92).to(dtype).cuda()
    assert fx.reorder(odd, (4, 6, 3), (1, 0, 2)) is None  # runs of 3 elements: not whole vectors


@pytest.mark.parametrize("n", [1, 7, 4096, 1000003])
@pytest.mark.parametrize("half", [torch.bfloat16, torch.float16])
def test_astype_matches_torch(fx, n, half):
    """flb200_astype against torch's conversion (round to nearest even), both directions, lengths
    that are not multiples of the vector width, and a view that starts off a 16-byte boundary."""
    x = (randn(n + 3, seed=93) * 3).cuda()
    for src in (x[:n], x[3:3 + n].contiguous(), x[1:1 + n]):
        down = fx.astype(src, half)
        assert down is not None and torch.equal(down, src.to(half))
        up = fx.astype(down, torch.float32)
        assert torch.equal(up, down.float())
    assert torch.equal(fx.astype(x, torch.float32), x)
    assert fx.astype(x.to(half), torch.float16 if half == torch.bfloat16 else torch.bfloat16) is None


def test_rnn_backward_without_output_gradient(ext):
    """dy absent counts as zeros (backend/cudnn/RNN.cpp:269-272): only dhy drives the gradient."""
    from flashlight_b200.extension import AutogradPayload, RNNGradData
    I, H, L_, B, T = 3, 4, 1, 2, 4
    w = randn(R.rnn_num_params(I, H, L_, R.RNN_LSTM, False), seed=47) * 0.5
    x = randn(T, B, I, seed=48)
    payload = AutogradPayload()
    y, hy, cy = ext.rnn(x.cuda(), None, None, w.cuda(), H, L_, R.RNN_LSTM, False, 0.0, payload)
    ghy = randn(L_, B, H, seed=49)
    dx, _, _, dw = ext.rnnBackward(x.cuda(), None, None, w.cuda(), RNNGradData(None, ghy.cuda(), None),
                                   y, L_, H, R.RNN_LSTM, False, 0.0, payload)
    wdx, _, _, wdw = R.rnn_backward(x.double(), None, None, w.double(), H, L_, R.RNN_LSTM, False, None,
                                    ghy.double(), None)
    assert_close(dx, wdx, STRICT_TOL, "dx")
    assert_close(dw, wdw, STRICT_TOL, "dw")
    with pytest.raises(ValueError):
        ext.rnnBackward(x.cuda(), None, None, w.cuda(), RNNGradData(), y, L_, H, R.RNN_LSTM, False, 0.0,
                        None)


@pytest.mark.parametrize("n", [1, 7, 8, 9, 1000, 4096 + 5, 3 * 1024 * 1024 + 3])
def test_relu_bit_mask(fx, n):
    """relu with the x > 0 predicate packed 8 per byte: same y as the plain kernel, the mask
    bits equal the predicate, and the masked gradient equals (x > 0) * dy bit for bit — also for
    NaN (propagates through y, no gradient), negative zero and ragged tails."""
    x = randn(n, seed=51)
    if n >= 9:
        x[3], x[4], x[5] = float("nan"), -0.0, 0.0
    g = randn(n, seed=52)
    xd, gd = x.cuda(), g.cuda()
    y, mask = fx.relu_with_mask(xd)
    assert torch.equal(torch.nan_to_num(y, nan=123.0), torch.nan_to_num(fx.relu(xd), nan=123.0))
    bits = (x > 0).to(torch.uint8)
    bits = torch.cat([bits, torch.zeros((-n) % 8, dtype=torch.uint8)]).reshape(-1, 8)
    want_mask = (bits * (2 ** torch.arange(8, dtype=torch.uint8))).sum(1).to(torch.uint8)
    assert torch.equal(mask.cpu(), want_mask)
    gx = fx.relu_backward_mask(mask, gd)
    assert torch.equal(gx.cpu(), torch.where(x > 0, g, torch.zeros_like(g)))


@pytest.mark.parametrize("n", [1, 7, 8, 9, 1000, 4096 + 5, 3 * 1024 * 1024 + 3])
def test_add_relu_bit_mask(fx, n):
    """The fused residual join: y = relu(a + b) and its mask bit for bit equal to the add kernel
    followed by the relu kernel; the two-addend gradient equals mask * (ga + gb) computed with
    the add kernel first.  NaN in either addend propagates, ragged tails included."""
    a, b = randn(n, seed=53), randn(n, seed=54)
    if n >= 9:
        a[3], b[4], a[5], b[5] = float("nan"), float("nan"), 1.5, -1.5
    ga, gb = randn(n, seed=55), randn(n, seed=56)
    ad, bd = a.cuda(), b.cuda()
    y, mask = fx.add_relu_with_mask(ad, bd)
    y_ref, mask_ref = fx.relu_with_mask(fx.add(ad, bd))
    assert torch.equal(torch.nan_to_num(y, nan=123.0), torch.nan_to_num(y_ref, nan=123.0))
    assert torch.equal(mask, mask_ref)
    assert torch.equal(torch.nan_to_num(y.cpu(), nan=123.0),
                       torch.nan_to_num(torch.relu(a + b), nan=123.0))
    gx = fx.relu_backward_mask_sum(mask, ga.cuda(), gb.cuda())
    assert torch.equal(gx, fx.relu_backward_mask(mask, fx.add(ga.cuda(), gb.cuda())))
    assert torch.equal(gx.cpu(), torch.where((a + b) > 0, ga + gb, torch.zeros_like(ga)))


def test_tape_fused_residual_join_matches_operator_chain():
    """autograd.add_relu (one kernel each way, two-consumer gradients summed inside it) gives
    the same output and the same input gradients, bit for bit, as relu(add(a, b)) with the
    tape's whole-tensor gradient accumulation."""
    from flashlight_b200 import autograd as A
    from flashlight_b200.autograd import Variable

    def run(fused):
        a = Variable(randn(4, 8, 6, 6, seed=71).cuda(), True)
        b = Variable(randn(4, 8, 6, 6, seed=72).cuda(), True)
        y = A.add_relu(a, b) if fused else A.relu(A.add(a, b))
        # two consumers of y, then a third so that every accumulation path is walked
        z = A.add(A.tanh(y), A.gelu(y))
        z = A.add(z, y)
        z.backward(randn(4, 8, 6, 6, seed=73).cuda())
        return y.tensor.clone(), a.grad.clone(), b.grad.clone()

    y0, ga0, gb0 = run(False)
    y1, ga1, gb1 = run(True)
    assert torch.equal(y0, y1)
    # the fused path sums three contributions in a different association order
    assert_close(ga1, ga0.cpu().double(), 1e-6, "fused residual join: grad a")
    assert_close(gb1, gb0.cpu().double(), 1e-6, "fused residual join: grad b")

    def run2(fused):
        a = Variable(randn(4, 8, 6, 6, seed=71).cuda(), True)
        b = Variable(randn(4, 8, 6, 6, seed=72).cuda(), True)
        y = A.add_relu(a, b) if fused else A.relu(A.add(a, b))
        z = A.add(A.tanh(y), A.gelu(y))  # exactly two consumers: the in-kernel sum
        z.backward(randn(4, 8, 6, 6, seed=73).cuda())
        return a.grad.clone()

    assert torch.equal(run2(False), run2(True))


@pytest.mark.parametrize("cfg", [
    (0.1, 0.9, 0.1, False, 1.0),      # the reference benchmark's setting
    (0.05, 0.9, 0.0, True, 0.125),    # Nesterov, gradient averaged over 8 ranks
    (0.01, 0.0, 0.01, False, 1.0),    # no momentum: no velocity buffer
])
@pytest.mark.parametrize("n", [1, 1023, 4096 + 3, 2_000_003])
def test_sgd_step(cfg, n):
    """Fused SGD step against the reference's update rule, three steps in a row."""
    from flashlight_b200.autograd import Variable
    from flashlight_b200.optim import SGDOptimizer
    lr, mu, wd, nesterov, scale = cfg
    p0 = randn(n, seed=61)
    param = Variable(p0.clone().cuda(), True)
    opt = SGDOptimizer([param], lr, mu, wd, nesterov)
    want_p, want_v = p0.double(), torch.zeros(n, dtype=torch.float64)
    for it in range(3):
        g = randn(n, seed=62 + it)
        param.grad = g.clone().cuda()
        opt.step(grad_scale=scale, zero_grad=(it == 2))
        want_p, want_v = R.sgd_step(want_p, g.double(), want_v, lr, mu, wd, nesterov, scale)
    assert_close(param.tensor, want_p, 1e-5, "sgd parameter")
    if mu != 0:
        assert_close(opt.velocities[0], want_v, 1e-5, "sgd velocity")
    assert float(param.grad.abs().max()) == 0.0  # cleared by the last step


@pytest.mark.parametrize("case", [
    (97, 64, 72, torch.int64, torch.float32),       # toy vocabulary, repeated ids
    (1000, 768, 513, torch.int32, torch.float32),   # dim of the transformer workload
    (50, 1100, 40, torch.int64, torch.float32),     # dim > 1024: two column chunks
    (300, 96, 700, torch.int64, torch.bfloat16),    # bf16 activations, f32 table gradient
])
def test_embedding(fx, case):
    """Row gather and its scatter-add gradient (no atomics: two runs are bit-identical)."""
    vocab, dim, rows, itype, dtype = case
    g = torch.Generator().manual_seed(71)
    table = randn(vocab, dim, seed=72).to(dtype)
    ids = torch.randint(0, vocab, (rows,), generator=g).to(itype)
    ids[: rows // 3] = ids[0]  # one heavily repeated id
    out = fx.embedding(table.cuda(), ids.cuda())
    assert torch.equal(out.cpu(), table[ids.long()])
    gy = randn(rows, dim, seed=73).to(dtype)
    got = fx.embedding_backward(gy.cuda(), ids.cuda(), vocab)
    again = fx.embedding_backward(gy.cuda(), ids.cuda(), vocab)
    assert got.dtype == torch.float32 and torch.equal(got, again)
    want = torch.zeros(vocab, dim, dtype=torch.float64).index_add_(0, ids.long(), gy.double())
    assert_close(got, want, 1e-5, "embedding gradient")


@pytest.mark.parametrize("case", [
    (24, 24, 3, True, torch.float32),      # toy attention block, causal
    (512, 512, 2, True, torch.float32),    # the transformer workload's row length
    (100, 37, 1, False, torch.float32),    # ragged, no mask
    (1500, 64, 1, False, torch.float32),   # > 1024 columns
    (128, 128, 2, True, torch.bfloat16),
])
def test_attention_softmax(fx, case):
    """Scaled softmax with the causal mask folded in, and its gradient, against fp64."""
    cols, T, nmat, causal, dtype = case
    rows = T * nmat
    x = randn(rows, cols, seed=81).to(dtype)
    gy = randn(rows, cols, seed=82).to(dtype)
    scale = 0.37
    z = x.double() * scale
    if causal:
        r = torch.arange(rows).remainder(T)[:, None]
        z = z.masked_fill(torch.arange(cols)[None, :] > r, float("-inf"))
    want = torch.softmax(z, -1)
    y = fx.softmax(x.cuda(), scale, T if causal else 0)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert_close(y.float(), want, tol, "softmax")
    if causal:
        assert float(y.float().cpu().masked_select(torch.arange(cols)[None, :] > r).abs().max()) == 0.0
    yd = y.double().cpu()
    want_dx = scale * yd * (gy.double() - (gy.double() * yd).sum(-1, keepdim=True))
    dx = fx.softmax_backward(y, gy.cuda(), scale)
    assert_close(dx.float(), want_dx, tol, "softmax gradient")
