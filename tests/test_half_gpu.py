"""f16 / bf16 tensors through convolution, pooling and batch-norm.

The reference accepts f16 for these operators (backend/cudnn/CudnnAutogradExtension.cpp:27-36,
backend/cudnn/Conv2D.cpp:231,266,321, backend/cudnn/BatchNorm.cpp:92-95: f16 activations with f32
parameters; its test is flashlight/fl/test/autograd/AutogradConv2DTest.cpp:76-135).  Here every
operand is rounded to the 16-bit type first, the oracle computes in fp64 from those rounded values,
and the result may differ by the rounding of the output (2^-11 relative for f16, 2^-8 for bf16)
plus, in TF32 mode, the TF32 bound."""
import pytest
import torch

from oracle import flref as R
from tests.parity import assert_close_scaled, randn

pytestmark = pytest.mark.gpu

TOL = {torch.float16: 3e-3, torch.bfloat16: 1.6e-2}


@pytest.fixture(scope="module")
def L():
    from flashlight_b200 import _lib
    return _lib


def ext_for(L, math):
    from flashlight_b200.extension import B200AutogradExtension
    return B200AutogradExtension(math_mode=L.MATH_BY_NAME[math])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("math", ["strict", "tf32"])
@pytest.mark.parametrize("case", [
    (4, 32, 14, 14, 64, 3, 1, 1, 1, False),
    (4, 32, 14, 14, 64, 3, 1, 1, 1, True),     # channels-last
    (3, 64, 9, 9, 128, 1, 1, 0, 1, True),      # 1 x 1, the GEMM route
    (2, 8, 11, 7, 12, 3, 2, 1, 2, False),      # groups, strided, odd sizes
])
def test_conv2d_16bit(L, dtype, math, case):
    N, Cc, H, W, Co, k, s, p, groups, cl = case
    ext = ext_for(L, math)
    x = randn(N, Cc, H, W, seed=80).to(dtype)
    w = (randn(Co, Cc // groups, k, k, seed=81) * (1.0 / (Cc // groups * k * k) ** 0.5)).to(dtype)
    b = randn(Co, seed=82).to(dtype)
    args = (s, s, p, p, 1, 1, groups)
    xd = x.cuda().contiguous(memory_format=torch.channels_last) if cl else x.cuda()
    y = ext.conv2d(xd, w.cuda(), b.cuda(), *args)
    assert y.dtype == dtype and y.shape[1] == Co
    want = R.conv2d(x.double(), w.double(), b.double(), *args)
    tol = TOL[dtype]
    assert_close_scaled(y.float(), want, tol, f"conv2d {dtype}")
    gy = randn(*y.shape, seed=83).to(dtype)
    gyd = gy.cuda().contiguous(memory_format=torch.channels_last) if cl else gy.cuda()
    gx = ext.conv2dBackwardData(gyd, xd, w.cuda(), *args)
    gw, gb = ext.conv2dBackwardFilterBias(gyd, xd, w.cuda(), b.cuda(), *args)
    assert gx.dtype == dtype and gw.dtype == dtype and gb.dtype == dtype
    assert_close_scaled(gx.float(), R.conv2d_backward_data(gy.double(), x.shape, w.double(), *args),
                        tol, f"conv2dBackwardData {dtype}")
    wgw, wgb = R.conv2d_backward_filter_bias(gy.double(), x.double(), w.shape, True, *args)
    assert_close_scaled(gw.float(), wgw, tol, f"conv2dBackwardFilterBias dw {dtype}")
    assert_close_scaled(gb.float(), wgb, tol, f"conv2dBackwardFilterBias db {dtype}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("mode", [R.POOL_MAX, R.POOL_AVG_INCLUDE_PAD, R.POOL_AVG_EXCLUDE_PAD])
@pytest.mark.parametrize("cl", [False, True])
def test_pool2d_16bit(L, dtype, mode, cl):
    from flashlight_b200.extension import AutogradPayload
    ext = ext_for(L, "strict")
    x = randn(3, 16, 13, 12, seed=84).to(dtype)
    xd = x.cuda().contiguous(memory_format=torch.channels_last) if cl else x.cuda()
    payload = AutogradPayload()
    y = ext.pool2d(xd, 3, 3, 2, 2, 1, 1, mode, payload)
    want = R.pool2d(x.double(), 3, 3, 2, 2, 1, 1, mode)
    assert y.dtype == dtype
    assert_close_scaled(y.float(), want, TOL[dtype], f"pool2d {dtype}")
    gy = randn(*y.shape, seed=85).to(dtype)
    gyd = gy.cuda().contiguous(memory_format=torch.channels_last) if cl else gy.cuda()
    gx = ext.pool2dBackward(gyd, xd, y, 3, 3, 2, 2, 1, 1, mode, payload)
    wgx = R.pool2d_backward(gy.double(), x.double(), 3, 3, 2, 2, 1, 1, mode)
    assert_close_scaled(gx.float(), wgx, TOL[dtype], f"pool2dBackward {dtype}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cl", [False, True])
def test_batchnorm_16bit_activations_fp32_parameters(L, dtype, cl):
    ext = ext_for(L, "strict")
    N, Cc, H, W = 6, 24, 9, 10
    x = (randn(N, Cc, H, W, seed=86) * 1.5 + 0.3).to(dtype)
    gamma, beta = randn(Cc, seed=87) * 0.5 + 1.0, randn(Cc, seed=88)
    xd = x.cuda().contiguous(memory_format=torch.channels_last) if cl else x.cuda()
    rm, rv = torch.zeros(Cc).cuda(), torch.ones(Cc).cuda()
    y, sm, sv = ext.batchnorm(xd, gamma.cuda(), beta.cuda(), rm, rv, [2], True, 0.1, 1e-5)
    assert y.dtype == dtype and sm.dtype == torch.float32
    wy, wm, winv, _, _ = R.batchnorm(x.double(), gamma.double(), beta.double(), None, None, [2], True,
                                     0.1, 1e-5)
    assert_close_scaled(y.float(), wy, TOL[dtype], f"batchnorm {dtype}")
    assert_close_scaled(sm, wm, 1e-4, "saved mean")
    gy = randn(N, Cc, H, W, seed=89).to(dtype)
    gyd = gy.cuda().contiguous(memory_format=torch.channels_last) if cl else gy.cuda()
    gx, gg, gb = ext.batchnormBackward(gyd, sm, sv, xd, gamma.cuda(), [2], True, 1e-5)
    wgx, wgg, wgb = R.batchnorm_backward(gy.double(), x.double(), gamma.double(), [2], 1e-5)
    assert gx.dtype == dtype and gg.dtype == torch.float32
    assert_close_scaled(gx.float(), wgx, TOL[dtype], f"batchnormBackward dx {dtype}")
    assert_close_scaled(gg, wgg, 1e-3, "dgamma")
    assert_close_scaled(gb, wgb, 1e-3, "dbeta")


def test_16bit_types_are_reported_supported():
    from flashlight_b200.extension import B200AutogradExtension
    ext = B200AutogradExtension()
    assert all(ext.isDataTypeSupported(t) for t in (torch.float32, torch.float16, torch.bfloat16))
    assert not ext.isDataTypeSupported(torch.float64)
