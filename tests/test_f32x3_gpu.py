"""F32X3 mode (three TF32 tensor-core passes per product) against the fp64 oracle.

Bound: the strict metric of tests/parity.py (element-wise relative error with a floor at 1 % of
the tensor's largest magnitude) <= 1e-3, i.e. absolute error <= 1e-5 of the tensor's scale — two
hundred times tighter than TF32 mode (2e-3 of the scale), ten times the strict fp32-FMA bound.
The products carry ~21 mantissa bits; what remains is the accumulation in tensor memory, which
truncates when aligning addends, so every one of the 3K/8 accumulator updates can lose up to one
unit in the last place, always toward zero.  Measured on these cases: 1.2e-4 .. 5.0e-4 on the
strict metric (TF32 mode on the same cases: 2.1e-2 .. 2.4e-2); results are run-to-run identical."""
import pytest
import torch

from oracle import flref as R
from tests.parity import assert_close, randn

F32X3_TOL = 1e-3

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    from flashlight_b200 import _lib
    if not _lib.lib.flb200_has_tensor_core_path():
        pytest.fail("tensor-core path unavailable on this device")
    return _lib


CASES = [
    (2, 64, 16, 16, 256, 1, 1, 1, 1, 0, 0, 1, 1, 1),    # direct 1x1
    (2, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1, 1, 1, 1),     # channels-last patch route
    (2, 128, 14, 14, 128, 3, 3, 2, 2, 1, 1, 1, 1, 1),   # strided, parity classes
    (2, 256, 14, 14, 512, 1, 1, 2, 2, 0, 0, 1, 1, 1),   # 256-column tiles (no CTA pairs in this mode)
    (2, 3, 32, 32, 64, 7, 7, 2, 2, 3, 3, 1, 1, 1),      # row-window route
    (7, 8, 9, 10, 6, 3, 4, 1, 1, 2, 1, 1, 1, 1),        # gather route
]


@pytest.mark.parametrize("case", CASES)
def test_conv2d_f32x3(L, case):
    from flashlight_b200.extension import B200AutogradExtension
    N, Cin, H, W, Cout, kH, kW, sx, sy, px, py, dx, dy, groups = case
    ext = B200AutogradExtension(math_mode=L.MATH_F32X3)
    x = randn(N, Cin, H, W, seed=21)
    w = randn(Cout, Cin, kH, kW, seed=22) * (1.0 / (Cin * kH * kW) ** 0.5)
    b = randn(Cout, seed=23)
    args = (sx, sy, px, py, dx, dy, groups)
    before = L.lib.flb200_tc_kernel_launches()
    y = ext.conv2d(x.cuda(), w.cuda(), b.cuda(), *args)
    assert L.lib.flb200_tc_kernel_launches() > before
    want = R.conv2d(x.double(), w.double(), b.double(), *args)
    assert_close(y, want, F32X3_TOL, "conv forward")
    gy = randn(*want.shape, seed=24)
    gx = ext.conv2dBackwardData(gy.cuda(), x.cuda(), w.cuda(), *args)
    assert_close(gx, R.conv2d_backward_data(gy.double(), x.shape, w.double(), *args), F32X3_TOL,
                 "conv backward data")
    gw, gb = ext.conv2dBackwardFilterBias(gy.cuda(), x.cuda(), w.cuda(), b.cuda(), *args)
    wgw, wgb = R.conv2d_backward_filter_bias(gy.double(), x.double(), w.shape, True, *args)
    assert_close(gw, wgw, F32X3_TOL, "conv backward filter")
    assert_close(gb, wgb, F32X3_TOL, "conv backward bias")


@pytest.mark.parametrize("mnk", [(256, 128, 512), (200, 72, 136), (64, 300, 4096)])
def test_matmul_f32x3(L, mnk):
    from flashlight_b200 import functions as F
    m, n, k = mnk
    a, b = randn(m, k, seed=31), randn(k, n, seed=32)
    got = F.matmul(a.cuda(), b.cuda(), m=m, n=n, k=k, a_strides=(k, 1), b_strides=(n, 1),
                   math_mode=L.MATH_F32X3)
    assert_close(got, a.double() @ b.double(), F32X3_TOL, "matmul f32x3")


def test_resnet_step_f32x3(L):
    """A scaled-down ResNet training step in F32X3 mode meets the strict-mode bounds of
    tests/test_workloads_gpu.py (loss 1e-4, every gradient within 1e-3 of its largest magnitude)."""
    from flashlight_b200 import autograd as A
    from flashlight_b200 import workloads
    from oracle import cpu_workloads as CW
    A.set_math_mode(L.MATH_F32X3)
    try:
        model = workloads.resnet50(seed=7, blocks=(1, 1, 1), classes=10, width=16)
        g = torch.Generator().manual_seed(11)
        x = torch.randn(4, 3, 112, 112, generator=g)
        t = torch.randint(0, 10, (4,), generator=g, dtype=torch.int32)
        loss = model.loss(x.cuda(), t.cuda())
        loss.backward()
    finally:
        A.set_math_mode(L.MATH_STRICT_F32)
    params = [p.tensor.detach().cpu().double() for p in model.parameters()]
    want_loss, want_grads = CW.resnet50_step(params, x.double(), t, blocks=(1, 1, 1))
    assert abs(float(loss.tensor.cpu()) - float(want_loss)) <= 1e-4 * max(1.0, abs(float(want_loss)))
    for i, (p, wg) in enumerate(zip(model.parameters(), want_grads)):
        gg = p.grad.detach().cpu().double().reshape(wg.shape)
        err = float((gg - wg).abs().max()) / (float(wg.abs().max()) or 1.0)
        assert err <= 1e-3, f"parameter {i}: {err:.3e}"
