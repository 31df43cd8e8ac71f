"""Benchmark-size shapes, checked on randomly sampled output elements.

The per-operator parity tests use shapes a CPU oracle finishes in seconds; the shapes the
benchmark runs (batch 256 ResNet-50 layers with up to 3.2 million pixels in a contraction,
split-K plans of dozens of splits, CTA-pair tiles with phantom halves, the strided backward-data
classes sharing a launch; the conv-ASR 13 x 1 layers; the 32000-class projection of the language
model) are checked here instead: for every operator at least 256 output elements, drawn with a
fixed seed, are recomputed as direct fp64 dot products over the same inputs (torch on the GPU
is only the checker's arithmetic) and compared with the library's TF32 and 3xTF32 results.
Bounds: error relative to the largest sampled magnitude <= 2e-3 (TF32, the per-operator bound
of tests/test_tf32_gpu.py) and <= 2e-4 (3xTF32: products carry ~21 mantissa bits, but the
accumulator in tensor memory truncates, and over the 10^4 .. 3 * 10^6 terms of these
contractions that is what remains: measured worst case 1.0e-4, ten to twenty times below
TF32 on the same shapes)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
SAMPLES = 256
TOL = {"tf32": 2e-3, "f32x3": 2e-4}


@pytest.fixture(scope="module")
def L():
    from flashlight_b200 import _lib
    if not _lib.lib.flb200_has_tensor_core_path():
        pytest.fail("tensor-core path unavailable on this device")
    return _lib


def rnd(*shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, generator=g, device="cuda")


def picks(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return [tuple(int(torch.randint(0, d, (1,), generator=g)) for d in shape) for _ in range(SAMPLES)]


def check(got, want, tol, what):
    got, want = torch.stack(got).double().cpu(), torch.stack(want).double().cpu()
    scale = float(want.abs().max()) or 1.0
    err = float((got - want).abs().max()) / scale
    print(f"sampled error {what}: {err:.2e}")
    assert err <= tol, f"{what}: sampled error {err:.3e} of the scale > {tol:.1e}"


def conv_samples(x, w, gy, stride, pad, seed):
    """Direct fp64 values of y, gx and gw at sampled positions: lists of (index, value)."""
    N, C, H, W = x.shape
    Co, _, kH, kW = w.shape
    _, _, P, Q = gy.shape
    ph, pw = pad
    sh, sw = stride
    xp = F.pad(x, (pw, pw, ph, ph))
    wd = w.double()
    ys, gxs, gws = [], [], []
    for (n, co, p, q) in picks((N, Co, P, Q), seed):
        patch = xp[n, :, p * sh:p * sh + kH, q * sw:q * sw + kW].double()
        ys.append(((n, co, p, q), (patch * wd[co]).sum()))
    for (n, ci, h, ww) in picks((N, C, H, W), seed + 1):
        acc = torch.zeros((), dtype=torch.float64, device="cuda")
        for r in range(kH):
            if (h + ph - r) % sh or not 0 <= (h + ph - r) // sh < P:
                continue
            for s in range(kW):
                if (ww + pw - s) % sw or not 0 <= (ww + pw - s) // sw < Q:
                    continue
                acc += (gy[n, :, (h + ph - r) // sh, (ww + pw - s) // sw].double() * wd[:, ci, r, s]).sum()
        gxs.append(((n, ci, h, ww), acc))
    for (co, ci, r, s) in picks((Co, C, kH, kW), seed + 2):
        win = xp[:, ci, r:r + sh * (P - 1) + 1:sh, s:s + sw * (Q - 1) + 1:sw].double()
        gws.append(((co, ci, r, s), (gy[:, co].double() * win).sum()))
    return ys, gxs, gws


# name, (N, C, H, W), Cout, (kH, kW), stride, pad, passes
CONV_SHAPES = [
    ("resnet stem 7x7/2 (backward-filter over 3.2 M pixels)", (256, 3, 224, 224), 64, (7, 7), (2, 2), (3, 3), "yw"),
    ("3x3 64->64 56x56", (256, 64, 56, 56), 64, (3, 3), (1, 1), (1, 1), "yxw"),
    ("1x1/2 256->512 downsample 56x56", (256, 256, 56, 56), 512, (1, 1), (2, 2), (0, 0), "yxw"),
    ("3x3/2 256->256 28x28 (CTA pairs, classes share a launch)", (256, 256, 28, 28), 256, (3, 3), (2, 2), (1, 1), "yxw"),
    ("1x1 1024->256 14x14", (256, 1024, 14, 14), 256, (1, 1), (1, 1), (0, 0), "yxw"),
    ("1x1 512->2048 7x7 (49-pixel planes)", (256, 512, 7, 7), 2048, (1, 1), (1, 1), (0, 0), "yxw"),
    ("conv-ASR 13x1 1024->1024, T = 1000, batch 16", (16, 1024, 1, 1000), 1024, (1, 13), (1, 1), (0, 6), "yxw"),
]


@pytest.mark.parametrize("mode", ["tf32", "f32x3"])
@pytest.mark.parametrize("layout", ["fl", "channels_last"])
@pytest.mark.parametrize("case", CONV_SHAPES, ids=[c[0] for c in CONV_SHAPES])
def test_convolutions_at_benchmark_size(L, case, layout, mode):
    from flashlight_b200.extension import AutogradPayload, B200AutogradExtension
    name, xs, Co, (kH, kW), (sh, sw), (ph, pw), passes = case
    if layout == "channels_last" and (xs[1] < 16 or xs[2] == 1):
        pytest.skip("the workloads keep this layer's input in fl order")
    ext = B200AutogradExtension(math_mode=L.MATH_BY_NAME[mode])
    x = rnd(*xs, seed=1)
    w = rnd(Co, xs[1], kH, kW, seed=2) * (1.0 / (xs[1] * kH * kW) ** 0.5)
    args = (sw, sh, pw, ph, 1, 1, 1)  # fl order: x is the W axis
    cl = (lambda t: t.contiguous(memory_format=torch.channels_last)) if layout == "channels_last" \
        else (lambda t: t)
    payload = AutogradPayload()
    before = L.lib.flb200_tc_kernel_launches()
    y = ext.conv2d(cl(x), w, None, *args, payload)
    gy = rnd(*y.shape, seed=3)
    ys, gxs, gws = conv_samples(x, w, gy, (sh, sw), (ph, pw), seed=10)
    tol = TOL[mode]
    check([y[i] for i, _ in ys], [v for _, v in ys], tol, name + " forward")
    if "x" in passes:
        gx = ext.conv2dBackwardData(cl(gy), cl(x), w, *args, None, payload)
        check([gx[i] for i, _ in gxs], [v for _, v in gxs], tol, name + " backward data")
    gw, _ = ext.conv2dBackwardFilterBias(cl(gy), cl(x), w, None, *args, None, None, payload)
    check([gw[i] for i, _ in gws], [v for _, v in gws], tol, name + " backward filter")
    torch.cuda.synchronize()
    assert L.lib.flb200_tc_kernel_launches() - before >= len(passes)


@pytest.mark.parametrize("mode", ["tf32", "f32x3"])
def test_vocabulary_projection_at_benchmark_size(L, mode):
    """fl::linear 768 -> 32000 over 4096 tokens (the language model's head): y, dx, dW."""
    from flashlight_b200 import functions as fx
    m = L.MATH_BY_NAME[mode]
    rows, I, O = 4096, 768, 32000
    x, w = rnd(rows, I, seed=4), rnd(I, O, seed=5) * (1.0 / I ** 0.5)
    gy = rnd(rows, O, seed=6)
    y = fx.linear(x, w, None, math_mode=m)
    gx, gw, _ = fx.linear_backward(x, w, gy, False, math_mode=m)
    xd, wd, gd = x.double(), w.double(), gy.double()
    tol = TOL[mode]
    p = picks((rows, O), 20)
    check([y[i] for i in p], [(xd[r] * wd[:, o]).sum() for r, o in p], tol, "head forward")
    p = picks((rows, I), 21)
    check([gx[i] for i in p], [(gd[r] * wd[i_]).sum() for r, i_ in p], tol, "head backward input")
    p = picks((I, O), 22)
    check([gw[i] for i in p], [(xd[:, i_] * gd[:, o]).sum() for i_, o in p], tol, "head backward weight")
