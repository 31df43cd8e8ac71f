"""B200AutogradExtension running behind real fl::Tensor objects.

flashlight_b200/csrc/fl/libflb200_fl.so holds the C++ extension class, a minimal device tensor
(B200Tensor / B200Backend in the reference's `Stub` backend slot) and the reference's own
tensor, runtime and autograd-dispatch sources compiled in place from the flashlight checkout
(build_harness.py).  Its extern "C" calls take host buffers, wrap them as fl::Tensor and call
fl::detail::conv2d / ... / rnnBackward, so everything between fl::Tensor and the kernels —
registration, TensorBackend::getExtension, fl::DevicePtr, fl::relativeSync across the tensor's
and the extension's streams, payloads, output allocation — executes on the GPU.  Results are
compared with the committed golden vectors (fp64 oracle) at the strict-mode bound.

The library is built where the checkout is present and travels with the repository to machines
that have a GPU but no checkout; with neither, the tests are skipped."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.parity import STRICT_TOL, assert_close
from tests.test_golden import load

FL_DIR = Path(__file__).resolve().parent.parent / "flashlight_b200" / "csrc" / "fl"
f32p, i32p, vp = C.POINTER(C.c_float), C.POINTER(C.c_int), C.c_void_p


def _built_library():
    import importlib.util
    spec = importlib.util.spec_from_file_location("build_harness", FL_DIR / "build_harness.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build()


@pytest.fixture(scope="module")
def H():
    lib_path = _built_library()
    if lib_path is None or not Path(lib_path).exists():
        pytest.skip("libflb200_fl.so is not built and the flashlight checkout is not present")
    from flashlight_b200 import _lib  # noqa: F401  (loads libflb200.so first)
    lib = C.CDLL(str(lib_path))
    lib.flb200_fl_last_error.restype = C.c_char_p
    lib.flb200_fl_payload_new.restype = vp
    lib.flb200_fl_payload_free.argtypes = [vp]
    return lib


def test_harness_library_exports_the_shim():
    """CPU-side check (no GPU call): the library loads and exports every shim entry."""
    lib_path = _built_library()
    if lib_path is None or not Path(lib_path).exists():
        pytest.skip("libflb200_fl.so is not built and the flashlight checkout is not present")
    from flashlight_b200 import _lib  # noqa: F401
    lib = C.CDLL(str(lib_path))
    for name in ("init", "registered", "last_error", "payload_new", "payload_free", "conv2d",
                 "conv2d_backward_data", "conv2d_backward_filter_bias", "pool2d", "pool2d_backward",
                 "batchnorm", "batchnorm_backward", "rnn", "rnn_backward", "distributed_init",
                 "world_rank", "world_size", "all_reduce", "all_reduce_multiple", "benchmark_new",
                 "benchmark_free", "benchmark_mode", "benchmark_state", "conv2d_backward_tuned",
                 "half_chain"):
        assert hasattr(lib, "flb200_fl_" + name), name


def arr(t):
    return None if t is None else np.ascontiguousarray(t.detach().cpu().numpy(), dtype=np.float32)


def ptr(a):
    return None if a is None else a.ctypes.data_as(f32p)


def ok(lib, rc):
    assert rc == 0, lib.flb200_fl_last_error().decode()


@pytest.mark.gpu
def test_extension_is_registered_for_fl_tensors(H):
    ok(H, H.flb200_fl_init())
    assert H.flb200_fl_registered() == 1, H.flb200_fl_last_error().decode()


@pytest.mark.gpu
@pytest.mark.parametrize("with_payload", [True, False])
def test_conv2d_through_fl_tensors(H, with_payload):
    ok(H, H.flb200_fl_init())
    c = load("conv")
    sx, sy, px, py, dx, dy, groups = (int(v) for v in c["args"])
    x, w, b, gy = arr(c["x"]), arr(c["w"]), arr(c["b"]), arr(c["gy"])
    N, Cin, Hh, W = x.shape
    Cout, _, kH, kW = w.shape
    _, _, Ho, Wo = gy.shape
    geo = (W, Hh, Cin, N, kW, kH, Cout, Wo, Ho, sx, sy, px, py, dx, dy, groups)
    pl = H.flb200_fl_payload_new() if with_payload else None
    y = np.empty_like(gy)
    ok(H, H.flb200_fl_conv2d(ptr(x), ptr(w), ptr(b), ptr(y), *geo, vp(pl)))
    assert_close(torch.from_numpy(y), c["y"], STRICT_TOL, "fl conv2d")
    gx = np.empty_like(x)
    ok(H, H.flb200_fl_conv2d_backward_data(ptr(gy), ptr(x), ptr(w), ptr(gx), *geo, vp(pl)))
    assert_close(torch.from_numpy(gx), c["gx"], STRICT_TOL, "fl conv2dBackwardData")
    gw, gb = np.empty_like(w), np.empty_like(b)
    ok(H, H.flb200_fl_conv2d_backward_filter_bias(ptr(gy), ptr(x), ptr(w), ptr(b), ptr(gw), ptr(gb),
                                                  *geo, vp(pl)))
    assert_close(torch.from_numpy(gw), c["gw"], STRICT_TOL, "fl conv2dBackwardFilterBias dw")
    assert_close(torch.from_numpy(gb), c["gb"], STRICT_TOL, "fl conv2dBackwardFilterBias db")
    # no bias: the bias gradient is skipped (an empty tensor comes back)
    ok(H, H.flb200_fl_conv2d_backward_filter_bias(ptr(gy), ptr(x), ptr(w), None, ptr(gw), None, *geo,
                                                  vp(pl)))
    assert_close(torch.from_numpy(gw), c["gw"], STRICT_TOL, "fl conv2dBackwardFilterBias dw, no bias")
    if pl:
        H.flb200_fl_payload_free(vp(pl))


@pytest.mark.gpu
def test_conv2d_tensor_core_routes_through_fl_tensors(H, monkeypatch):
    """A shape that takes the channels-last patch route with its per-call-site layout cache
    (payload), driven through fl::Tensor: forward, backward-data and backward-filter share the
    payload the way fl::conv2d's gradFunc does.  The extension reads the math mode once, so
    this runs in whatever mode the process started with; the bound is the looser TF32 one."""
    from oracle import flref as R
    from tests.parity import TF32_SCALED_TOL, assert_close_scaled, randn
    ok(H, H.flb200_fl_init())
    x, w = randn(2, 64, 14, 14, seed=1), randn(64, 64, 3, 3, seed=2) * (1.0 / 24.0)
    args = (1, 1, 1, 1, 1, 1, 1)
    want = R.conv2d(x.double(), w.double(), None, *args)
    gy = randn(*want.shape, seed=3)
    xa, wa, gya = arr(x), arr(w), arr(gy)
    geo = (14, 14, 64, 2, 3, 3, 64, 14, 14, *args)
    pl = H.flb200_fl_payload_new()
    y, gx, gw = np.empty_like(gya), np.empty_like(xa), np.empty_like(wa)
    ok(H, H.flb200_fl_conv2d(ptr(xa), ptr(wa), None, ptr(y), *geo, vp(pl)))
    ok(H, H.flb200_fl_conv2d_backward_data(ptr(gya), ptr(xa), ptr(wa), ptr(gx), *geo, vp(pl)))
    ok(H, H.flb200_fl_conv2d_backward_filter_bias(ptr(gya), ptr(xa), ptr(wa), None, ptr(gw), None,
                                                  *geo, vp(pl)))
    H.flb200_fl_payload_free(vp(pl))
    assert_close_scaled(torch.from_numpy(y), want, TF32_SCALED_TOL, "fl conv2d 3x3")
    assert_close_scaled(torch.from_numpy(gx), R.conv2d_backward_data(gy.double(), x.shape, w.double(), *args),
                        TF32_SCALED_TOL, "fl conv2dBackwardData 3x3")
    wgw, _ = R.conv2d_backward_filter_bias(gy.double(), x.double(), w.shape, False, *args)
    assert_close_scaled(torch.from_numpy(gw), wgw, TF32_SCALED_TOL, "fl conv2dBackwardFilterBias 3x3")


@pytest.mark.gpu
def test_pool2d_through_fl_tensors(H):
    ok(H, H.flb200_fl_init())
    p = load("pool")
    wx, wy, sx, sy, px, py = (int(v) for v in p["geo"])
    x, gy = arr(p["x"]), arr(p["gy"])
    N, Cc, Hh, W = x.shape
    Ho, Wo = gy.shape[2:]
    for mode, ykey, gkey in ((0, "y", "gx"), (2, "y_avg", "gx_avg")):
        pl = H.flb200_fl_payload_new()
        y, gx = np.empty_like(gy), np.empty_like(x)
        ok(H, H.flb200_fl_pool2d(ptr(x), ptr(y), W, Hh, Cc, N, Wo, Ho, wx, wy, sx, sy, px, py, mode,
                                 vp(pl)))
        assert_close(torch.from_numpy(y), p[ykey], 1e-5, "fl pool2d")
        ok(H, H.flb200_fl_pool2d_backward(ptr(gy), ptr(x), ptr(y), ptr(gx), W, Hh, Cc, N, Wo, Ho, wx,
                                          wy, sx, sy, px, py, mode, vp(pl)))
        assert_close(torch.from_numpy(gx), p[gkey], 1e-5, "fl pool2dBackward")
        H.flb200_fl_payload_free(vp(pl))
    # the gradient without the forward payload: the selection is recomputed from x
    gx = np.empty_like(x)
    y = arr(p["y"])
    ok(H, H.flb200_fl_pool2d_backward(ptr(gy), ptr(x), ptr(y), ptr(gx), W, Hh, Cc, N, Wo, Ho, wx, wy,
                                      sx, sy, px, py, 0, None))
    assert_close(torch.from_numpy(gx), p["gx"], 1e-5, "fl pool2dBackward without payload")


@pytest.mark.gpu
def test_batchnorm_through_fl_tensors(H):
    ok(H, H.flb200_fl_init())
    b = load("batchnorm")
    x, g, beta, gy = arr(b["x"]), arr(b["g"]), arr(b["b"]), arr(b["gy"])
    shape = (C.c_int * 4)(*reversed(x.shape))
    axes = (C.c_int * 1)(2)
    ch = x.shape[1]
    rm, rv = np.zeros(ch, np.float32), np.ones(ch, np.float32)
    sm, sv, y = np.empty(ch, np.float32), np.empty(ch, np.float32), np.empty_like(x)
    ok(H, H.flb200_fl_batchnorm(ptr(x), ptr(g), ptr(beta), ptr(rm), ptr(rv), ptr(sm), ptr(sv), ptr(y),
                                shape, 4, axes, 1, ch, 1, C.c_double(0.1), C.c_double(1e-5)))
    assert_close(torch.from_numpy(y), b["y"], STRICT_TOL, "fl batchnorm y")
    assert_close(torch.from_numpy(sm), b["mean"], STRICT_TOL, "fl batchnorm saveMean")
    assert_close(torch.from_numpy(sv), b["invstd"], STRICT_TOL, "fl batchnorm saveVar")
    assert_close(torch.from_numpy(rm), b["rm"], STRICT_TOL, "fl batchnorm runningMean")
    assert_close(torch.from_numpy(rv), b["rv"], STRICT_TOL, "fl batchnorm runningVar")
    gx, gw, gb = np.empty_like(x), np.empty(ch, np.float32), np.empty(ch, np.float32)
    ok(H, H.flb200_fl_batchnorm_backward(ptr(gy), ptr(sm), ptr(sv), ptr(x), ptr(g), ptr(gx), ptr(gw),
                                         ptr(gb), shape, 4, axes, 1, ch, 1, C.c_float(1e-5)))
    assert_close(torch.from_numpy(gx), b["gx"], STRICT_TOL, "fl batchnormBackward dx")
    assert_close(torch.from_numpy(gw), b["gg"], STRICT_TOL, "fl batchnormBackward dgamma")
    assert_close(torch.from_numpy(gb), b["gb"], STRICT_TOL, "fl batchnormBackward dbeta")
    # the reference's error behaviour: no gradient without train (cudnn/BatchNorm.cpp:196-199)
    rc = H.flb200_fl_batchnorm_backward(ptr(gy), ptr(sm), ptr(sv), ptr(x), ptr(g), ptr(gx), ptr(gw),
                                        ptr(gb), shape, 4, axes, 1, ch, 0, C.c_float(1e-5))
    assert rc != 0 and b"train" in H.flb200_fl_last_error()


@pytest.mark.gpu
def test_rnn_through_fl_tensors(H):
    ok(H, H.flb200_fl_init())
    r = load("rnn_lstm")
    I, Hd, L_, B, T = (int(v) for v in r["dims"])
    x, hx, cx, w, gy = (arr(r[k]) for k in ("x", "hx", "cx", "w", "gy"))
    n = C.c_longlong(w.size)
    y, hy, cy = np.empty_like(gy), np.empty_like(hx), np.empty_like(cx)
    pl = H.flb200_fl_payload_new()
    ok(H, H.flb200_fl_rnn(ptr(x), ptr(hx), ptr(cx), ptr(w), n, ptr(y), ptr(hy), ptr(cy), I, B, T, Hd,
                          L_, 2, 1, C.c_float(0.0), vp(pl)))
    assert_close(torch.from_numpy(y), r["y"], STRICT_TOL, "fl rnn y")
    assert_close(torch.from_numpy(hy), r["hy"], STRICT_TOL, "fl rnn hy")
    assert_close(torch.from_numpy(cy), r["cy"], STRICT_TOL, "fl rnn cy")
    dx, dhx, dcx, dw = np.empty_like(x), np.empty_like(hx), np.empty_like(cx), np.empty_like(w)
    ok(H, H.flb200_fl_rnn_backward(ptr(x), ptr(hx), ptr(cx), ptr(w), n, ptr(y), ptr(gy), None, None,
                                   ptr(dx), ptr(dhx), ptr(dcx), ptr(dw), I, B, T, Hd, L_, 2, 1,
                                   C.c_float(0.0), vp(pl)))
    assert_close(torch.from_numpy(dx), r["dx"], STRICT_TOL, "fl rnnBackward dx")
    assert_close(torch.from_numpy(dhx), r["dhx"], STRICT_TOL, "fl rnnBackward dhx")
    assert_close(torch.from_numpy(dcx), r["dcx"], STRICT_TOL, "fl rnnBackward dcx")
    assert_close(torch.from_numpy(dw), r["dw"], STRICT_TOL, "fl rnnBackward dw")
    H.flb200_fl_payload_free(vp(pl))
    # rnnBackward without the forward payload is refused, as the reference backends do
    rc = H.flb200_fl_rnn_backward(ptr(x), ptr(hx), ptr(cx), ptr(w), n, ptr(y), ptr(gy), None, None,
                                  ptr(dx), ptr(dhx), ptr(dcx), ptr(dw), I, B, T, Hd, L_, 2, 1,
                                  C.c_float(0.0), None)
    assert rc != 0


@pytest.mark.gpu
def test_run_time_kernel_mode_selection(H):
    """createBenchmarkOptions() + DynamicBenchmark::audit (flashlight/fl/common/DynamicBenchmark.h:
    196-263): with benchmark mode on, the convolution gradients try fp32 FMA, TF32 and the
    three-pass split kDynamicBenchmarkDefaultCount (10) times each and then stay on the fastest by
    wall clock, which on a tensor-core-sized layer is one of the two tensor-core modes (the
    first timed call of a mode also pays its one-time set-up, so which of the two wins is not
    asserted); with benchmark mode off the configured mode runs."""
    from oracle import flref as R
    from tests.parity import assert_close_scaled
    ok(H, H.flb200_fl_init())
    H.flb200_fl_benchmark_new.restype = vp
    H.flb200_fl_benchmark_free.argtypes = [vp]
    H.flb200_fl_benchmark_state.argtypes = [vp, i32p]
    N, Cc, Hh, W, Co, k = 64, 256, 14, 14, 256, 3
    g = torch.Generator().manual_seed(5)
    x = torch.randn(N, Cc, Hh, W, generator=g)
    w = torch.randn(Co, Cc, k, k, generator=g) * 0.02
    gy = torch.randn(N, Co, Hh, W, generator=g)
    wgx = R.conv2d_backward_data(gy.double(), x.shape, w.double(), 1, 1, 1, 1, 1, 1, 1)
    wgw, _ = R.conv2d_backward_filter_bias(gy.double(), x.double(), w.shape, False, 1, 1, 1, 1, 1, 1, 1)
    xa, wa, gya = arr(x), arr(w), arr(gy)
    gx, gw = np.empty_like(xa), np.empty_like(wa)
    geo = (W, Hh, Cc, N, k, k, Co, W, Hh, 1, 1, 1, 1, 1, 1, 1)
    db, fb = H.flb200_fl_benchmark_new(), H.flb200_fl_benchmark_new()
    assert db and fb, H.flb200_fl_last_error().decode()
    done = C.c_int(0)
    assert H.flb200_fl_benchmark_state(vp(db), C.byref(done)) == 0 and done.value == 0
    H.flb200_fl_benchmark_mode(1)
    try:
        seen = set()
        for _ in range(31):
            seen.add(H.flb200_fl_benchmark_state(vp(db), C.byref(done)))
            ok(H, H.flb200_fl_conv2d_backward_tuned(ptr(gya), ptr(xa), ptr(wa), ptr(gx), ptr(gw), *geo,
                                                    vp(db), vp(fb)))
            assert_close_scaled(torch.from_numpy(gx), wgx, 2e-3, "tuned conv2dBackwardData")
            assert_close_scaled(torch.from_numpy(gw), wgw, 2e-3, "tuned conv2dBackwardFilterBias")
        assert seen == {0, 1, 2}                       # every mode was tried
        for b in (db, fb):
            assert H.flb200_fl_benchmark_state(vp(b), C.byref(done)) in (1, 2) and done.value == 1
    finally:
        H.flb200_fl_benchmark_mode(0)
    # benchmark mode off: the benchmark objects are ignored
    ok(H, H.flb200_fl_conv2d_backward_tuned(ptr(gya), ptr(xa), ptr(wa), ptr(gx), ptr(gw), *geo,
                                            vp(db), vp(fb)))
    assert_close_scaled(torch.from_numpy(gx), wgx, 2e-3, "conv2dBackwardData")
    H.flb200_fl_benchmark_free(vp(db))
    H.flb200_fl_benchmark_free(vp(fb))


@pytest.mark.gpu
def test_f16_activations_through_fl_tensors(H):
    """isDataTypeSupported(f16): conv2d -> batchnorm (f32 parameters) -> pool2d and all their
    gradients on f16 fl::Tensor objects.  The oracle runs the same chain in fp64 from the
    f16-rounded inputs; each stage here rounds its result to f16 once."""
    from oracle import flref as R
    from tests.parity import assert_close_scaled
    ok(H, H.flb200_fl_init())
    N, Cc, Hh, W, Co, k, pad = 4, 32, 12, 12, 64, 3, 1
    g = torch.Generator().manual_seed(9)
    x = torch.randn(N, Cc, Hh, W, generator=g).half()
    w = (torch.randn(Co, Cc, k, k, generator=g) * 0.06).half()
    gamma = torch.rand(Co, generator=g) + 0.5
    beta = torch.randn(Co, generator=g)
    gy = torch.randn(N, Co, Hh // 2, W // 2, generator=g).half()
    xr = x.double().requires_grad_(True)
    wr = w.double().requires_grad_(True)
    gr, br = gamma.double().requires_grad_(True), beta.double().requires_grad_(True)
    c = torch.nn.functional.conv2d(xr, wr, None, 1, pad)
    b = torch.nn.functional.batch_norm(c, None, None, gr, br, True, 0.1, 1e-5)
    p = torch.nn.functional.avg_pool2d(b, 2, 2)
    p.backward(gy.double())
    xa, wa, ga, ba, gya = arr(x), arr(w), arr(gamma), arr(beta), arr(gy)
    y = np.empty(p.shape, dtype=np.float32)
    gx, gw, gg, gb = np.empty_like(xa), np.empty_like(wa), np.empty_like(ga), np.empty_like(ba)
    ok(H, H.flb200_fl_half_chain(ptr(xa), ptr(wa), ptr(ga), ptr(ba), ptr(gya), ptr(y), ptr(gx),
                                 ptr(gw), ptr(gg), ptr(gb), W, Hh, Cc, N, k, Co, pad))
    tol = 6e-3   # three f16 roundings (2^-11 each) amplified by the normalisation
    assert_close_scaled(torch.from_numpy(y), p.detach(), tol, "f16 chain output")
    assert_close_scaled(torch.from_numpy(gx), xr.grad, tol, "f16 chain dx")
    assert_close_scaled(torch.from_numpy(gw), wr.grad, tol, "f16 chain dw")
    assert_close_scaled(torch.from_numpy(gg), gr.grad, tol, "f16 chain dgamma")
    assert_close_scaled(torch.from_numpy(gb), br.grad, tol, "f16 chain dbeta")


@pytest.mark.gpu
def test_rnn_dropout_through_fl_tensors(H):
    """The C++ extension draws the inter-layer dropout mask itself and keeps it in the payload:
    the result differs from the run without dropout, a second call draws another mask, and
    rnnBackward with the same payload is repeatable."""
    ok(H, H.flb200_fl_init())
    r = load("rnn_lstm")
    I, Hd, L_, B, T = (int(v) for v in r["dims"])
    assert L_ >= 2
    x, hx, cx, w, gy = (arr(r[k]) for k in ("x", "hx", "cx", "w", "gy"))
    n = C.c_longlong(w.size)
    outs = []
    for _ in range(2):
        y, hy, cy = np.empty_like(gy), np.empty_like(hx), np.empty_like(cx)
        pl = H.flb200_fl_payload_new()
        ok(H, H.flb200_fl_rnn(ptr(x), ptr(hx), ptr(cx), ptr(w), n, ptr(y), ptr(hy), ptr(cy), I, B, T,
                              Hd, L_, 2, 1, C.c_float(0.5), vp(pl)))
        grads = []
        for _ in range(2):
            dx, dhx, dcx, dw = (np.empty_like(x), np.empty_like(hx), np.empty_like(cx),
                                np.empty_like(w))
            ok(H, H.flb200_fl_rnn_backward(ptr(x), ptr(hx), ptr(cx), ptr(w), n, ptr(y), ptr(gy), None,
                                           None, ptr(dx), ptr(dhx), ptr(dcx), ptr(dw), I, B, T, Hd,
                                           L_, 2, 1, C.c_float(0.5), vp(pl)))
            grads.append((dx, dw))
        assert np.array_equal(grads[0][0], grads[1][0]) and np.array_equal(grads[0][1], grads[1][1])
        assert np.isfinite(y).all() and np.isfinite(grads[0][1]).all()
        H.flb200_fl_payload_free(vp(pl))
        outs.append(y)
    assert np.abs(outs[0] - r["y"].numpy()).max() > 1e-3      # not the dropout-free result
    assert np.abs(outs[0] - outs[1]).max() > 1e-4              # a fresh mask per call
    assert H.flb200_fl_rnn(ptr(x), ptr(hx), ptr(cx), ptr(w), n, ptr(outs[0]), None, None, I, B, T, Hd,
                           L_, 2, 1, C.c_float(1.0), None) == 1


@pytest.mark.gpu
def test_distributed_backend_through_fl_tensors(H, tmp_path):
    """fl::allReduce / allReduceMultiple / syncDistributed on fl::Tensor objects, answered by
    B200DistributedBackend.cpp over the native NCCL backend.  One process is a communicator of
    size 1: every collective, copy and stream dependency still runs.  Error behaviour follows
    flashlight/fl/distributed/backend/cuda/DistributedBackend.cpp:114-175."""
    ok(H, H.flb200_fl_init())
    H.flb200_fl_all_reduce.argtypes = [f32p, C.c_longlong, C.c_int]
    H.flb200_fl_all_reduce_multiple.argtypes = [C.POINTER(f32p), C.POINTER(C.c_longlong), C.c_int,
                                                C.c_int, C.c_int]
    x = np.arange(1000, dtype=np.float32)
    if H.flb200_fl_world_size() == 1 and H.flb200_fl_world_rank() == 0:
        rc = H.flb200_fl_all_reduce(ptr(x), x.size, 0)
        if rc != 0:   # not yet initialised in this process
            assert rc == 2 and b"not initialized" in H.flb200_fl_last_error()
    assert H.flb200_fl_distributed_init(b"", 0, 1, 8) == 1          # std::invalid_argument
    assert b"FilePath" in H.flb200_fl_last_error()
    ok(H, H.flb200_fl_distributed_init(str(tmp_path / "id").encode(), 0, 1, 8))
    assert (H.flb200_fl_world_rank(), H.flb200_fl_world_size()) == (0, 1)
    for async_ in (0, 1):
        y = x.copy()
        ok(H, H.flb200_fl_all_reduce(ptr(y), y.size, async_))
        assert np.array_equal(y, x)
    bufs = [np.full(n, float(i + 1), dtype=np.float32) for i, n in enumerate((5, 4096, 33))]
    for async_, contiguous in ((0, 0), (1, 0), (0, 1), (1, 1)):
        work = [b.copy() for b in bufs]
        ptrs = (f32p * 3)(*[ptr(b) for b in work])
        counts = (C.c_longlong * 3)(*[b.size for b in work])
        ok(H, H.flb200_fl_all_reduce_multiple(ptrs, counts, 3, async_, contiguous))
        for a, b in zip(work, bufs):
            assert np.array_equal(a, b)
    big = [np.zeros(3 << 20, dtype=np.float32) for _ in range(2)]   # 24 MB > the 20 MB buffer
    ptrs = (f32p * 2)(*[ptr(b) for b in big])
    counts = (C.c_longlong * 2)(*[b.size for b in big])
    assert H.flb200_fl_all_reduce_multiple(ptrs, counts, 2, 0, 1) == 2
    assert b"Total coalesce buffer size" in H.flb200_fl_last_error()
    ok(H, H.flb200_fl_all_reduce_multiple(ptrs, counts, 2, 0, 0))    # fine when not packed
