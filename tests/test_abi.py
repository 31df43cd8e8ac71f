"""CPU checks of the C ABI: the shared object loads, exports every function the header
declares, and its host-side logic (geometry, extents, sizes, argument validation) behaves
like the reference's host code.  No kernel is launched here."""
import ctypes as C
import re
from pathlib import Path

import pytest

from flashlight_b200 import _lib as L
from oracle import flref as R

HEADER = Path(__file__).resolve().parent.parent / "include" / "flb200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(flb200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert len(names) >= 40
    raw = C.CDLL(str(L.LIB_PATH))
    for n in names:
        assert hasattr(raw, n), f"{n} is declared in include/flb200.h but not exported"
    # and the binding table covers the header exactly
    assert sorted(L.SIGNATURES) == names


def test_status_strings_and_version():
    assert L.lib.flb200_abi_version() == 2
    assert L.lib.flb200_status_string(0) == b"ok"
    assert b"invalid" in L.lib.flb200_status_string(L.INVALID_ARG)


@pytest.mark.parametrize("W,H,k,s,p,d", [(28, 28, 5, 1, 2, 1), (224, 224, 7, 2, 3, 1),
                                         (56, 56, 3, 2, 1, 1), (1000, 1, 13, 1, 6, 1),
                                         (10, 9, 4, 1, 2, 2)])
def test_conv_output_dims_follow_reference_formula(W, H, k, s, p, d):
    kh = k if H > 1 else 1
    ph = p if H > 1 else 0
    desc = L.Conv2dDesc(W, H, 3, 2, k, kh, 8, s, s, p, ph, d, d, 1, L.F32, 0)
    wo, ho = L.i32(), L.i32()
    L.check(L.lib.flb200_conv2d_output_dims(C.byref(desc), C.byref(wo), C.byref(ho)))
    assert wo.value == R.conv_out_dim(W, k, s, p, d)
    assert ho.value == R.conv_out_dim(H, kh, s, ph, d)


def test_conv_rejects_bad_groups_like_invalid_argument():
    desc = L.Conv2dDesc(8, 8, 6, 1, 3, 3, 8, 1, 1, 1, 1, 1, 1, 4, L.F32, 0)
    with pytest.raises(ValueError):
        L.check(L.lib.flb200_conv2d_output_dims(C.byref(desc), None, None))
    assert b"groups" in L.lib.flb200_last_error()


def test_pool_output_dims():
    d = L.Pool2dDesc(112, 112, 64, 2, 3, 3, 2, 2, 1, 1, L.POOL_MAX, L.F32)
    wo, ho = L.i32(), L.i32()
    L.check(L.lib.flb200_pool2d_output_dims(C.byref(d), C.byref(wo), C.byref(ho)))
    assert (wo.value, ho.value) == (56, 56) == (R.pool_out_dim(112, 3, 2, 1),) * 2


@pytest.mark.parametrize("shape,axes", [((5, 6, 7, 8), [2]), ((5, 6, 7, 8), [0, 1, 2]),
                                        ((768, 512, 8), [1, 2]), ((1000, 1, 1024, 16), [3]),
                                        ((4, 4, 4, 4), [0, 1, 2, 3]), ((9, 3), [1])])
def test_batchnorm_geometry_matches_oracle(shape, axes):
    d = L.BatchnormDesc()
    L.check(L.lib.flb200_batchnorm_geometry((L.i64 * len(shape))(*shape), len(shape),
                                            (L.i32 * len(axes))(*axes), len(axes), C.byref(d)))
    assert (d.outer, d.channels, d.inner) == R.batchnorm_geometry(shape, axes)
    assert L.lib.flb200_batchnorm_workspace_bytes(C.byref(d)) > 0


def test_batchnorm_geometry_errors():
    d = L.BatchnormDesc()
    shape = (L.i64 * 4)(5, 6, 7, 8)
    with pytest.raises(ValueError, match="continuous"):
        L.check(L.lib.flb200_batchnorm_geometry(shape, 4, (L.i32 * 2)(0, 2), 2, C.byref(d)))
    with pytest.raises(ValueError, match="exceeds"):
        L.check(L.lib.flb200_batchnorm_geometry(shape, 4, (L.i32 * 1)(4), 1, C.byref(d)))


@pytest.mark.parametrize("mode,expect", [(L.RNN_RELU, 56), (L.RNN_LSTM, 224), (L.RNN_GRU, 168)])
def test_rnn_param_count_of_reference_test(mode, expect):
    """flashlight/fl/test/autograd/AutogradRnnTest.cpp:38-50: in=2, H=2, 2 layers, bidirectional."""
    d = L.RnnDesc(2, 2, 2, 2, 3, mode, 1, L.F32, 0)
    assert L.lib.flb200_rnn_num_params(C.byref(d)) == expect
    assert L.lib.flb200_rnn_reserve_bytes(C.byref(d)) > 0
    assert L.lib.flb200_rnn_workspace_bytes(C.byref(d), 1) > 0


def test_rnn_param_count_of_the_bilstm_workload():
    d = L.RnnDesc(80, 1024, 3, 32, 500, L.RNN_LSTM, 1, L.F32, 0)
    assert L.lib.flb200_rnn_num_params(C.byref(d)) == 59424768
    assert L.lib.flb200_rnn_num_params(C.byref(d)) == R.rnn_num_params(80, 1024, 3, R.RNN_LSTM, True)


def test_null_and_bad_arguments_return_status_not_crash():
    assert L.lib.flb200_relu_forward(None, None, -1, L.F32, None) == L.INVALID_ARG
    assert L.lib.flb200_relu_forward(None, None, 0, L.F32, None) == L.OK  # empty tensor: no-op
    assert L.lib.flb200_add(None, None, None, 4, L.F32, None) == L.INVALID_ARG
    assert L.lib.flb200_log_softmax_forward(None, None, 0, 3, L.F32, None) == L.INVALID_ARG
    assert L.lib.flb200_cce_forward(None, None, None, None, None, 3, 3, 7, -1, L.F32, None, 0,
                                    None) == L.INVALID_ARG
    assert b"unknown reduction" in L.lib.flb200_last_error()
    md = L.MatmulDesc(4, 4, 4, 1, 4, 1, 0, 4, 1, 0, 4, 1, 0, 1.0, 0.0, L.F16, 0)
    assert L.lib.flb200_matmul(C.byref(md), None, None, None, None, 0, None) == L.INVALID_ARG


def test_cpp_extension_compiles_against_reference_headers(reference_root):
    """B200AutogradExtension overrides every pure virtual of fl::AutogradExtension with the exact
    reference signatures: compiling it against the reference headers is the proof."""
    import subprocess
    import sys
    script = (Path(__file__).resolve().parent.parent / "flashlight_b200" / "csrc" / "fl" /
              "check_against_reference.py")
    res = subprocess.run([sys.executable, str(script), str(reference_root)], capture_output=True,
                         text=True)
    assert res.returncode == 0, res.stderr
    assert "compiles against the reference headers" in res.stdout


def test_dynamic_benchmark_host_logic():
    """fl::DynamicBenchmarkOptions semantics (flashlight/fl/common/DynamicBenchmark.h:60-194):
    options are tried in order `count` times each, then the fastest stays."""
    from flashlight_b200.extension import DynamicBenchmark
    b = DynamicBenchmark([7, 8, 9], count=2)
    assert b.currentOption() == 7 and not b.timingsComplete()
    fake = {7: 3.0, 8: 1.0, 9: 2.0}
    DynamicBenchmark.setBenchmarkMode(True)
    try:
        order = []
        for _ in range(6):
            opt = b.currentOption()
            order.append(opt)
            b.times[b._idx] += fake[opt]      # what audit() does around the call
            b.counts[b._idx] += 1
        assert order == [7, 7, 8, 8, 9, 9]
        assert b.timingsComplete() and b.currentOption() == 8
        ran = []
        assert b.audit(lambda: ran.append(1) or "x") == "x" and ran == [1]   # no more timing
        assert b.counts == [2, 2, 2]
    finally:
        DynamicBenchmark.setBenchmarkMode(False)
    with pytest.raises(ValueError):
        DynamicBenchmark([])


def test_unbind_returns_one_gradient_for_all_parts():
    """Host logic of the tape's unbind(): the parts' gradients meet in one buffer and reach the
    packed tensor once, mapped back by the inverse of the forward copy, whatever order they
    arrive in; a second backward pass through a fresh call starts from a clean state."""
    import torch
    from flashlight_b200 import autograd as A
    B, T, h, hd = 2, 3, 2, 4
    d = h * hd
    fwd = lambda t: t.reshape(B, T, 3, h, hd).permute(2, 0, 3, 1, 4).reshape(3, B * h, T, hd).contiguous()
    bwd = lambda g: g.reshape(3, B, h, T, hd).permute(1, 3, 0, 2, 4).reshape(B * T, 3 * d).contiguous()
    for order in ((0, 1, 2), (2, 0, 1)):
        x = A.Variable(torch.arange(B * T * 3 * d, dtype=torch.float32).reshape(B * T, 3 * d), True)
        parts = A.unbind(x, fwd, bwd, 3)
        ref = x.tensor.reshape(B, T, 3, h, hd)
        for i, p in enumerate(parts):
            assert torch.equal(p.tensor, ref[:, :, i].permute(0, 2, 1, 3).reshape(B * h, T, hd))
        grads = [torch.full((B * h, T, hd), float(i + 1)) for i in range(3)]
        for i in order:
            parts[i].grad_func(parts[i].inputs, grads[i])
            if i != order[-1]:
                assert x.grad is None  # nothing is handed on before the last part has arrived
        want = torch.empty(B, T, 3, h, hd)
        for i in range(3):
            want[:, :, i] = float(i + 1)
        assert torch.equal(x.grad, want.reshape(B * T, 3 * d))
