"""ctypes binding of libflb200.so — the C ABI declared in include/flb200.h.

The library is the product: there is no Python or CPU fallback.  Importing this
module without the built shared object raises, and every wrapper raises on a
non-zero status (ValueError for FLB200_INVALID_ARG, the counterpart of the
std::invalid_argument the C++ extension throws; RuntimeError otherwise).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "csrc" / "libflb200.so"

OK, INVALID_ARG, UNSUPPORTED, LAUNCH_FAILURE, TIMEOUT, WORKSPACE_TOO_SMALL = range(6)
F32, F16, BF16 = 0, 1, 2
POOL_MAX, POOL_AVG_INCLUDE_PAD, POOL_AVG_EXCLUDE_PAD = 0, 1, 2
RNN_RELU, RNN_TANH, RNN_LSTM, RNN_GRU = 0, 1, 2, 3
MATH_STRICT_F32, MATH_TF32, MATH_F32X3 = 0, 1, 2
LAYOUT_NCHW, LAYOUT_NCHW_IN_NHWC_OUT, LAYOUT_NHWC = 0, 2, 3
MATH_BY_NAME = {"strict": MATH_STRICT_F32, "tf32": MATH_TF32, "f32x3": MATH_F32X3}
REDUCE_NONE, REDUCE_MEAN, REDUCE_SUM = 0, 1, 2
ACT_NONE, ACT_GELU = 0, 1
IDS_I32, IDS_I64 = 0, 1

i32, i64, f32, f64, vp, sz = C.c_int32, C.c_int64, C.c_float, C.c_double, C.c_void_p, C.c_size_t


class Conv2dDesc(C.Structure):
    _fields_ = [(n, i32) for n in (
        "W", "H", "C", "N", "kW", "kH", "Cout", "sx", "sy", "px", "py", "dx", "dy", "groups",
        "dtype", "math_mode", "layout")]


class Conv2dCache(C.Structure):
    _fields_ = [("x_cl", vp), ("x_cl_bytes", sz), ("x_cl_valid", i32),
                ("gy_cl", vp), ("gy_cl_bytes", sz), ("gy_cl_valid", i32)]


class Pool2dDesc(C.Structure):
    _fields_ = [(n, i32) for n in (
        "W", "H", "C", "N", "wx", "wy", "sx", "sy", "px", "py", "mode", "dtype", "layout")]


class BatchnormDesc(C.Structure):
    _fields_ = [("outer", i64), ("channels", i64), ("inner", i64), ("dtype", i32)]


class MatmulDesc(C.Structure):
    _fields_ = [(n, i64) for n in (
        "m", "n", "k", "batch", "a_row", "a_col", "a_batch", "b_row", "b_col", "b_batch",
        "c_row", "c_col", "c_batch")] + [("alpha", f32), ("beta", f32), ("dtype", i32),
                                         ("math_mode", i32)]


class RnnDesc(C.Structure):
    _fields_ = [(n, i32) for n in (
        "input_size", "hidden_size", "num_layers", "batch", "seq_len", "mode", "bidirectional",
        "dtype", "math_mode")]


P = C.POINTER
# name -> (restype, argtypes); one entry per declaration in include/flb200.h
SIGNATURES = {
    "flb200_abi_version": (C.c_int, []),
    "flb200_status_string": (C.c_char_p, [C.c_int]),
    "flb200_last_error": (C.c_char_p, []),
    "flb200_kernel_launches": (C.c_longlong, []),
    "flb200_has_tensor_core_path": (C.c_int, []),
    "flb200_tc_kernel_launches": (C.c_longlong, []),
    "flb200_tc_poll_status": (C.c_int, [vp]),
    "flb200_conv2d_output_dims": (C.c_int, [P(Conv2dDesc), P(i32), P(i32)]),
    "flb200_conv2d_workspace_bytes": (sz, [P(Conv2dDesc), C.c_int]),
    "flb200_conv2d_forward": (C.c_int, [P(Conv2dDesc), vp, vp, vp, vp, vp, sz, vp]),
    "flb200_conv2d_stats_bytes": (sz, [P(Conv2dDesc), P(i64)]),
    "flb200_conv2d_forward_stats": (C.c_int, [P(Conv2dDesc), vp, vp, vp, vp, vp, sz, vp, sz, vp, vp]),
    "flb200_batchnorm_from_stats_workspace_bytes": (sz, [P(BatchnormDesc), i64]),
    "flb200_batchnorm_forward_from_stats": (C.c_int, [P(BatchnormDesc), vp, vp, C.c_int, vp, i64, vp,
                                                      vp, vp, vp, vp, vp, f64, f64, vp, vp, vp, sz,
                                                      vp]),
    "flb200_conv2d_backward_data": (C.c_int, [P(Conv2dDesc), vp, vp, vp, vp, sz, vp]),
    "flb200_conv2d_backward_filter_bias": (C.c_int, [P(Conv2dDesc), vp, vp, vp, vp, vp, sz, vp]),
    "flb200_conv2d_cache_bytes": (sz, [P(Conv2dDesc), C.c_int]),
    "flb200_conv2d_forward_cached": (
        C.c_int, [P(Conv2dDesc), vp, vp, vp, vp, vp, sz, P(Conv2dCache), vp]),
    "flb200_conv2d_backward_data_cached": (
        C.c_int, [P(Conv2dDesc), vp, vp, vp, vp, sz, P(Conv2dCache), vp]),
    "flb200_conv2d_backward_filter_bias_cached": (
        C.c_int, [P(Conv2dDesc), vp, vp, vp, vp, vp, sz, P(Conv2dCache), vp]),
    "flb200_pool2d_output_dims": (C.c_int, [P(Pool2dDesc), P(i32), P(i32)]),
    "flb200_pool2d_forward": (C.c_int, [P(Pool2dDesc), vp, vp, vp, vp]),
    "flb200_pool2d_backward": (C.c_int, [P(Pool2dDesc), vp, vp, vp, vp, vp]),
    "flb200_selftest_bounded_wait_workspace_bytes": (sz, []),
    "flb200_selftest_bounded_wait": (C.c_int, [f64, vp, sz, vp]),
    "flb200_layernorm_affine_forward": (C.c_int, [vp, vp, vp, vp, i64, i64, C.c_int, vp]),
    "flb200_layernorm_affine_workspace_bytes": (sz, [i64, i64]),
    "flb200_layernorm_affine_backward": (C.c_int, [vp, vp, vp, vp, vp, vp, i64, i64, C.c_int, vp,
                                                   sz, vp]),
    "flb200_batchnorm_geometry": (C.c_int, [P(i64), C.c_int, P(i32), C.c_int, P(BatchnormDesc)]),
    "flb200_batchnorm_workspace_bytes": (sz, [P(BatchnormDesc)]),
    "flb200_batchnorm_forward": (C.c_int, [P(BatchnormDesc), vp, vp, vp, vp, vp, vp, vp, C.c_int,
                                           f64, f64, vp, vp, sz, vp]),
    "flb200_batchnorm_backward": (C.c_int, [P(BatchnormDesc), vp, vp, vp, vp, vp, vp, vp, vp, vp,
                                            sz, vp]),
    "flb200_batchnorm_relu_forward": (C.c_int, [P(BatchnormDesc), vp, vp, vp, vp, vp, vp, vp,
                                                C.c_int, f64, f64, vp, vp, sz, vp]),
    "flb200_batchnorm_add_relu_forward": (C.c_int, [P(BatchnormDesc), vp, vp, vp, vp, vp, vp, vp,
                                                    vp, C.c_int, f64, f64, vp, vp, vp, sz, vp]),
    "flb200_batchnorm_add_relu_backward": (C.c_int, [P(BatchnormDesc), vp, vp, vp, vp, vp, vp, vp,
                                                     vp, vp, vp, vp, vp, sz, vp]),
    "flb200_batchnorm_relu_backward": (C.c_int, [P(BatchnormDesc), vp, vp, vp, vp, vp, vp, vp, vp,
                                                 vp, vp, sz, vp]),
    "flb200_matmul_workspace_bytes": (sz, [P(MatmulDesc)]),
    "flb200_matmul": (C.c_int, [P(MatmulDesc), vp, vp, vp, vp, sz, vp]),
    "flb200_linear_workspace_bytes": (sz, [i64, i64, i64, C.c_int]),
    "flb200_linear_forward": (C.c_int, [i64, i64, i64, vp, vp, vp, vp, C.c_int, vp, sz, vp]),
    "flb200_linear_bias_act_forward": (C.c_int, [i64, i64, i64, vp, vp, vp, vp, vp, C.c_int, C.c_int,
                                                 C.c_int, vp, sz, vp]),
    "flb200_linear_backward_input": (C.c_int, [i64, i64, i64, vp, vp, vp, C.c_int, vp, sz, vp]),
    "flb200_linear_backward_weight": (C.c_int, [i64, i64, i64, vp, vp, vp, C.c_int, vp, sz, vp]),
    "flb200_channel_sum_workspace_bytes": (sz, [i64, i64, i64]),
    "flb200_channel_sum": (C.c_int, [vp, vp, i64, i64, i64, C.c_int, vp, sz, vp]),
    "flb200_channel_sum_static_scratch": (C.c_int, [vp, vp, i64, i64, i64, C.c_int, vp]),
    "flb200_channel_bias_add": (C.c_int, [vp, vp, vp, i64, i64, i64, C.c_int, vp]),
    "flb200_embedding_forward": (C.c_int, [vp, vp, C.c_int, vp, i64, i64, i64, C.c_int, vp]),
    "flb200_embedding_backward": (C.c_int, [vp, vp, C.c_int, vp, i64, i64, i64, C.c_int, vp]),
    "flb200_softmax_forward": (C.c_int, [vp, vp, i64, i64, f32, i64, C.c_int, vp]),
    "flb200_softmax_backward": (C.c_int, [vp, vp, vp, i64, i64, f32, C.c_int, vp]),
    "flb200_softmax_forward_lse": (C.c_int, [vp, vp, vp, i64, i64, f32, i64, C.c_int, vp]),
    "flb200_attention_backward_supported": (C.c_int, [i64, i64, C.c_int]),
    "flb200_attention_backward_workspace_bytes": (sz, [i64, i64, i64]),
    "flb200_attention_backward": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, f32,
                                            C.c_int, C.c_int, vp, sz, vp]),
    "flb200_sgd_step": (C.c_int, [vp, vp, vp, i64, f32, f32, f32, C.c_int, f32, C.c_int, C.c_int, vp]),
    "flb200_relu_forward_mask": (C.c_int, [vp, vp, vp, i64, C.c_int, vp]),
    "flb200_relu_backward_mask": (C.c_int, [vp, vp, vp, i64, C.c_int, vp]),
    "flb200_add_relu_forward_mask": (C.c_int, [vp, vp, vp, vp, i64, C.c_int, vp]),
    "flb200_relu_backward_mask_sum": (C.c_int, [vp, vp, vp, vp, i64, C.c_int, vp]),
    "flb200_relu_forward": (C.c_int, [vp, vp, i64, C.c_int, vp]),
    "flb200_relu_backward": (C.c_int, [vp, vp, vp, i64, C.c_int, vp]),
    "flb200_gelu_forward": (C.c_int, [vp, vp, i64, C.c_int, vp]),
    "flb200_gelu_backward": (C.c_int, [vp, vp, vp, i64, C.c_int, vp]),
    "flb200_tanh_forward": (C.c_int, [vp, vp, i64, C.c_int, vp]),
    "flb200_tanh_backward": (C.c_int, [vp, vp, vp, i64, C.c_int, vp]),
    "flb200_dropout_apply": (C.c_int, [vp, vp, vp, f32, i64, C.c_int, vp]),
    "flb200_layernorm_forward": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, i64, i64, f64, C.c_int, vp]),
    "flb200_layernorm_backward_workspace_bytes": (sz, [i64, i64]),
    "flb200_layernorm_backward": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, i64, i64, C.c_int, vp, sz,
                                            vp]),
    "flb200_bernoulli_mask": (C.c_int, [vp, i64, f32, C.c_uint64, C.c_uint64, C.c_int, vp]),
    "flb200_add": (C.c_int, [vp, vp, vp, i64, C.c_int, vp]),
    "flb200_astype": (C.c_int, [vp, C.c_int, vp, C.c_int, i64, vp]),
    "flb200_reorder": (C.c_int, [vp, vp, C.POINTER(C.c_int64), C.POINTER(C.c_int64), i64, C.c_int, vp]),
    "flb200_log_softmax_forward": (C.c_int, [vp, vp, i64, i64, C.c_int, vp]),
    "flb200_log_softmax_backward": (C.c_int, [vp, vp, vp, i64, i64, C.c_int, vp]),
    "flb200_cce_workspace_bytes": (sz, [i64]),
    "flb200_cce_forward": (C.c_int, [vp, vp, vp, vp, vp, i64, i64, C.c_int, C.c_int, C.c_int, vp,
                                     sz, vp]),
    "flb200_cce_backward": (C.c_int, [vp, vp, vp, vp, i64, i64, C.c_int, C.c_int, C.c_int, vp]),
    "flb200_log_softmax_cce_backward": (C.c_int, [vp, vp, vp, vp, vp, i64, i64, C.c_int, C.c_int,
                                                  C.c_int, vp]),
    "flb200_rnn_num_params": (i64, [P(RnnDesc)]),
    "flb200_rnn_reserve_bytes": (sz, [P(RnnDesc)]),
    "flb200_rnn_workspace_bytes": (sz, [P(RnnDesc), C.c_int]),
    "flb200_rnn_forward": (C.c_int, [P(RnnDesc), vp, vp, vp, vp, vp, vp, vp, vp, sz, vp, sz, vp]),
    "flb200_rnn_backward": (C.c_int, [P(RnnDesc), vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp,
                                      vp, sz, vp, sz, vp]),
    "flb200_rnn_dropout_mask_elements": (i64, [P(RnnDesc)]),
    "flb200_rnn_reserve_bytes_dropout": (sz, [P(RnnDesc)]),
    "flb200_rnn_forward_dropout": (C.c_int, [P(RnnDesc), vp, vp, vp, vp, vp, f32, vp, vp, vp, vp,
                                             sz, vp, sz, vp]),
    "flb200_rnn_backward_dropout": (C.c_int, [P(RnnDesc), vp, vp, vp, vp, vp, f32, vp, vp, vp, vp,
                                              vp, vp, vp, vp, vp, sz, vp, sz, vp]),
}


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m flashlight_b200.csrc.build` "
            "(there is no fallback path)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class Flb200Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"flb200 status {status} ({lib.flb200_status_string(status).decode()}): {message}")
        self.status = status


class Flb200InvalidArgument(Flb200Error, ValueError):
    """FLB200_INVALID_ARG — the counterpart of std::invalid_argument in the reference."""


def check(status: int) -> None:
    if status == OK:
        return
    msg = lib.flb200_last_error().decode(errors="replace")
    if status == INVALID_ARG:
        raise Flb200InvalidArgument(status, msg)
    raise Flb200Error(status, msg)


def kernel_launches() -> int:
    return int(lib.flb200_kernel_launches())
