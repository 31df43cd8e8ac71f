"""Fused forward / gradient kernels for the tensor-op chains of Flashlight's
autograd functions that are NOT behind fl::AutogradExtension
(flashlight/fl/autograd/Functions.cpp): relu, gelu, tanh, dropout, linear,
logSoftmax, categoricalCrossEntropy, bias tile/sumAs and gradient accumulation.

Tensor convention as in extension.py: torch shape = reversed fl shape, None for
an absent tensor.  Every function launches flb200 kernels through the C ABI on
torch's current stream; nothing is computed by torch itself.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib as L
from .extension import (default_math_mode, dtype_code, ptr, same_layout, stream_handle,
                        workspace)


def _unary(fn, x):
    out = torch.empty_like(x)
    L.check(fn(ptr(x), ptr(out), x.numel(), dtype_code(x), stream_handle()))
    return out


def _binary(fn, a, b):
    if not same_layout(a, b) or a.dtype != b.dtype:
        raise ValueError("operands must have the same shape, memory layout and dtype")
    out = torch.empty_like(a)
    L.check(fn(ptr(a), ptr(b), ptr(out), a.numel(), dtype_code(a), stream_handle()))
    return out


def relu(x):
    """fl::relu = max(x, 0) (Functions.cpp:1787-1789)."""
    return _unary(L.lib.flb200_relu_forward, x)


def relu_backward(x, grad_y):
    """(x > 0) * dy (Functions.cpp:329-338).  Passing the output y instead of x gives the same mask."""
    return _binary(L.lib.flb200_relu_backward, x, grad_y)


def relu_with_mask(x):
    """relu that also returns the predicate x > 0 packed 8 elements per byte."""
    y = torch.empty_like(x)
    mask = torch.empty((x.numel() + 7) // 8, dtype=torch.uint8, device=x.device)
    L.check(L.lib.flb200_relu_forward_mask(ptr(x), ptr(y), ptr(mask), x.numel(), dtype_code(x),
                                           stream_handle()))
    return y, mask


def relu_backward_mask(mask, grad_y):
    gx = torch.empty_like(grad_y)
    L.check(L.lib.flb200_relu_backward_mask(ptr(mask), ptr(grad_y), ptr(gx), grad_y.numel(),
                                            dtype_code(grad_y), stream_handle()))
    return gx


def add_relu_with_mask(a, b):
    """relu(a + b) in one pass, with the predicate (a + b) > 0 packed 8 elements per byte."""
    if not same_layout(a, b):
        raise ValueError("operands must have the same shape and memory layout")
    y = torch.empty_like(a)
    mask = torch.empty((a.numel() + 7) // 8, dtype=torch.uint8, device=a.device)
    L.check(L.lib.flb200_add_relu_forward_mask(ptr(a), ptr(b), ptr(y), ptr(mask), a.numel(),
                                               dtype_code(a), stream_handle()))
    return y, mask


def relu_backward_mask_sum(mask, grad_a, grad_b):
    """mask ? grad_a + grad_b : 0 — the relu gradient of an output with two consumers."""
    if not same_layout(grad_a, grad_b):
        raise ValueError("operands must have the same shape and memory layout")
    gx = torch.empty_like(grad_a)
    L.check(L.lib.flb200_relu_backward_mask_sum(ptr(mask), ptr(grad_a), ptr(grad_b), ptr(gx),
                                                grad_a.numel(), dtype_code(grad_a),
                                                stream_handle()))
    return gx


def gelu(x):
    """fl::gelu, tanh form (Functions.cpp:1791-1796)."""
    return _unary(L.lib.flb200_gelu_forward, x)


def gelu_backward(x, grad_y):
    return _binary(L.lib.flb200_gelu_backward, x, grad_y)


def tanh(x):
    return _unary(L.lib.flb200_tanh_forward, x)


def tanh_backward(y, grad_y):
    """(1 - y^2) * dy from the saved output (Functions.cpp:454-463)."""
    return _binary(L.lib.flb200_tanh_backward, y, grad_y)


def dropout_apply(x, mask, p: float):
    """x * mask / (1 - p): forward with x, gradient with dy (Functions.cpp:1777-1785)."""
    if not same_layout(x, mask) or x.dtype != mask.dtype:
        raise ValueError("mask must match the tensor's shape, memory layout and dtype")
    out = torch.empty_like(x)
    L.check(L.lib.flb200_dropout_apply(ptr(x), ptr(mask), ptr(out), 1.0 / (1.0 - p), x.numel(),
                                       dtype_code(x), stream_handle()))
    return out


def add(a, b, out=None):
    """Gradient fan-in accumulation of Variable::addGrad (Variable.cpp:205-211)."""
    if not same_layout(a, b) or a.dtype != b.dtype:
        raise ValueError("operands must have the same shape, memory layout and dtype")
    if out is None:
        out = torch.empty_like(a)
    L.check(L.lib.flb200_add(ptr(a), ptr(b), ptr(out), a.numel(), dtype_code(a), stream_handle()))
    return out


_ASTYPE_CODES = {torch.float32: L.F32, torch.float16: L.F16, torch.bfloat16: L.BF16}


def astype(x, dtype):
    """x.to(dtype) between float32 and float16 / bfloat16 through flb200_astype (contiguous
    tensors); None for anything else (the caller then lets torch convert)."""
    src, dst = _ASTYPE_CODES.get(x.dtype), _ASTYPE_CODES.get(dtype)
    if src is None or dst is None or not x.is_cuda or not x.is_contiguous():
        return None
    if src != dst and L.F32 not in (src, dst):
        return None
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    L.check(L.lib.flb200_astype(x.data_ptr(), src, out.data_ptr(), dst, x.numel(),
                                stream_handle()))
    return out


def reorder(x, shape, perm):
    """`x.reshape(shape).permute(perm).contiguous()` through flb200_reorder: `shape` has up to five
    extents, `perm` keeps the last one in place (the contiguous run).  Returns the permuted,
    contiguous tensor; None where the kernel's 16-byte rules do not hold (the caller then uses
    the torch copy)."""
    import ctypes as C
    n = len(shape)
    if n < 2 or n > 5 or perm[-1] != n - 1 or not x.is_contiguous():
        return None
    es = x.element_size()
    inner = shape[-1]
    strides = [1] * n
    for k in range(n - 2, -1, -1):
        strides[k] = strides[k + 1] * shape[k + 1]
    outer = [shape[p] for p in perm[:-1]]
    ostr = [strides[p] for p in perm[:-1]]
    while len(outer) < 4:
        outer.insert(0, 1)
        ostr.insert(0, 0)
    vec = 16 // es
    if (inner * es) % 16 or any(s % vec for s in ostr) or x.data_ptr() % 16:
        return None
    out = torch.empty([shape[p] for p in perm], dtype=x.dtype, device=x.device)
    d = (C.c_int64 * 4)(*outer)
    st = (C.c_int64 * 4)(*ostr)
    L.check(L.lib.flb200_reorder(ptr(x), ptr(out), d, st, inner, dtype_code(x), stream_handle()))
    return out


def channel_sum(x, outer: int, channels: int, inner: int):
    """out[c] = sum_{o,i} x[o][c][i] (conv bias gradient; detail::sumAs onto a bias)."""
    if x.numel() != outer * channels * inner:
        raise ValueError("channel_sum: geometry does not match the tensor")
    out = torch.empty(channels, dtype=torch.float32, device=x.device)
    nbytes = L.lib.flb200_channel_sum_workspace_bytes(outer, channels, inner)
    ws = workspace(nbytes, x)
    L.check(L.lib.flb200_channel_sum(ptr(x), ptr(out), outer, channels, inner, dtype_code(x), ptr(ws),
                                     nbytes, stream_handle()))
    return out


def channel_bias_add(x, bias, outer: int, channels: int, inner: int, out=None):
    if out is None:
        out = torch.empty_like(x)
    L.check(L.lib.flb200_channel_bias_add(ptr(x), ptr(bias), ptr(out), outer, channels, inner,
                                          dtype_code(x), stream_handle()))
    return out


def layernorm_affine(xhat, weight, bias):
    """y = xhat * weight + bias over rows of features (the affine part of fl::LayerNorm);
    weight / bias are fp32 parameter vectors of the last dimension's length."""
    feat = xhat.shape[-1]
    xh = xhat.contiguous()
    y = torch.empty_like(xh)
    L.check(L.lib.flb200_layernorm_affine_forward(ptr(xh), ptr(weight), ptr(bias), ptr(y),
                                                  xh.numel() // feat, feat, dtype_code(xh),
                                                  stream_handle()))
    return y


def layernorm(x, weight, bias, eps: float):
    """fl::LayerNorm over the last dimension in one kernel: returns (y, xhat, invstd)."""
    feat = x.shape[-1]
    xc = x.contiguous()
    rows = xc.numel() // feat
    y, xhat = torch.empty_like(xc), torch.empty_like(xc)
    invstd = torch.empty(rows, dtype=torch.float32, device=xc.device)
    L.check(L.lib.flb200_layernorm_forward(ptr(xc), ptr(weight), ptr(bias), ptr(y), ptr(xhat), None,
                                           ptr(invstd), rows, feat, float(eps), dtype_code(xc),
                                           stream_handle()))
    return y, xhat, invstd


def layernorm_backward(grad_y, xhat, weight, invstd, need_input_grad=True, need_param_grads=True):
    """Returns (grad_x, grad_weight, grad_bias); the parameter gradients are fp32."""
    feat = xhat.shape[-1]
    rows = xhat.numel() // feat
    gy = grad_y.contiguous()
    gx = torch.empty_like(xhat) if need_input_grad else None
    gw = gb = None
    if need_param_grads:
        gw = torch.empty(feat, dtype=torch.float32, device=xhat.device)
        gb = torch.empty(feat, dtype=torch.float32, device=xhat.device)
    nbytes = L.lib.flb200_layernorm_backward_workspace_bytes(rows, feat)
    ws = workspace(nbytes, xhat)
    L.check(L.lib.flb200_layernorm_backward(ptr(gy), ptr(xhat), ptr(weight), ptr(invstd), ptr(gx),
                                            ptr(gw), ptr(gb), rows, feat, dtype_code(xhat), ptr(ws),
                                            nbytes, stream_handle()))
    return gx, gw, gb


def layernorm_affine_backward(grad_y, xhat, weight, need_input_grad=True, need_param_grads=True):
    """Returns (grad_xhat, grad_weight, grad_bias); the parameter gradients are fp32."""
    feat = xhat.shape[-1]
    rows = xhat.numel() // feat
    gy, xh = grad_y.contiguous(), xhat.contiguous()
    gx = torch.empty_like(xh) if need_input_grad else None
    gw = gb = None
    if need_param_grads:
        gw = torch.empty(feat, dtype=torch.float32, device=xh.device)
        gb = torch.empty(feat, dtype=torch.float32, device=xh.device)
    nbytes = L.lib.flb200_layernorm_affine_workspace_bytes(rows, feat)
    ws = workspace(nbytes, xh)
    L.check(L.lib.flb200_layernorm_affine_backward(ptr(gy), ptr(xh), ptr(weight), ptr(gx), ptr(gw),
                                                   ptr(gb), rows, feat, dtype_code(xh), ptr(ws),
                                                   nbytes, stream_handle()))
    return gx, gw, gb


# ------------------------------------------------------------------ linear
def _linear_dims(weight, x):
    I = x.shape[-1]
    cols = x.numel() // I
    O, I_w = weight.shape[1], weight.shape[0]  # fl weight [O, I] is torch (I, O)
    if I_w != I:
        raise ValueError(f"linear: weight expects {I_w} input features, input has {I}")
    return O, I, cols


def linear(x, weight, bias=None, math_mode: Optional[int] = None):
    """fl::linear forward (Functions.cpp:1255-1275): fl weight [O,I] (torch (I,O)), x fl [I,...]."""
    mode = default_math_mode() if math_mode is None else math_mode
    O, I, cols = _linear_dims(weight, x)
    y = torch.empty(tuple(x.shape[:-1]) + (O,), dtype=x.dtype, device=x.device)
    nbytes = L.lib.flb200_linear_workspace_bytes(O, I, cols, 0)
    ws = workspace(nbytes, x)
    L.check(L.lib.flb200_linear_forward(O, I, cols, ptr(weight), ptr(x), ptr(bias), ptr(y), mode,
                                        ptr(ws), nbytes, stream_handle()))
    return y


def linear_bias_act(x, weight, bias, gelu: bool = False, math_mode: Optional[int] = None):
    """y = act(x W + bias) in one kernel (flb200_linear_bias_act_forward): returns (y, pre) with
    pre = x W + bias when gelu is on (None otherwise), or None where the tensor-core path does
    not cover the call and the operators have to run one by one."""
    mode = default_math_mode() if math_mode is None else math_mode
    O, I, cols = _linear_dims(weight, x)
    if O % 32 or not x.is_contiguous() or not weight.is_contiguous() or (
            x.dtype == torch.float32 and mode == L.MATH_STRICT_F32):
        return None
    y = torch.empty(tuple(x.shape[:-1]) + (O,), dtype=x.dtype, device=x.device)
    pre = torch.empty_like(y) if gelu else None
    nbytes = L.lib.flb200_linear_workspace_bytes(O, I, cols, 0)
    ws = workspace(nbytes, x)
    st = L.lib.flb200_linear_bias_act_forward(O, I, cols, ptr(weight), ptr(x), ptr(bias), ptr(y),
                                              ptr(pre), L.ACT_GELU if gelu else L.ACT_NONE,
                                              dtype_code(x), mode, ptr(ws), nbytes, stream_handle())
    if st == L.UNSUPPORTED:
        return None
    L.check(st)
    return y, pre


def linear_backward(x, weight, grad_y, has_bias: bool, need_input_grad=True, need_weight_grad=True,
                    math_mode: Optional[int] = None):
    """The linear gradFunc (Functions.cpp:1277-1305): returns (grad_x, grad_weight, grad_bias)."""
    mode = default_math_mode() if math_mode is None else math_mode
    O, I, cols = _linear_dims(weight, x)
    gx = gw = gb = None
    if has_bias:
        gb = channel_sum(grad_y, cols, O, 1)
    if need_input_grad:
        gx = torch.empty_like(x)
        nbytes = L.lib.flb200_linear_workspace_bytes(O, I, cols, 1)
        ws = workspace(nbytes, x)
        L.check(L.lib.flb200_linear_backward_input(O, I, cols, ptr(weight), ptr(grad_y), ptr(gx),
                                                   mode, ptr(ws), nbytes, stream_handle()))
    if need_weight_grad:
        gw = torch.empty_like(weight)
        nbytes = L.lib.flb200_linear_workspace_bytes(O, I, cols, 2)
        ws = workspace(nbytes, x)
        L.check(L.lib.flb200_linear_backward_weight(O, I, cols, ptr(grad_y), ptr(x), ptr(gw), mode,
                                                    ptr(ws), nbytes, stream_handle()))
    return gx, gw, gb


def matmul(a, b, c=None, *, m, n, k, a_strides, b_strides, c_strides=None, batch=1,
           batch_strides=(0, 0, 0), alpha=1.0, beta=0.0, math_mode: Optional[int] = None):
    """C[m,n] = alpha * A(m,k) B(k,n) + beta * C on strided row-major views (flb200_matmul)."""
    mode = default_math_mode() if math_mode is None else math_mode
    if c is None:
        c = torch.empty((batch, m, n) if batch > 1 else (m, n), dtype=a.dtype, device=a.device)
        c_strides = (n, 1)
        batch_strides = (batch_strides[0], batch_strides[1], m * n)
    d = L.MatmulDesc(m, n, k, batch, a_strides[0], a_strides[1], batch_strides[0], b_strides[0],
                     b_strides[1], batch_strides[1], c_strides[0], c_strides[1], batch_strides[2],
                     alpha, beta, dtype_code(a), mode)
    nbytes = L.lib.flb200_matmul_workspace_bytes(C.byref(d))
    ws = workspace(nbytes, a)
    L.check(L.lib.flb200_matmul(C.byref(d), ptr(a), ptr(b), ptr(c), ptr(ws), nbytes, stream_handle()))
    return c


# --------------------------------------------------- logSoftmax and CE loss
def _cx(x):
    Cc = x.shape[-1]
    return Cc, x.numel() // Cc


def log_softmax(x):
    """fl::logSoftmax(input, 0) (Functions.cpp:1044-1060): over fl dim 0 = torch's last dim."""
    Cc, X = _cx(x)
    y = torch.empty_like(x)
    L.check(L.lib.flb200_log_softmax_forward(ptr(x), ptr(y), Cc, X, dtype_code(x), stream_handle()))
    return y


def log_softmax_backward(y, grad_y):
    Cc, X = _cx(y)
    gx = torch.empty_like(y)
    L.check(L.lib.flb200_log_softmax_backward(ptr(y), ptr(grad_y), ptr(gx), Cc, X, dtype_code(y),
                                              stream_handle()))
    return gx


class CrossEntropyState:
    """What the categoricalCrossEntropy gradFunc captures: targets, kept-target count, mode."""

    def __init__(self, targets, count, reduction, ignore_index):
        self.targets, self.count, self.reduction, self.ignore_index = (
            targets, count, reduction, ignore_index)


def categorical_cross_entropy(logp, targets, reduction: int = L.REDUCE_MEAN, ignore_index: int = -1):
    """fl::categoricalCrossEntropy (Functions.cpp:1078-1154).  Returns (loss, state).
    Raises ValueError when a target lies outside [0, C) and is not ignore_index."""
    Cc, X = _cx(logp)
    if targets.numel() != X:
        raise ValueError("dimension mismatch in categorical cross entropy")
    if targets.dtype != torch.int32:
        targets = targets.to(torch.int32)
    dev = logp.device
    loss = torch.empty(X if reduction == L.REDUCE_NONE else 1, dtype=torch.float32, device=dev)
    meta = torch.zeros(2, dtype=torch.int32, device=dev)  # [count, bad-target flag]
    nbytes = L.lib.flb200_cce_workspace_bytes(X)
    ws = workspace(nbytes, logp)
    L.check(L.lib.flb200_cce_forward(ptr(logp), ptr(targets), ptr(loss), meta.data_ptr(),
                                     meta.data_ptr() + 4, Cc, X, reduction, ignore_index,
                                     dtype_code(logp), ptr(ws), nbytes, stream_handle()))
    state = CrossEntropyState(targets, meta, reduction, ignore_index)
    return loss, state


def check_targets(state: CrossEntropyState) -> None:
    """Host-side read of the bad-target flag (one synchronising copy); the
    reference performs the same check eagerly (Functions.cpp:1100-1107)."""
    if int(state.count[1].item()) != 0:
        raise ValueError("target contains elements out of valid range [0, num_categories) "
                         "in categorical cross entropy")


def categorical_cross_entropy_backward(grad_loss, state: CrossEntropyState, C_classes: int, like):
    X = state.targets.numel()
    gx = torch.empty_like(like)
    L.check(L.lib.flb200_cce_backward(ptr(grad_loss), ptr(state.targets), state.count.data_ptr(),
                                      ptr(gx), C_classes, X, state.reduction, state.ignore_index,
                                      dtype_code(like), stream_handle()))
    return gx


def log_softmax_cross_entropy_backward(y, grad_loss, state: CrossEntropyState):
    """Gradient of categoricalCrossEntropy(logSoftmax(x)) w.r.t. x in one pass."""
    Cc, X = _cx(y)
    gx = torch.empty_like(y)
    L.check(L.lib.flb200_log_softmax_cce_backward(
        ptr(y), ptr(grad_loss), ptr(state.targets), state.count.data_ptr(), ptr(gx), Cc, X,
        state.reduction, state.ignore_index, dtype_code(y), stream_handle()))
    return gx


# ------------------------------------------------------------------ embedding
def _ids(ids):
    if ids.dtype == torch.int64:
        return ids.contiguous(), L.IDS_I64
    if ids.dtype == torch.int32:
        return ids.contiguous(), L.IDS_I32
    raise ValueError("embedding: ids must be int32 or int64")


def embedding(table, ids):
    """fl::embedding forward: rows of `table` (vocab, dim) picked by `ids` (any shape)."""
    flat, code = _ids(ids.reshape(-1))
    vocab, dim = table.shape
    out = torch.empty((flat.numel(), dim), dtype=table.dtype, device=table.device)
    L.check(L.lib.flb200_embedding_forward(ptr(table), ptr(flat), code, ptr(out), flat.numel(), dim,
                                           vocab, dtype_code(table), stream_handle()))
    return out


def embedding_backward(grad_out, ids, vocab: int):
    """Gradient of the table (f32, (vocab, dim)), summed in position order without atomics."""
    flat, code = _ids(ids.reshape(-1))
    g = grad_out.contiguous()
    dim = g.shape[-1]
    table_grad = torch.empty((vocab, dim), dtype=torch.float32, device=g.device)
    L.check(L.lib.flb200_embedding_backward(ptr(g), ptr(flat), code, ptr(table_grad), flat.numel(),
                                            dim, vocab, dtype_code(g), stream_handle()))
    return table_grad


# ------------------------------------------------------------------ attention softmax
def softmax(x, scale: float = 1.0, causal_period: int = 0):
    """softmax over the last dim of scale * x, optionally with the causal mask of stacked
    (period x cols) score matrices folded in."""
    Cc, X = _cx(x)
    y = torch.empty_like(x)
    L.check(L.lib.flb200_softmax_forward(ptr(x), ptr(y), Cc, X, scale, causal_period, dtype_code(x),
                                         stream_handle()))
    return y


def softmax_lse(x, scale: float = 1.0, causal_period: int = 0):
    """softmax as above plus lse[row] = log sum exp(scale * x[row]) (fp32), the only thing the
    fused attention gradient keeps of the scores."""
    Cc, X = _cx(x)
    y = torch.empty_like(x)
    lse = torch.empty(X, dtype=torch.float32, device=x.device)
    L.check(L.lib.flb200_softmax_forward_lse(ptr(x), ptr(y), ptr(lse), Cc, X, scale, causal_period,
                                             dtype_code(x), stream_handle()))
    return y, lse


def attention_backward_supported(q) -> bool:
    return bool(L.lib.flb200_attention_backward_supported(q.shape[1], q.shape[2], dtype_code(q)))


def attention_backward(q, k, v, o, grad_o, lse, scale: float, causal: bool):
    """(dq, dk, dv) of o = softmax(scale * q k^T [+ causal mask]) v in one flash-style kernel;
    q, k, v, o, grad_o (batch * heads, T, head dim) dense, lse (batch * heads * T,) fp32."""
    Z, T, hd = q.shape
    for t in (q, k, v, o, grad_o):
        if tuple(t.shape) != (Z, T, hd) or not t.is_contiguous() or t.dtype != q.dtype:
            raise ValueError("attention_backward: q, k, v, o and grad_o must be dense and alike")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    nbytes = L.lib.flb200_attention_backward_workspace_bytes(Z, T, hd)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    L.check(L.lib.flb200_attention_backward(ptr(q), ptr(k), ptr(v), ptr(o), ptr(grad_o), ptr(lse),
                                            ptr(dq), ptr(dk), ptr(dv), Z, T, hd, float(scale),
                                            1 if causal else 0, dtype_code(q), ptr(ws), nbytes,
                                            stream_handle()))
    return dq, dk, dv


def softmax_backward(y, grad_y, scale: float = 1.0):
    Cc, X = _cx(y)
    gx = torch.empty_like(y)
    L.check(L.lib.flb200_softmax_backward(ptr(y), ptr(grad_y), ptr(gx), Cc, X, scale, dtype_code(y),
                                          stream_handle()))
    return gx
