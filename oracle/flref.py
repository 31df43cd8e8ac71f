"""CPU oracle for the autograd-backward hot path.  TEST INFRASTRUCTURE ONLY.

Nothing under flashlight_b200/ imports this module; only tests/, the smoke check
and the CPU-baseline leg of bench.py do, as the checker.

What it restates.  The reference computes this path with oneDNN primitives
(flashlight/fl/autograd/tensor/backend/onednn/*.cpp) and with tensor-op chains
in flashlight/fl/autograd/Functions.cpp.  Neither oneDNN nor ArrayFire sources
are part of the reference tree (un-vendored dependencies: oneDNN >= 2.5.2,
ArrayFire >= 3.7.3, floor constraints only) and the reference cannot be built
here, so this oracle restates the published arithmetic of each operator in two
ways: (1) torch CPU functional ops (torch links the same oneDNN generation) in
fp64 or fp32, and (2) plain numpy fp64 loops for small shapes, which pin (1).

Pins (tests/test_oracle_pins.py): the reference's own forward goldens for
RNN / LSTM / GRU (flashlight/fl/test/nn/ModuleTest.cpp:436-555, parsed from the
reference checkout at test time), its closed-form batchnorm / layer-norm checks
(flashlight/fl/test/autograd/AutogradNormalizationTest.cpp:37-226) and its
finite-difference Jacobian protocol (flashlight/fl/test/autograd/AutogradTestUtils.h:33-70).
Parity unpinned (no reference test fixes them): max-pool tie breaking, NaN
propagation in pooling, the meaning of batchnorm's saveVar slot, and the order of
bidirectional pseudo-layers in the flat RNN weight vector; here they follow
torch-CPU / cuDNN conventions.

Tensor convention: torch shape = reversed fl shape (fl is column-major), so an
fl image batch [W,H,C,N] is a torch (N,C,H,W) tensor over the same bytes; fl
linear weight [O,I] is torch (I,O).
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

POOL_MAX, POOL_AVG_INCLUDE_PAD, POOL_AVG_EXCLUDE_PAD = 0, 1, 2
RNN_RELU, RNN_TANH, RNN_LSTM, RNN_GRU = 0, 1, 2, 3
REDUCE_NONE, REDUCE_MEAN, REDUCE_SUM = 0, 1, 2


# ---------------------------------------------------------------- conv2d
def conv_out_dim(i, k, s, p, d):
    """flashlight/fl/autograd/tensor/backend/onednn/Conv2D.cpp:179-188."""
    return 1 + (i + 2 * p - (1 + (k - 1) * d)) // s


def conv2d(x, w, b, sx, sy, px, py, dx, dy, groups):
    """onednn/Conv2D.cpp:155-270 — cross-correlation; strides/padding/dilation are (y, x) pairs
    in oneDNN's NCHW order (Conv2D.cpp:101-105)."""
    return F.conv2d(x, w, None if b is None else b.reshape(-1), stride=(sy, sx), padding=(py, px),
                    dilation=(dy, dx), groups=groups)


def conv2d_backward_data(gy, x_shape, w, sx, sy, px, py, dx, dy, groups):
    """onednn/Conv2D.cpp:272-375."""
    return torch.nn.grad.conv2d_input(x_shape, w, gy, stride=(sy, sx), padding=(py, px),
                                      dilation=(dy, dx), groups=groups)


def conv2d_backward_filter_bias(gy, x, w_shape, has_bias, sx, sy, px, py, dx, dy, groups):
    """onednn/Conv2D.cpp:377-507: (dW, db) with db = sum of gy over batch and pixels."""
    gw = torch.nn.grad.conv2d_weight(x, w_shape, gy, stride=(sy, sx), padding=(py, px),
                                     dilation=(dy, dx), groups=groups)
    gb = gy.sum(dim=(0, 2, 3)) if has_bias else None
    return gw, gb


def conv2d_naive(x, w, b, sx, sy, px, py, dx, dy, groups):
    """Direct fp64 loops written in fl terms (x[W,H,C,N], w[kW,kH,C/g,Cout]); pins conv2d()."""
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(w, dtype=np.float64)
    N, Cin, H, W = x.shape
    Cout, Cg, kH, kW = w.shape
    Ho, Wo = conv_out_dim(H, kH, sy, py, dy), conv_out_dim(W, kW, sx, px, dx)
    y = np.zeros((N, Cout, Ho, Wo))
    coutg = Cout // groups
    for n in range(N):
        for co in range(Cout):
            g = co // coutg
            for p in range(Ho):
                for q in range(Wo):
                    acc = 0.0 if b is None else float(np.asarray(b).reshape(-1)[co])
                    for ci in range(Cg):
                        for r in range(kH):
                            h = p * sy - py + r * dy
                            if h < 0 or h >= H:
                                continue
                            for s in range(kW):
                                ww = q * sx - px + s * dx
                                if ww < 0 or ww >= W:
                                    continue
                                acc += w[co, ci, r, s] * x[n, g * Cg + ci, h, ww]
                    y[n, co, p, q] = acc
    return y


# ---------------------------------------------------------------- pool2d
def pool_out_dim(i, w, s, p):
    """onednn/Pool2D.cpp:100-102."""
    return 1 + (i + 2 * p - w) // s


def pool2d(x, wx, wy, sx, sy, px, py, mode):
    """onednn/Pool2D.cpp:78-176.  torch requires pad <= window/2; larger pads go through
    an explicit pad with -inf / 0, which is the same arithmetic."""
    if mode == POOL_MAX:
        if px * 2 > wx or py * 2 > wy:
            xp = F.pad(x, (px, px, py, py), value=float("-inf"))
            return F.max_pool2d(xp, (wy, wx), (sy, sx), 0)
        return F.max_pool2d(x, (wy, wx), (sy, sx), (py, px))
    include = mode == POOL_AVG_INCLUDE_PAD
    return F.avg_pool2d(x, (wy, wx), (sy, sx), (py, px), count_include_pad=include)


def pool2d_backward(gy, x, wx, wy, sx, sy, px, py, mode):
    """onednn/Pool2D.cpp:178-247 via autograd through pool2d()."""
    xr = x.detach().clone().requires_grad_(True)
    y = pool2d(xr, wx, wy, sx, sy, px, py, mode)
    (gx,) = torch.autograd.grad(y, xr, gy)
    return gx


def pool2d_naive(x, wx, wy, sx, sy, px, py, mode):
    """fp64 loops; returns (y, argmax) with argmax = ky*wx+kx of the FIRST maximal in-bounds
    element in scan order (ky outer, kx inner) — the tie rule of the torch-CPU stand-in."""
    x = np.asarray(x, dtype=np.float64)
    N, Cc, H, W = x.shape
    Ho, Wo = pool_out_dim(H, wy, sy, py), pool_out_dim(W, wx, sx, px)
    y = np.zeros((N, Cc, Ho, Wo))
    arg = np.zeros((N, Cc, Ho, Wo), dtype=np.uint8)
    for p in range(Ho):
        for q in range(Wo):
            vals, pos = [], []
            for ky in range(wy):
                h = p * sy - py + ky
                if h < 0 or h >= H:
                    continue
                for kx in range(wx):
                    ww = q * sx - px + kx
                    if ww < 0 or ww >= W:
                        continue
                    vals.append(x[:, :, h, ww])
                    pos.append(ky * wx + kx)
            v = np.stack(vals, axis=-1)
            if mode == POOL_MAX:
                idx = np.argmax(v, axis=-1)  # first maximal element
                y[:, :, p, q] = np.take_along_axis(v, idx[..., None], -1)[..., 0]
                arg[:, :, p, q] = np.asarray(pos, dtype=np.uint8)[idx]
            else:
                div = wx * wy if mode == POOL_AVG_INCLUDE_PAD else len(pos)
                y[:, :, p, q] = v.sum(-1) / div
    return y, arg


# ------------------------------------------------------------- batchnorm
def batchnorm_geometry(fl_shape, axes):
    """(outer, channels, inner) after flashlight/fl/autograd/tensor/backend/cudnn/BatchNorm.cpp:22-75
    (same rule: backend/onednn/BatchNorm.cpp:40-71)."""
    axes = list(axes)
    if any(a > len(fl_shape) - 1 or a < 0 for a in axes):
        raise ValueError("batchnorm - passed axes exceed the number of dimensions of the input")
    mn, mx = min(axes), max(axes)
    if len(axes) != mx - mn + 1:
        raise ValueError("axis array should be continuous")
    nfeat = int(np.prod([fl_shape[a] for a in axes]))
    total = int(np.prod(fl_shape))
    if mn == 0:
        return total // nfeat, nfeat, 1
    batch = int(np.prod(fl_shape[mx + 1:])) if mx + 1 < len(fl_shape) else 1
    return batch, nfeat, total // (nfeat * batch)


def batchnorm(x, weight, bias, running_mean, running_var, axes, train, momentum, eps):
    """Returns (y, save_mean, save_invstd, new_running_mean, new_running_var).
    Statistics per channel over outer*inner elements, biased variance for the
    normalisation (the closed form the reference tests check:
    test/autograd/AutogradNormalizationTest.cpp:158-189); running stats follow the
    cuDNN rule r = (1-m) r + m * batch with the unbiased variance."""
    fl_shape = tuple(reversed(x.shape))
    outer, Cc, inner = batchnorm_geometry(fl_shape, axes)
    xv = x.reshape(outer, Cc, inner).double()
    g = torch.ones(Cc, dtype=torch.float64) if weight is None else weight.double()
    b = torch.zeros(Cc, dtype=torch.float64) if bias is None else bias.double()
    if train:
        mean = xv.mean(dim=(0, 2))
        var = xv.var(dim=(0, 2), unbiased=False)
        cnt = outer * inner
        new_rm = new_rv = None
        if running_mean is not None:
            new_rm = (1 - momentum) * running_mean.double() + momentum * mean
        if running_var is not None:
            unb = var * cnt / (cnt - 1) if cnt > 1 else var
            new_rv = (1 - momentum) * running_var.double() + momentum * unb
    else:
        mean, var = running_mean.double(), running_var.double()
        new_rm, new_rv = running_mean, running_var
    invstd = 1.0 / torch.sqrt(var + eps)
    y = (xv - mean[None, :, None]) * (invstd * g)[None, :, None] + b[None, :, None]
    return y.reshape(x.shape).to(x.dtype), mean, invstd, new_rm, new_rv


def batchnorm_backward(gy, x, weight, axes, eps):
    """(dx, dgamma, dbeta) of training-mode batchnorm (onednn/BatchNorm.cpp:202-279), closed form."""
    fl_shape = tuple(reversed(x.shape))
    outer, Cc, inner = batchnorm_geometry(fl_shape, axes)
    xv = x.reshape(outer, Cc, inner).double()
    gv = gy.reshape(outer, Cc, inner).double()
    g = torch.ones(Cc, dtype=torch.float64) if weight is None else weight.double()
    mean = xv.mean(dim=(0, 2))
    var = xv.var(dim=(0, 2), unbiased=False)
    invstd = 1.0 / torch.sqrt(var + eps)
    xhat = (xv - mean[None, :, None]) * invstd[None, :, None]
    dbeta = gv.sum(dim=(0, 2))
    dgamma = (gv * xhat).sum(dim=(0, 2))
    m = outer * inner
    dx = (g * invstd)[None, :, None] * (gv - dbeta[None, :, None] / m - xhat * dgamma[None, :, None] / m)
    return dx.reshape(x.shape).to(x.dtype), dgamma, dbeta


# ---------------------------------------------------------------- linear
def linear(x, weight, bias):
    """flashlight/fl/autograd/Functions.cpp:1255-1275: y[O,...] = W[O,I] x[I,...] + tile(b)."""
    y = x @ weight  # torch views: x (..., I), weight (I, O)
    return y if bias is None else y + bias.reshape(-1)


def linear_backward(x, weight, gy, has_bias):
    """Functions.cpp:1277-1305: db = sumAs(dy), dx = W^T dy, dW = dy x^T."""
    I, O = weight.shape
    x2, g2 = x.reshape(-1, I), gy.reshape(-1, O)
    gx = (g2 @ weight.t()).reshape(x.shape)
    gw = x2.t() @ g2
    gb = g2.sum(0) if has_bias else None
    return gx, gw, gb


def embedding(table, ids):
    """flashlight/fl/autograd/Functions.cpp:1707-1749: column ids[r] of the fl table [dim, vocab]
    = row ids[r] of the torch view (vocab, dim)."""
    return table[ids.reshape(-1).long()]


def embedding_backward(grad_out, ids, vocab):
    g = torch.zeros(vocab, grad_out.shape[-1], dtype=grad_out.dtype)
    g.index_add_(0, ids.reshape(-1).long(), grad_out.reshape(-1, grad_out.shape[-1]))
    return g


def layer_norm(x, fl_axes, eps, weight=None, bias=None):
    """fl::LayerNorm (flashlight/fl/nn/modules/LayerNorm.cpp:60-131): batchnorm over the
    complement of the normalised fl axes with momentum 0 (statistics per position of the
    complement axes, biased variance), then the optional affine over the normalised axes.
    x is the torch view (reversed fl shape)."""
    nd = x.dim()
    comp = [a for a in range(nd) if a not in fl_axes]
    y = batchnorm(x, None, None, None, None, comp, True, 0.0, eps)[0] if comp else None
    if y is None:  # every axis normalised: one statistic for the whole tensor
        y = (x - x.mean()) / torch.sqrt(x.var(unbiased=False) + eps)
    if weight is not None:
        y = y * weight + (bias if bias is not None else 0)
    return y


# --------------------------------------------------------- eltwise chains
def relu(x):
    return torch.clamp_min(x, 0)  # fl::max(x, 0.0), Functions.cpp:1787-1789


def relu_backward(x, gy):
    return (x > 0).to(gy.dtype) * gy  # Functions.cpp:329-338


GELU_A, GELU_B = 0.7978845608, 0.044715


def gelu(x):
    """Functions.cpp:1791-1796."""
    return 0.5 * x * (1.0 + torch.tanh(GELU_A * (x + GELU_B * x * x * x)))


def gelu_backward(x, gy):
    xr = x.detach().clone().requires_grad_(True)
    (gx,) = torch.autograd.grad(gelu(xr), xr, gy)
    return gx


def tanh_backward(y, gy):
    return (1 - y * y) * gy  # Functions.cpp:454-463


def dropout_apply(x, mask, p):
    return x * mask * (1.0 / (1.0 - p))  # Functions.cpp:1777-1785


def log_softmax(x):
    """Functions.cpp:1044-1060 over fl dim 0 (torch last dim)."""
    m = x.amax(dim=-1, keepdim=True)
    return x - (torch.log(torch.exp(x - m).sum(-1, keepdim=True)) + m)


def log_softmax_backward(y, gy):
    return gy - torch.exp(y) * gy.sum(-1, keepdim=True)  # Functions.cpp:1062-1067


def categorical_cross_entropy(logp, targets, reduction=REDUCE_MEAN, ignore_index=-1):
    """Functions.cpp:1078-1136.  Returns (loss, denominator)."""
    Cc = logp.shape[-1]
    x = logp.reshape(-1, Cc)
    t = targets.reshape(-1).long()
    bad = ((t < 0) | (t >= Cc)) & (t != ignore_index)
    if bool(bad.any()):
        raise ValueError("target contains elements out of valid range [0, num_categories) "
                         "in categorical cross entropy")
    keep = t != ignore_index
    tt = torch.where(keep, t, torch.zeros_like(t))
    per = -x.gather(1, tt[:, None])[:, 0] * keep.to(x.dtype)
    denom = int(keep.sum())
    if reduction == REDUCE_NONE:
        return per.reshape(targets.shape), denom
    if reduction == REDUCE_MEAN:
        return per.sum().reshape(1) / denom, denom
    return per.sum().reshape(1), denom


def categorical_cross_entropy_backward(grad_loss, logp_shape, targets, reduction=REDUCE_MEAN,
                                       ignore_index=-1, dtype=torch.float32):
    """Functions.cpp:1138-1150: tile(g) * (-(onehot))."""
    Cc = logp_shape[-1]
    t = targets.reshape(-1).long()
    X = t.numel()
    keep = t != ignore_index
    if reduction == REDUCE_NONE:
        g = grad_loss.reshape(X).to(dtype)
    elif reduction == REDUCE_MEAN:
        g = (grad_loss.reshape(1) / int(keep.sum())).to(dtype).expand(X)
    else:
        g = grad_loss.reshape(1).to(dtype).expand(X)
    g = g * keep.to(dtype)
    out = torch.zeros(X, Cc, dtype=dtype)
    tt = torch.where(keep, t, torch.zeros_like(t))
    out.scatter_(1, tt[:, None], -g[:, None])
    return out.reshape(logp_shape)


# ------------------------------------------------------------------- rnn
def rnn_gates(mode):
    return {RNN_RELU: 1, RNN_TANH: 1, RNN_LSTM: 4, RNN_GRU: 3}[mode]


def rnn_num_params(input_size, hidden, layers, mode, bidirectional):
    """flashlight/fl/nn/Utils.cpp:45-84."""
    G, dirs = rnn_gates(mode), 2 if bidirectional else 1
    n = 0
    for l in range(layers):
        In = input_size if l == 0 else hidden * dirs
        n += dirs * (G * hidden * In + G * hidden * hidden + 2 * G * hidden)
    return n


def rnn_unpack(w, input_size, hidden, layers, mode, bidirectional):
    """Flat vector -> list over pseudo-layers of (W_ih, W_hh, b_ih, b_hh): all matrices
    first (layer-major, forward direction then reverse), then all biases
    (backend/onednn/RNN.cpp:66-158)."""
    G, dirs = rnn_gates(mode), 2 if bidirectional else 1
    w = w.reshape(-1)
    mats, off = [], 0
    for l in range(layers):
        In = input_size if l == 0 else hidden * dirs
        for _ in range(dirs):
            wih = w[off:off + G * hidden * In].reshape(G * hidden, In); off += G * hidden * In
            whh = w[off:off + G * hidden * hidden].reshape(G * hidden, hidden); off += G * hidden * hidden
            mats.append((wih, whh))
    out = []
    for (wih, whh) in mats:
        bih = w[off:off + G * hidden]; off += G * hidden
        bhh = w[off:off + G * hidden]; off += G * hidden
        out.append((wih, whh, bih, bhh))
    assert off == w.numel(), (off, w.numel())
    return out


def _cell(mode, gx, h, c, whh, bhh, H):
    """One time step.  gx = W_ih x + b_ih.  Gate order LSTM i,f,g,o; GRU r,z,n with the reset
    gate applied to (W_hn h + b_hn) — the cuDNN / torch definition the reference's forward
    goldens were produced with."""
    gh = h @ whh.t() + bhh
    if mode == RNN_LSTM:
        a = gx + gh
        i, f, g, o = (torch.sigmoid(a[:, :H]), torch.sigmoid(a[:, H:2 * H]),
                      torch.tanh(a[:, 2 * H:3 * H]), torch.sigmoid(a[:, 3 * H:]))
        c2 = f * c + i * g
        return o * torch.tanh(c2), c2
    if mode == RNN_GRU:
        r = torch.sigmoid(gx[:, :H] + gh[:, :H])
        z = torch.sigmoid(gx[:, H:2 * H] + gh[:, H:2 * H])
        n = torch.tanh(gx[:, 2 * H:] + r * gh[:, 2 * H:])
        return (1 - z) * n + z * h, c
    a = gx + gh
    return (torch.relu(a) if mode == RNN_RELU else torch.tanh(a)), c


def rnn(x, hx, cx, w, hidden, layers, mode, bidirectional, dropout=0.0, dropout_mask=None):
    """x (T,B,I); hx/cx (L*dirs,B,H) or None; returns (y (T,B,H*dirs), hy, cy).
    Written with differentiable torch ops so that torch.autograd gives rnn_backward().
    dropout_mask (layers-1, T, B, H*dirs) of 0 / 1: inter-layer dropout as cuDNN applies it
    (flashlight/fl/autograd/tensor/backend/cudnn/RNN.cpp:83-85): the input of every layer but
    the first is mask * value / (1 - dropout)."""
    T, B, I = x.shape
    dirs = 2 if bidirectional else 1
    params = rnn_unpack(w, I, hidden, layers, mode, bidirectional)
    inp = x
    hys, cys = [], []
    for l in range(layers):
        outs = []
        for d in range(dirs):
            p = l * dirs + d
            wih, whh, bih, bhh = params[p]
            h = hx[p] if hx is not None else x.new_zeros(B, hidden)
            c = cx[p] if cx is not None else x.new_zeros(B, hidden)
            gx_all = inp @ wih.t() + bih
            hs = [None] * T
            order = range(T) if d == 0 else range(T - 1, -1, -1)
            for t in order:
                h, c = _cell(mode, gx_all[t], h, c, whh, bhh, hidden)
                hs[t] = h
            outs.append(torch.stack(hs, 0))
            hys.append(h)
            cys.append(c)
        inp = torch.cat(outs, dim=-1)
        if dropout_mask is not None and l < layers - 1:
            inp = inp * dropout_mask[l].to(inp.dtype) / (1.0 - dropout)
    hy = torch.stack(hys, 0)
    cy = torch.stack(cys, 0) if mode == RNN_LSTM else None
    return inp, hy, cy


def rnn_backward(x, hx, cx, w, hidden, layers, mode, bidirectional, gy, ghy, gcy, dropout=0.0,
                 dropout_mask=None):
    """(dx, dhx, dcx, dw) by autograd through rnn(); absent output gradients count as zero
    (flashlight/fl/autograd/tensor/backend/cudnn/RNN.cpp:269-272)."""
    xr = x.detach().clone().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    hr = hx.detach().clone().requires_grad_(True) if hx is not None else None
    cr = cx.detach().clone().requires_grad_(True) if cx is not None else None
    y, hy, cy = rnn(xr, hr, cr, wr, hidden, layers, mode, bidirectional, dropout, dropout_mask)
    total = (y * (gy if gy is not None else 0)).sum()
    if ghy is not None:
        total = total + (hy * ghy).sum()
    if gcy is not None and cy is not None:
        total = total + (cy * gcy).sum()
    ins = [xr, wr] + ([hr] if hr is not None else []) + ([cr] if cr is not None else [])
    grads = torch.autograd.grad(total, ins, allow_unused=True)
    dx, dw = grads[0], grads[1]
    k = 2
    dhx = dcx = None
    if hr is not None:
        dhx = grads[k]; k += 1
    if cr is not None:
        dcx = grads[k]
        if dcx is None:
            dcx = torch.zeros_like(cr)
    return dx, dhx, dcx, dw


def sgd_step(p, g, v, lr, momentum, weight_decay, nesterov, grad_scale=1.0):
    """flashlight/fl/optim/SGDOptimizer.cpp:38-68 on one parameter; returns (p, v)."""
    g = g * grad_scale + weight_decay * p
    if momentum != 0:
        v = momentum * v + g
        g = g + momentum * v if nesterov else v
    return p - lr * g, v
