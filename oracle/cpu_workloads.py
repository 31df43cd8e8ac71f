"""CPU stand-in for the reference's oneDNN training step.  TEST / BASELINE INFRASTRUCTURE ONLY.

The reference's own CPU path (ArrayFire-CPU tensors + OneDnnAutogradExtension) cannot be built
in this image, so the timed CPU baseline is the same operator sequence on torch-CPU (which
links the same oneDNN generation), driven by torch autograd, on all host threads.  ResNet-50
topology: flashlight/pkg/vision/models/Resnet.cpp:67-121, 161-172, 210-230; used by bench.py's
cpu_baseline leg and its `--impl reference` arm.  The restatements of the other four synthetic
workloads (MNIST convnet, conv-ASR, biLSTM, Transformer-LM) further down are the checkers of
tests/test_workloads_gpu.py.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def same_pad(in_sz, k, s):
    """flashlight/fl/nn/Utils.cpp:87-100 with dilation 1."""
    new_pad = (k - 1) - s + 1 if in_sz % s == 0 else (k - 1) - (in_sz % s) + 1
    return max((new_pad + 1) // 2, 0)


def resnet50_loss(params, x, targets, blocks=(3, 4, 6, 3), eps=1e-5):
    """params: flat list of tensors in the order flashlight_b200.workloads.resnet50 creates them
    (conv weight, bn gamma, bn beta, ... , fc weight (I,O), fc bias).  Batch statistics
    (training mode), momentum has no effect on the loss."""
    it = iter(params)

    def conv_bn(h, k, s, relu=True):
        w = next(it)
        g, b = next(it), next(it)
        ph, pw = same_pad(h.shape[-2], k, s), same_pad(h.shape[-1], k, s)
        h = F.conv2d(h, w, None, stride=s, padding=(ph, pw))
        h = F.batch_norm(h, None, None, g, b, True, 0.0, eps)
        return F.relu(h) if relu else h

    h = conv_bn(x, 7, 2)
    p = same_pad(h.shape[-1], 3, 2)
    h = F.max_pool2d(h, 3, 2, p)
    in_c = h.shape[1]
    for i, nb in enumerate(blocks):
        planes = h.shape[1] if (i == 0) else None
        for j in range(nb):
            stride = (1 if i == 0 else 2) if j == 0 else 1
            inp = h
            out = conv_bn(inp, 1, 1)
            out = conv_bn(out, 3, stride)
            out = conv_bn(out, 1, 1, relu=False)
            if inp.shape[1] != out.shape[1] or stride > 1:
                inp = conv_bn(inp, 1, stride, relu=False)
            h = F.relu(out + inp)
    h = F.avg_pool2d(h, 7, 1, 0, count_include_pad=False)
    h = h.reshape(h.shape[0], -1)
    w, b = next(it), next(it)
    scores = h @ w + b
    return F.nll_loss(F.log_softmax(scores, -1), targets.long())


def resnet50_step(params, x, targets, blocks=(3, 4, 6, 3)):
    """One fwd+bwd; returns (loss, grads) with grads in parameter order."""
    ps = [p.detach().clone().requires_grad_(True) for p in params]
    loss = resnet50_loss(ps, x, targets, blocks)
    grads = torch.autograd.grad(loss, ps)
    return loss.detach(), grads


def _step(loss_fn, params, *args):
    ps = [p.detach().clone().requires_grad_(True) for p in params]
    loss = loss_fn(ps, *args)
    grads = torch.autograd.grad(loss, ps)
    return loss.detach(), grads


def mnist_convnet_loss(params, x, targets, dropout_mask, p_drop=0.5):
    """The README convnet (flashlight README.md quick start): conv 5x5 SAME + ReLU + maxpool 2x2
    twice, Linear 3136->1024, ReLU, Dropout (mask given as data, kept values scaled by
    1/(1-p): flashlight/fl/autograd/Functions.cpp:1777-1785), Linear 1024->10, logSoftmax, CE.
    params: conv1 w, b, conv2 w, b, fc1 w (I,O), b, fc2 w (I,O), b."""
    w1, b1, w2, b2, f1, c1, f2, c2 = params
    h = F.max_pool2d(F.relu(F.conv2d(x, w1, b1, padding=2)), 2, 2)
    h = F.max_pool2d(F.relu(F.conv2d(h, w2, b2, padding=2)), 2, 2)
    h = F.relu(h.reshape(h.shape[0], -1) @ f1 + c1)
    h = h * dropout_mask / (1.0 - p_drop)
    return F.nll_loss(F.log_softmax(h @ f2 + c2, -1), targets.long())


def mnist_convnet_step(params, x, targets, dropout_mask):
    return _step(mnist_convnet_loss, params, x, targets, dropout_mask)


def conv_asr_loss(params, x, targets, kw=13, eps=1e-5):
    """x (B, feat, 1, T).  Each layer: Conv2D kW x 1 SAME with bias
    (flashlight/pkg/runtime/common/SequentialBuilder.cpp:215-226), LayerNorm over fl axes
    {0,1,2} = all of (T, 1, C) of one batch element, no affine (:332-350), ReLU; then frames
    become rows (b, t) and a Linear gives class scores; frame-wise mean cross entropy.
    params: (conv w, conv b) per layer, then head w (C, classes), head b."""
    it = iter(params[:-2])
    h = x
    for w in it:
        b = next(it)
        h = F.conv2d(h, w, b, padding=(0, same_pad(h.shape[-1], kw, 1)))
        h = F.relu(F.layer_norm(h, h.shape[1:], None, None, eps))
    B, C, _, T = h.shape
    rows = h.permute(0, 3, 2, 1).reshape(B * T, C)
    scores = rows @ params[-2] + params[-1]
    return F.nll_loss(F.log_softmax(scores, -1), targets.long())


def conv_asr_step(params, x, targets, kw=13):
    return _step(lambda ps, a, b: conv_asr_loss(ps, a, b, kw), params, x, targets)


def bilstm_loss(params, x, target, hidden, layers):
    """x (T, B, I); fl::RNN(I, hidden, layers, LSTM, bidirectional) then mean squared error
    against a dense target (flashlight/fl/nn/modules/Loss.cpp:17-31).  params: the flat weight
    vector."""
    from oracle import flref
    y, _, _ = flref.rnn(x, None, None, params[0], hidden, layers, flref.RNN_LSTM, True)
    return ((y - target) ** 2).mean()


def bilstm_step(params, x, target, hidden, layers):
    return _step(lambda ps, a, b: bilstm_loss(ps, a, b, hidden, layers), params, x, target)


def transformer_lm_loss(params, ids, targets, heads, layers, eps=1e-6):
    """Pre-LayerNorm decoder (flashlight/pkg/vision/nn/VisionTransformer.cpp:169-170 block,
    causal additive mask as flashlight/fl/contrib/modules/Transformer.cpp:112-119, q scaled by
    1/sqrt(head dim), tanh-form GELU).  params in the order of
    flashlight_b200.workloads.TransformerLM.parameters(); Linear weights are (in, out)."""
    it = iter(params)
    embed = next(it)
    B, T = ids.shape
    d = embed.shape[1]
    hd = d // heads
    x = embed[ids.reshape(-1).long()]
    mask = torch.full((T, T), float("-inf"), dtype=x.dtype).triu(1)

    def ln(h):
        w, b = next(it), next(it)
        return F.layer_norm(h, (d,), w, b, eps)

    def lin(h):
        w, b = next(it), next(it)
        return h @ w + b

    for _ in range(layers):
        qkv = lin(ln(x)).reshape(B, T, 3, heads, hd)
        q = qkv[:, :, 0].permute(0, 2, 1, 3) / hd ** 0.5
        k = qkv[:, :, 1].permute(0, 2, 1, 3)
        v = qkv[:, :, 2].permute(0, 2, 1, 3)
        p = torch.softmax(q @ k.transpose(-1, -2) + mask, -1)
        ctx = (p @ v).permute(0, 2, 1, 3).reshape(B * T, d)
        x = x + lin(ctx)
        h = lin(ln(x))
        x = x + lin(F.gelu(h, approximate="tanh"))
    scores = lin(ln(x))
    return F.nll_loss(F.log_softmax(scores, -1), targets.long())


def transformer_lm_step(params, ids, targets, heads, layers):
    return _step(lambda ps, a, b: transformer_lm_loss(ps, a, b, heads, layers), params, ids, targets)
