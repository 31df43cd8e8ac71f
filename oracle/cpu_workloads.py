"""CPU stand-in for the reference's oneDNN training step.  TEST / BASELINE INFRASTRUCTURE ONLY.

The reference's own CPU path (ArrayFire-CPU tensors + OneDnnAutogradExtension) cannot be built
in this image, so the timed CPU baseline is the same operator sequence on torch-CPU (which
links the same oneDNN generation), driven by torch autograd, on all host threads.  Topology:
flashlight/pkg/vision/models/Resnet.cpp:67-121, 161-172, 210-230.  Used by bench.py's
cpu_baseline leg and its `--impl reference` arm, and by the end-to-end parity test.
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
