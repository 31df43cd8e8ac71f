"""The synthetic benchmark workloads: the reference's model definitions restated
operator for operator over the B200 kernels (nn.py / autograd.py).

  mnist_convnet   README MNIST convnet (reference README.md quick-start model)
  resnet50        flashlight/pkg/vision/models/Resnet.cpp:67-121, 161-172, 210-230
  conv_asr        12 x (Conv2D k=13x1 SAME, LayerNorm{0,1,2}, ReLU) + Linear + CE
                  (flashlight/pkg/runtime/common/SequentialBuilder.cpp:215-226, 332-350)
  bilstm          fl::RNN(80, 1024, 3, LSTM, bidirectional) + MSE
  TransformerLM   12 pre-LayerNorm decoder blocks, d = 768, 12 heads, FFN 3072, vocabulary
                  32000, causal mask; fp32 / TF32 or bf16 compute with fp32 master weights

Each builder returns a model whose `loss(inputs, targets)` builds the tape and
returns the scalar loss Variable; `loss(...).backward()` is the measured step.
"""
from __future__ import annotations

import math
import os
from typing import List, Optional

import torch

from . import _lib as L
from . import autograd as A
from . import functions as F
from . import nn
from .autograd import Variable


# Operator fusions of the ResNet block: relu(out + shortcut) as one kernel with a one-kernel
# gradient (autograd.add_relu), and relu(batchnorm(x)) as one operator (autograd.batchnorm
# with relu=True).  FLB200_FUSE=0 keeps the reference's operator-by-operator chain.
FUSE_RESIDUAL_RELU = os.environ.get("FLB200_FUSE", "1") not in ("0", "false")
FUSE_BATCHNORM_RELU = FUSE_RESIDUAL_RELU
# Activations stored channels-last from the first convolution's output on (the layout the
# tensor-core convolutions read natively: no layout copies anywhere in the step).
# FLB200_CHANNELS_LAST=0 keeps every tensor in fl's own [W,H,C,N] order.
CHANNELS_LAST = os.environ.get("FLB200_CHANNELS_LAST", "1") not in ("0", "false")


class Bottleneck(nn.Module):
    """ResNetBottleneckBlock (Resnet.cpp:67-121): 1x1, 3x3 (carries the stride), 1x1 x4,
    BatchNorm after each, ReLU after the first two and after the residual add."""

    def __init__(self, in_c, planes, stride, gen, device):
        super().__init__()
        out_c = planes * 4
        mk = lambda i, o, k, s: nn.Conv2D(i, o, k, k, s, s, nn.SAME, nn.SAME, 1, 1, False, 1, gen, device,
                                         stats=True)  # every convolution here feeds a batch-norm
        self.c1, self.b1 = mk(in_c, planes, 1, 1), nn.BatchNorm(2, planes, gen=gen, device=device)
        self.c2, self.b2 = mk(planes, planes, 3, stride), nn.BatchNorm(2, planes, gen=gen, device=device)
        self.c3, self.b3 = mk(planes, out_c, 1, 1), nn.BatchNorm(2, out_c, gen=gen, device=device)
        self.children = [self.c1, self.b1, self.c2, self.b2, self.c3, self.b3]
        self.down = None
        if in_c != out_c or stride > 1:
            self.down = nn.Sequential(mk(in_c, out_c, 1, stride),
                                      nn.BatchNorm(2, out_c, gen=gen, device=device))
            self.children.append(self.down)

    def forward(self, x):
        if FUSE_BATCHNORM_RELU:
            out = self.b1(self.c1(x), relu=True)
            out = self.b2(self.c2(out), relu=True)
        else:
            out = A.relu(self.b1(self.c1(x)))
            out = A.relu(self.b2(self.c2(out)))
        shortcut = self.down(x) if self.down is not None else x
        if FUSE_BATCHNORM_RELU:
            return self.b3(self.c3(out), addend=shortcut)
        out = self.b3(self.c3(out))
        if FUSE_RESIDUAL_RELU:
            return A.add_relu(out, shortcut)
        return A.relu(A.add(out, shortcut))


class ClassifierModel(nn.Module):
    """A trunk that ends in class scores [classes, batch]; loss = mean CE of logSoftmax."""

    def __init__(self, trunk: nn.Module, fused_loss: bool = True):
        super().__init__()
        self.trunk = trunk
        self.children = [trunk]
        self.fused_loss = fused_loss

    def forward(self, x: Variable) -> Variable:
        return self.trunk(x)

    def loss(self, x: torch.Tensor, targets: torch.Tensor) -> Variable:
        scores = self.forward(Variable(x, False))
        if self.fused_loss:
            return A.log_softmax_cross_entropy(scores, targets)
        return A.categorical_cross_entropy(A.log_softmax(scores), targets)


def resnet50(seed: int = 1234, device: str = "cuda", blocks=(3, 4, 6, 3), classes: int = 1000,
             width: int = 64, channels_last: Optional[bool] = None) -> ClassifierModel:
    """resnet50() of Resnet.cpp:210-230; `blocks` / `width` only shrink it for tests.
    channels_last (default: CHANNELS_LAST): the stem takes the images in fl's order and every
    activation after it is stored channels-last; parameters and their gradients keep the
    reference's layout either way."""
    gen = torch.Generator().manual_seed(seed)
    if channels_last is None:
        channels_last = CHANNELS_LAST
    m = nn.Sequential()
    m.add(nn.Conv2D(3, width, 7, 7, 2, 2, nn.SAME, nn.SAME, 1, 1, False, 1, gen, device,
                    channels_last_out=True if channels_last else None, stats=True))
    if FUSE_BATCHNORM_RELU:
        m.add(nn.BatchNormReLU(2, width, gen=gen, device=device))
    else:
        m.add(nn.BatchNorm(2, width, gen=gen, device=device))
        m.add(nn.ReLU())
    m.add(nn.Pool2D(3, 3, 2, 2, nn.SAME, nn.SAME, L.POOL_MAX))
    in_c = width
    for i, nb in enumerate(blocks):
        planes = width * (2 ** i)
        for j in range(nb):
            m.add(Bottleneck(in_c, planes, (1 if i == 0 else 2) if j == 0 else 1, gen, device))
            in_c = planes * 4
    m.add(nn.Pool2D(7, 7, 1, 1, 0, 0, L.POOL_AVG_EXCLUDE_PAD))
    m.add(nn.View((-1, in_c)))
    m.add(nn.Linear(in_c, classes, True, gen, device))
    return ClassifierModel(m)


def mnist_convnet(seed: int = 1234, device: str = "cuda",
                  device_dropout: bool = False) -> ClassifierModel:
    """Conv 1->32 5x5 SAME, ReLU, MaxPool 2x2/2, Conv 32->64 5x5 SAME, ReLU, MaxPool 2x2/2,
    View 3136, Linear 3136->1024, ReLU, Dropout(0.5), Linear 1024->10, LogSoftmax.
    device_dropout: draw the dropout masks on the device (no host generator, see nn.Dropout)."""
    gen = torch.Generator().manual_seed(seed)
    m = nn.Sequential(
        nn.Conv2D(1, 32, 5, 5, 1, 1, nn.SAME, nn.SAME, 1, 1, True, 1, gen, device), nn.ReLU(),
        nn.Pool2D(2, 2, 2, 2, 0, 0, L.POOL_MAX),
        nn.Conv2D(32, 64, 5, 5, 1, 1, nn.SAME, nn.SAME, 1, 1, True, 1, gen, device), nn.ReLU(),
        nn.Pool2D(2, 2, 2, 2, 0, 0, L.POOL_MAX),
        nn.View((-1, 7 * 7 * 64)),
        nn.Linear(7 * 7 * 64, 1024, True, gen, device), nn.ReLU(),
        nn.Dropout(0.5, None if device_dropout else gen),
        nn.Linear(1024, 10, True, gen, device))
    return ClassifierModel(m, fused_loss=False)


class ConvAsr(nn.Module):
    """Input fl [T,1,feat,B]; 12 x (Conv2D kW=13 kH=1 SAME + bias, LayerNorm over fl axes
    {0,1,2}, ReLU); then per-frame Linear channels->classes and frame-wise cross entropy."""

    def __init__(self, feat=80, channels=1024, layers=12, classes=30, kw=13, seed=1234, device="cuda"):
        super().__init__()
        gen = torch.Generator().manual_seed(seed)
        self.convs = [nn.Conv2D(feat if i == 0 else channels, channels, kw, 1, 1, 1, nn.SAME, 0, 1, 1,
                                True, 1, gen, device) for i in range(layers)]
        self.ln = nn.LayerNorm([0, 1, 2], 4)
        self.head = nn.Linear(channels, classes, True, gen, device)
        self.children = self.convs + [self.head]
        self.channels, self.classes = channels, classes

    def loss(self, x: torch.Tensor, targets: torch.Tensor) -> Variable:
        h = Variable(x, False)  # torch (B, feat, 1, T)
        for conv in self.convs:
            h = A.relu(self.ln(conv(h)))
        B, Cc, _, T = h.tensor.shape
        # frames as columns: fl reorder to [C, T, B]; done with a torch permute copy, which is
        # data movement outside the measured operators' arithmetic
        ht = Variable(h.tensor.permute(0, 3, 2, 1).contiguous().reshape(B * T, Cc), False)
        hv = _ReorderBridge.apply(h, ht)
        scores = self.head(hv)
        return A.log_softmax_cross_entropy(scores, targets)


class _ReorderBridge:
    """fl::reorder between the conv stack and the per-frame Linear (Functions.cpp:513-535):
    forward and gradient are pure permutations of the same values."""

    @staticmethod
    def apply(src: Variable, dst: Variable) -> Variable:
        B, Cc, _, T = src.tensor.shape

        def grad_func(inputs, gy):
            g = gy.reshape(B, T, 1, Cc).permute(0, 3, 2, 1).contiguous()
            inputs[0].addGrad(g)

        return Variable(dst.tensor, False, [src], grad_func)


class BiLstm(nn.Module):
    """fl::RNN(80, 1024, 3, LSTM, bidirectional=true) + MSE against a dense target."""

    def __init__(self, input_size=80, hidden=1024, layers=3, seed=1234, device="cuda"):
        super().__init__()
        gen = torch.Generator().manual_seed(seed)
        d = L.RnnDesc(input_size, hidden, layers, 1, 1, L.RNN_LSTM, 1, L.F32, 0)
        import ctypes as C
        n = int(L.lib.flb200_rnn_num_params(C.byref(d)))
        bound = 1.0 / math.sqrt(hidden)  # flashlight/fl/nn/modules/RNN.cpp:58-65
        w = ((torch.rand(n, generator=gen, dtype=torch.float32) * 2 - 1) * bound).to(device)
        self.params = [Variable(w, True)]
        self.hidden, self.layers = hidden, layers

    def loss(self, x: torch.Tensor, target: torch.Tensor) -> Variable:
        y, _, _ = A.rnn(Variable(x, False), None, None, self.params[0], self.hidden, self.layers,
                        L.RNN_LSTM, True)
        return mse(y, target)


def mse(y: Variable, target: torch.Tensor) -> Variable:
    """fl::MeanSquaredError (flashlight/fl/nn/modules/Loss.cpp:17-31): mean over all elements of
    (y - t)^2; gradient 2 (y - t) / n.  Built from flb200 kernels: add with a negated target,
    then the scalar reduction through channel_sum."""
    n = y.tensor.numel()
    diff = F.add(y.tensor, -target)  # negation of the constant target is input preparation
    sq = F.dropout_apply(diff, diff, 0.0)  # diff * diff * 1
    total = F.channel_sum(sq.reshape(-1), 1, 1, n)  # one channel, n contiguous elements

    def grad_func(inputs, gl):
        # d/dy = 2 (y - t) / n * gl ; gl is a device scalar of ones in the benchmark
        scale = torch.full_like(diff, 2.0 / n)
        g = F.dropout_apply(diff, scale, 0.0)
        inputs[0].addGrad(F.dropout_apply(g, gl.expand_as(g).contiguous(), 0.0))

    loss = Variable(total / n, False, [y], grad_func)
    return loss


def _reorder(t: torch.Tensor, shape, perm) -> torch.Tensor:
    """t.reshape(shape).permute(perm), contiguous: the library's reorder kernel where its
    16-byte rules hold, a torch copy otherwise."""
    t = t.contiguous()
    out = F.reorder(t, tuple(shape), tuple(perm))
    return out if out is not None else t.reshape(shape).permute(perm).contiguous()


class TransformerLM(nn.Module):
    """Decoder-only language model of the fifth benchmark configuration: token embedding,
    `layers` pre-LayerNorm blocks (x += attn(LN1(x)); x += mlp(LN2(x)), the block of
    flashlight/pkg/vision/nn/VisionTransformer.cpp:169-170 with LayerNorm eps 1e-6 and affine),
    multi-head attention with a causal additive mask and q scaled by 1/sqrt(head dim)
    (flashlight/fl/contrib/modules/Transformer.cpp:112-119, Functions.cpp:1828-1891), mlp =
    w2(gelu(w1 x)) with the tanh-form GELU (Functions.cpp:1791-1796), a final LayerNorm, an
    untied output projection and full-softmax cross entropy.

    Runs in fp32 / TF32, or with compute_dtype=torch.bfloat16 (bf16 activations and matrix
    operands, fp32 accumulation, fp32 master weights).  The contractions (q k v projections, scores, context, output and mlp
    projections, vocabulary projection and all their gradients), LayerNorm statistics, GELU,
    logSoftmax, the loss, the residual adds and the embedding lookup with its scatter-add
    gradient and the scaled causal softmax run on this library's kernels; head split / merge
    permutations are torch data movement (autograd.glue); nothing arithmetic is left to torch."""

    def __init__(self, vocab=32000, d=768, heads=12, ffn=3072, layers=12, seed=1234, device="cuda",
                 compute_dtype=torch.float32):
        super().__init__()
        gen = torch.Generator().manual_seed(seed)
        self.d, self.heads, self.layers = d, heads, layers
        # bf16 compute with fp32 master weights: parameters stay fp32; the matrices and the
        # embedding are cast to bf16 where they are used and their gradients come back as fp32
        # (autograd.cast); biases and LayerNorm parameters are used in fp32 by the kernels or
        # cast likewise; the class scores are cast to fp32 for the loss.
        self.compute_dtype = compute_dtype
        mk = lambda i, o: nn.Linear(i, o, True, gen, device)
        ones = lambda n: Variable(torch.ones(n, device=device), True)
        zeros = lambda n: Variable(torch.zeros(n, device=device), True)
        self.embed = Variable((torch.randn(vocab, d, generator=gen) * 0.02).to(device), True)
        self.params = [self.embed]
        self.blocks = []
        for _ in range(layers):
            blk = {"ln1": (ones(d), zeros(d)), "qkv": mk(d, 3 * d), "proj": mk(d, d),
                   "ln2": (ones(d), zeros(d)), "w1": mk(d, ffn), "w2": mk(ffn, d)}
            self.blocks.append(blk)
            self.params += list(blk["ln1"]) + list(blk["ln2"])
            self.children += [blk["qkv"], blk["proj"], blk["w1"], blk["w2"]]
        self.ln_f = (ones(d), zeros(d))
        self.params += list(self.ln_f)
        self.head = mk(d, vocab)
        self.children.append(self.head)
        self.norm = nn.LayerNorm([0], 2, eps=1e-6)

    def parameters(self):
        """embedding; per block ln1 w, b, qkv w, b, proj w, b, ln2 w, b, w1 w, b, w2 w, b;
        final LayerNorm w, b; head w, b."""
        out = [self.embed]
        for blk in self.blocks:
            out += list(blk["ln1"]) + blk["qkv"].parameters() + blk["proj"].parameters()
            out += list(blk["ln2"]) + blk["w1"].parameters() + blk["w2"].parameters()
        return out + list(self.ln_f) + self.head.parameters()

    def _ln(self, x, wb):
        # one kernel forward, two backward; the operator chain (normalisation, then the affine
        # part) where the fused operator declines
        y = A.layernorm(x, wb[0], wb[1], 1e-6)
        return y if y is not None else A.affine_rows(self.norm(x), wb[0], wb[1])

    def _lin(self, mod, x, gelu=False):
        w = A.cast(mod.params[0], self.compute_dtype)
        return A.linear(x, w, mod.params[1], gelu=gelu)

    def _attention(self, x, blk, B, T, mask):
        d, h = self.d, self.heads
        hd = d // h
        qkv = self._lin(blk["qkv"], x)  # (B*T, 3d)

        # pure data movement (fl::reorder with the head vectors kept whole): one copy brings the
        # head index forward for q, k and v together, (B*T, 3d) -> (3, B*h, T, hd); their
        # gradients travel back the same way in one copy
        q, k, v = A.unbind(
            qkv,
            lambda t: _reorder(t, (B, T, 3, h, hd), (2, 0, 3, 1, 4)).reshape(3, B * h, T, hd),
            lambda g: _reorder(g, (3, B, h, T, hd), (1, 3, 0, 2, 4)).reshape(B * T, 3 * d), 3)
        # scores (B*h, T, T) -> softmax with the scale 1/sqrt(head dim) and the causal mask folded
        # in -> context (B*h, T, hd); the gradient is the fused kernel where it is built (bf16,
        # head dim 64, T a multiple of 128), which keeps no T x T tensor for the backward pass
        ctx = A.attention(q, k, v, 1.0 / math.sqrt(hd), causal=True)
        merged = A.glue(
            ctx, lambda t: _reorder(t, (B, h, T, hd), (0, 2, 1, 3)).reshape(B * T, d),
            lambda g: _reorder(g, (B, T, h, hd), (0, 2, 1, 3)).reshape(B * h, T, hd))
        return self._lin(blk["proj"], merged)

    def loss(self, ids: torch.Tensor, targets: torch.Tensor) -> Variable:
        """ids (B, T) token ids; targets (B*T,) next-token labels."""
        B, T = ids.shape
        x = A.embedding(A.cast(self.embed, self.compute_dtype), ids)  # (B*T, d)
        mask = None
        for blk in self.blocks:
            x = A.add(x, self._attention(self._ln(x, blk["ln1"]), blk, B, T, mask))
            h = self._lin(blk["w1"], self._ln(x, blk["ln2"]), gelu=True)  # Linear + bias + GELU
            x = A.add(x, self._lin(blk["w2"], h))
        scores = A.cast(self._lin(self.head, self._ln(x, self.ln_f)), torch.float32)
        return A.log_softmax_cross_entropy(scores, targets)
