"""The handful of Flashlight modules the five benchmark workloads are made of,
restated over autograd.py so that the workloads execute the same operator
sequence, with the same parameter shapes and initialisers, as the reference's
fl::Sequential models.  Not a module library: only what the workloads name.

Parameter tensors use the torch-order convention of extension.py (reversed fl
shape): Conv2D weight (Cout, Cin/g, kH, kW); Linear weight (I, O).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from . import _lib as L
from . import autograd as A
from .autograd import Variable

SAME = -1  # fl::PaddingMode::SAME


def derive_padding(in_sz: int, filter_sz: int, stride: int, pad: int, dilation: int) -> int:
    """flashlight/fl/nn/Utils.cpp:87-100."""
    if pad == SAME:
        if in_sz % stride == 0:
            new_pad = (filter_sz - 1) * dilation - stride + 1
        else:
            new_pad = (filter_sz - 1) * dilation - (in_sz % stride) + 1
        return max((new_pad + 1) // 2, 0)
    return pad


def _uniform(shape, bound, gen, device):
    return ((torch.rand(shape, generator=gen, dtype=torch.float32) * 2 - 1) * bound).to(device)


class Module:
    def __init__(self):
        self.params: List[Variable] = []
        self.children: List["Module"] = []
        self.train_mode = True

    def parameters(self) -> List[Variable]:
        out = list(self.params)
        for c in self.children:
            out.extend(c.parameters())
        return out

    def zeroGrad(self):
        for p in self.parameters():
            p.zeroGrad()

    def train(self, mode=True):
        self.train_mode = mode
        for c in self.children:
            c.train(mode)

    def __call__(self, x, **kwargs):
        return self.forward(x, **kwargs)


class Sequential(Module):
    def __init__(self, *mods):
        super().__init__()
        self.children = list(mods)

    def add(self, m):
        self.children.append(m)

    def forward(self, x):
        for m in self.children:
            x = m(x)
        return x


class Conv2D(Module):
    """fl::Conv2D (flashlight/fl/nn/modules/Conv2D.cpp:142-194): kaiming-uniform weight with
    fan-in kW*kH*Cin/groups, bias U(+-sqrt(1/fan_in))."""

    def __init__(self, n_in, n_out, wx, wy, sx=1, sy=1, px=0, py=0, dx=1, dy=1, bias=True, groups=1,
                 gen=None, device="cuda", channels_last_out=None, stats=False):
        super().__init__()
        self.cfg = (n_in, n_out, wx, wy, sx, sy, px, py, dx, dy, groups)
        # True where a batch-norm over the channels follows: the convolution's epilogue takes
        # the batch-norm's statistics (autograd.conv2d)
        self.stats = stats
        # True on a network's first convolution: its output, and with it every activation
        # downstream, is stored channels-last (see extension.py)
        self.channels_last_out = channels_last_out
        fan_in = wx * wy * n_in // groups
        bound = math.sqrt(3.0) * math.sqrt(1.0 / fan_in)
        self.params.append(Variable(_uniform((n_out, n_in // groups, wy, wx), bound, gen, device), True))
        if bias:
            self.params.append(Variable(_uniform((n_out,), math.sqrt(1.0 / fan_in), gen, device), True))

    def forward(self, x):
        n_in, n_out, wx, wy, sx, sy, px, py, dx, dy, groups = self.cfg
        H, W = x.tensor.shape[-2], x.tensor.shape[-1]
        px = derive_padding(W, wx, sx, px, dx)
        py = derive_padding(H, wy, sy, py, dy)
        b = self.params[1] if len(self.params) > 1 else None
        return A.conv2d(x, self.params[0], b, sx, sy, px, py, dx, dy, groups,
                        channels_last_out=self.channels_last_out, stats=self.stats)


class Linear(Module):
    """fl::Linear (flashlight/fl/nn/modules/Linear.cpp:52-74)."""

    def __init__(self, n_in, n_out, bias=True, gen=None, device="cuda"):
        super().__init__()
        bound = math.sqrt(3.0) * math.sqrt(1.0 / n_in)
        self.params.append(Variable(_uniform((n_in, n_out), bound, gen, device), True))
        if bias:
            self.params.append(Variable(_uniform((n_out,), math.sqrt(1.0 / n_in), gen, device), True))

    def forward(self, x):
        return A.linear(x, self.params[0], self.params[1] if len(self.params) > 1 else None)


class BatchNorm(Module):
    """fl::BatchNorm(featAxis, featSize) (flashlight/fl/nn/modules/BatchNorm.cpp:15-111):
    gamma ~ U(0,1), beta = 0, running mean 0 / var 1, momentum 0.1, eps 1e-5."""

    def __init__(self, feat_axes, feat_size, momentum=0.1, eps=1e-5, affine=True, gen=None,
                 device="cuda"):
        super().__init__()
        self.axes = [feat_axes] if isinstance(feat_axes, int) else list(feat_axes)
        self.momentum, self.eps = momentum, eps
        if affine:
            self.params.append(Variable(
                torch.rand(feat_size, generator=gen, dtype=torch.float32).to(device), True))
            self.params.append(Variable(torch.zeros(feat_size, device=device), True))
        self.running_mean = torch.zeros(feat_size, device=device)
        self.running_var = torch.ones(feat_size, device=device)

    def forward(self, x, relu=False, addend=None):
        """relu=True: the module's output is relu(batchnorm(x)), computed as one operator;
        with `addend` it is relu(batchnorm(x) + addend), a residual block's tail."""
        w = self.params[0] if self.params else None
        b = self.params[1] if self.params else None
        if addend is not None:
            return A.batchnorm_add_relu(x, addend, w, b, self.running_mean, self.running_var,
                                        self.axes, self.train_mode, self.momentum, self.eps)
        return A.batchnorm(x, w, b, self.running_mean, self.running_var, self.axes, self.train_mode,
                           self.momentum, self.eps, relu=relu)


class BatchNormReLU(BatchNorm):
    """fl::BatchNorm followed by fl::ReLU as one operator (same parameters and statistics)."""

    def forward(self, x, relu=True, addend=None):
        return super().forward(x, relu=relu, addend=addend)


class LayerNorm(Module):
    """fl::LayerNorm (flashlight/fl/nn/modules/LayerNorm.cpp:42-131): batchnorm over the
    complement of the normalised axes with momentum 0, then a separate affine over the
    normalised axes when affine is on.  Only the no-affine form and the full-size affine that
    the workloads use are built here; the affine is applied by the caller's modules."""

    def __init__(self, axes, ndim, eps=1e-5):
        super().__init__()
        self.axes_complement = [a for a in range(ndim) if a not in axes]
        self.eps = eps

    def forward(self, x):
        nd = x.tensor.dim()
        comp = [a for a in self.axes_complement if a < nd]
        return A.batchnorm(x, None, None, None, None, comp, True, 0.0, self.eps)


class ReLU(Module):
    def forward(self, x):
        return A.relu(x)


class GELU(Module):
    def forward(self, x):
        return A.gelu(x)


class Pool2D(Module):
    def __init__(self, wx, wy, sx, sy, px, py, mode=L.POOL_MAX):
        super().__init__()
        self.cfg = (wx, wy, sx, sy, px, py, mode)

    def forward(self, x):
        wx, wy, sx, sy, px, py, mode = self.cfg
        H, W = x.tensor.shape[-2], x.tensor.shape[-1]
        px = derive_padding(W, wx, sx, px, 1)
        py = derive_padding(H, wy, sy, py, 1)
        return A.pool2d(x, wx, wy, sx, sy, px, py, mode)


class View(Module):
    def __init__(self, shape):
        super().__init__()
        self.shape = shape

    def forward(self, x):
        return A.view(x, self.shape)


class Dropout(Module):
    """fl::Dropout with the mask supplied as data.  With a host generator the mask is drawn on
    the host, so that a run is reproducible on both sides of a parity test; without one it comes
    from the library's counter-based device generator (flb200_bernoulli_mask): nothing crosses
    the bus and the step can be captured as a CUDA graph (every replay of one captured graph
    then applies the mask of the captured offsets)."""

    def __init__(self, p, gen=None):
        super().__init__()
        self.p, self.gen = p, gen

    def forward(self, x):
        if not self.train_mode or self.p == 0:
            return x
        if self.gen is None:
            from .extension import bernoulli_mask
            mask = bernoulli_mask(tuple(x.tensor.shape), 1.0 - self.p, x.tensor.device,
                                  x.tensor.dtype)
            return A.dropout(x, self.p, mask)
        mask = (torch.rand(x.tensor.shape, generator=self.gen) > self.p).to(x.tensor.dtype)
        return A.dropout(x, self.p, mask.to(x.tensor.device))


class LogSoftmax(Module):
    def forward(self, x):
        return A.log_softmax(x)
