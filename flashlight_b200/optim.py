"""fl::SGDOptimizer (flashlight/fl/optim/SGDOptimizer.{h,cpp}) over the fused step kernel."""
from __future__ import annotations

from typing import List

import torch

from . import _lib as L
from .autograd import Variable
from .extension import ptr, stream_handle


class SGDOptimizer:
    """Same constructor arguments and update rule as fl::SGDOptimizer(parameters, learningRate,
    momentum, weightDecay, useNesterov).  `step(grad_scale, zero_grad)` applies one update per
    parameter in a single pass (flb200_sgd_step); grad_scale is the 1/world-size of a
    data-parallel average when the all-reduce summed, zero_grad clears the gradients in the
    same pass instead of a separate zeroGrad()."""

    def __init__(self, parameters: List[Variable], learning_rate: float, momentum: float = 0.0,
                 weight_decay: float = 0.0, use_nesterov: bool = False):
        self.parameters = list(parameters)
        self.lr, self.mu, self.wd, self.nesterov = learning_rate, momentum, weight_decay, use_nesterov
        self.velocities = [torch.zeros_like(p.tensor) if momentum != 0 else None
                           for p in self.parameters]

    def step(self, grad_scale: float = 1.0, zero_grad: bool = False) -> None:
        for p, v in zip(self.parameters, self.velocities):
            if p.grad is None:  # isGradAvailable() false: skipped like the reference
                continue
            g = p.grad if p.grad.is_contiguous() else p.grad.contiguous()
            if not p.tensor.is_contiguous():
                raise ValueError("SGDOptimizer: parameters must be contiguous")
            L.check(L.lib.flb200_sgd_step(ptr(p.tensor), ptr(g), ptr(v), p.tensor.numel(), self.lr,
                                          self.mu, self.wd, 1 if self.nesterov else 0, grad_scale,
                                          1 if zero_grad else 0, L.F32, stream_handle()))

    def zeroGrad(self) -> None:
        for p in self.parameters:
            p.zeroGrad()
