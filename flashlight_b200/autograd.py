"""A minimal restatement of Flashlight's autograd tape, just enough to drive the
five benchmark workloads through the B200 kernels the way fl::Variable does.

Variable mirrors flashlight/fl/autograd/Variable.cpp:185-294 (shared grad,
addGrad accumulation, reverse-topological backward, grad hooks fired once the
gradient of a leaf is complete).  The differentiable functions mirror the ones in
flashlight/fl/autograd/Functions.cpp that sit on the backward hot path; each
builds its result with flb200 kernels and registers a gradFunc closure that calls
the matching backward kernels.  This file holds no arithmetic of its own.
"""
from __future__ import annotations

import os
from typing import Callable, List, Optional, Sequence

import torch

from . import _lib as L
from . import functions as F
from .extension import (AutogradPayload, B200AutogradExtension, RNNGradData, is_dense,
                        same_layout)

_ext: Optional[B200AutogradExtension] = None


# FLB200_CONV_STATS=0: batch-norm always runs its own statistics pass
CONV_STATS_ON = os.environ.get("FLB200_CONV_STATS", "1") != "0"
# FLB200_FUSED_LAYERNORM=0: layernorm() declines, callers run normalisation + affine_rows
LAYERNORM_FUSED_OFF = os.environ.get("FLB200_FUSED_LAYERNORM", "1") == "0"
# FLB200_FUSED_LINEAR=0: linear() runs contraction, bias and activation as separate kernels
LINEAR_FUSED_ON = os.environ.get("FLB200_FUSED_LINEAR", "1") != "0"
# FLB200_FUSED_ATTENTION=0: attention() runs the operator chain (matmul, softmax, matmul)
FUSED_ATTENTION_OFF = os.environ.get("FLB200_FUSED_ATTENTION", "1") == "0"


def extension() -> B200AutogradExtension:
    """The process-wide extension instance (created lazily, once, like
    TensorBackend::getExtension, flashlight/fl/tensor/TensorBackend.h:283-300)."""
    global _ext
    if _ext is None:
        _ext = B200AutogradExtension()
    return _ext


def set_math_mode(mode: int) -> None:
    extension().math_mode = mode


class Variable:
    def __init__(self, tensor: torch.Tensor, calc_grad: bool = False,
                 inputs: Sequence["Variable"] = (), grad_func: Optional[Callable] = None):
        self.tensor = tensor
        self.inputs: List[Variable] = list(inputs)
        self.grad_func = grad_func
        self.calc_grad = calc_grad or any(i.calc_grad for i in self.inputs)
        self._grad: Optional[torch.Tensor] = None
        self._grad_owned = False
        # A second gradient contribution is kept apart until somebody reads `grad`: a
        # grad_func that can take two addends (grad_func2) then sums them inside its own
        # kernel instead of paying a whole-tensor addition first.
        self._grad_second: Optional[torch.Tensor] = None
        self.grad_func2: Optional[Callable] = None
        self.grad_hook: Optional[Callable[["Variable"], None]] = None

    @property
    def grad(self) -> Optional[torch.Tensor]:
        if self._grad_second is not None:
            second, self._grad_second = self._grad_second, None
            if self._grad_owned:
                F.add(self._grad, second, out=self._grad)
            else:  # the first gradient may be shared with another Variable: never write into it
                self._grad, self._grad_owned = F.add(self._grad, second), True
        return self._grad

    @grad.setter
    def grad(self, value: Optional[torch.Tensor]) -> None:
        self._grad, self._grad_second, self._grad_owned = value, None, False

    # Variable::isCalcGrad / addGrad (Variable.cpp:185-211)
    def isCalcGrad(self) -> bool:
        return self.calc_grad

    def addGrad(self, g: torch.Tensor) -> None:
        if not self.calc_grad:
            return
        if g.shape != self.tensor.shape:
            raise ValueError(f"addGrad: given gradient has dimensions not equal to this Variable's "
                             f"dimensions: {tuple(g.shape)} vs {tuple(self.tensor.shape)}")
        if self._grad is None:
            self._grad, self._grad_owned = g, False
        elif self._grad_second is None and self.grad_func2 is not None:
            self._grad_second = g
        else:
            total = self.grad  # folds a pending second contribution in
            if self._grad_owned:
                F.add(total, g, out=total)
            else:
                self._grad, self._grad_owned = F.add(total, g), True

    def zeroGrad(self) -> None:
        self.grad = None

    def registerGradHook(self, hook: Callable[["Variable"], None]) -> None:
        self.grad_hook = hook

    # Variable::backward / build (Variable.cpp:248-294): iterative topological sort
    def backward(self, grad: Optional[torch.Tensor] = None, retain_graph: bool = False) -> None:
        if grad is None:
            grad = torch.ones_like(self.tensor)
        self.addGrad(grad)
        order: List[Variable] = []
        seen = set()
        stack = [(self, False)]
        while stack:
            node, done = stack.pop()
            if done:
                order.append(node)
                continue
            if id(node) in seen or not node.calc_grad:
                continue
            seen.add(id(node))
            stack.append((node, True))
            for inp in node.inputs:
                if id(inp) not in seen:
                    stack.append((inp, False))
        for node in reversed(order):
            if node.grad_func2 is not None and node._grad_second is not None:
                first, second = node._grad, node._grad_second
                node._grad_second = None
                node.grad_func2(node.inputs, first, second)
            elif node.grad_func is not None and node.grad is not None:
                node.grad_func(node.inputs, node.grad)
            if node.grad_hook is not None and node.grad is not None:
                node.grad_hook(node)
            if not retain_graph and node.grad_func is not None:
                node.grad_func = None
                node.grad_func2 = None
                node.inputs = []
                node.grad = None


# ------------------------------------------------------------------ functions
def conv2d(x: Variable, w: Variable, b: Optional[Variable], sx=1, sy=1, px=0, py=0, dx=1, dy=1,
           groups=1, channels_last_out: Optional[bool] = None, stats: bool = False) -> Variable:
    """fl::conv2d (Functions.cpp:1327-1452).  channels_last_out=True: the output is stored
    channels-last although the input is in fl's order (a network's first convolution).
    stats=True (a convolution that feeds a training-mode batch-norm over its channels, the
    pairing of flashlight/pkg/vision/models/Resnet.cpp:67-121): where the library can, the
    per-channel sums of the output are taken in the convolution's epilogue and travel with the
    result (`conv_stats`); batchnorm() / batchnorm_add_relu() then skip their statistics pass."""
    ext = extension()
    args = (sx, sy, px, py, dx, dy, groups)
    payload = AutogradPayload()
    bt = b.tensor if b is not None else None
    sums: Optional[list] = [] if (stats and CONV_STATS_ON) else None
    y = ext.conv2d(x.tensor, w.tensor, bt, *args, payload, channels_last_out=channels_last_out,
                   stats_out=sums)
    xt, wt = x.tensor, w.tensor

    def grad_func(inputs, gy):
        if inputs[0].isCalcGrad():
            inputs[0].addGrad(ext.conv2dBackwardData(gy, xt, wt, *args, None, payload))
        need_b = b is not None and inputs[2].isCalcGrad()
        if inputs[1].isCalcGrad() or need_b:
            gw, gb = ext.conv2dBackwardFilterBias(gy, xt, wt, bt if need_b else None, *args, None,
                                                  None, payload)
            if inputs[1].isCalcGrad():
                inputs[1].addGrad(gw)
            if need_b:
                inputs[2].addGrad(gb.reshape(bt.shape))

    out = Variable(y, False, [x, w] + ([b] if b is not None else []), grad_func)
    if sums:
        out.conv_stats = sums[0]
    return out


def _conv_stats(x: Variable, axes: Sequence[int], train: bool):
    """What a producing convolution attached to x, if it is the statistics this batch-norm
    needs (training mode, per channel of an image batch)."""
    st = getattr(x, "conv_stats", None)
    if st is None or not train or list(axes) != [2] or x.tensor.dim() != 4:
        return None
    return st


def pool2d(x: Variable, wx, wy, sx, sy, px, py, mode=L.POOL_MAX) -> Variable:
    """fl::pool2d (Functions.cpp:1459-1496)."""
    ext = extension()
    payload = AutogradPayload()
    y = ext.pool2d(x.tensor, wx, wy, sx, sy, px, py, mode, payload)
    xt = x.tensor

    def grad_func(inputs, gy):
        inputs[0].addGrad(ext.pool2dBackward(gy, xt, y, wx, wy, sx, sy, px, py, mode, payload))

    return Variable(y, False, [x], grad_func)


def batchnorm(x: Variable, weight: Optional[Variable], bias: Optional[Variable],
              running_mean: Optional[torch.Tensor], running_var: Optional[torch.Tensor],
              axes: Sequence[int], train: bool, momentum: float, epsilon: float,
              relu: bool = False) -> Variable:
    """fl::batchnorm (Functions.cpp:1498-1565).  relu=True is relu(batchnorm(x)) as one
    operator: no separate relu pass forward or backward, nothing extra saved."""
    ext = extension()
    wt = weight.tensor if weight is not None else None
    bt = bias.tensor if bias is not None else None
    y, save_mean, save_var = ext.batchnorm(x.tensor, wt, bt, running_mean, running_var, axes, train,
                                           momentum, epsilon, None, relu=relu,
                                           conv_stats=_conv_stats(x, axes, train))
    xt = x.tensor
    ins = [x] + ([weight] if weight is not None else []) + ([bias] if bias is not None else [])

    def grad_func(inputs, gy):
        if relu:
            gx, gw, gb = ext.batchnormReluBackward(gy, save_mean, save_var, xt, wt, bt, axes, train,
                                                   epsilon, None)
        else:
            gx, gw, gb = ext.batchnormBackward(gy, save_mean, save_var, xt, wt, axes, train,
                                               epsilon, None)
        inputs[0].addGrad(gx)
        k = 1
        if weight is not None:
            inputs[k].addGrad(gw.reshape(wt.shape)); k += 1
        if bias is not None:
            inputs[k].addGrad(gb.reshape(bt.shape))

    return Variable(y, False, ins, grad_func)


def batchnorm_add_relu(x: Variable, addend: Variable, weight: Optional[Variable],
                       bias: Optional[Variable], running_mean, running_var, axes: Sequence[int],
                       train: bool, momentum: float, epsilon: float) -> Variable:
    """relu(batchnorm(x) + addend): the tail of a residual block.  Forward is the statistics
    pass plus ONE apply pass that also reads the shortcut and writes the relu mask; backward is
    the masked (two-consumer-summing) relu gradient, which is the addend's gradient, followed by
    the batchnorm gradient.  Shapes the fused kernel does not take run the operators one by one."""
    ext = extension()
    if not ext.batchnormAddReluSupported(x.tensor, addend.tensor, axes):
        return add_relu(batchnorm(x, weight, bias, running_mean, running_var, axes, train, momentum,
                                  epsilon), addend)
    wt = weight.tensor if weight is not None else None
    bt = bias.tensor if bias is not None else None
    xt = x.tensor
    y, mask, save_mean, save_var = ext.batchnormAddRelu(
        xt, addend.tensor, wt, bt, running_mean, running_var, axes, train, momentum, epsilon,
        conv_stats=_conv_stats(x, axes, train))
    ins = [x, addend] + ([weight] if weight is not None else []) + ([bias] if bias is not None else [])

    def grad_func2(inputs, ga, gb):
        # the first batch-norm pass forms mask ? ga + gb : 0, writes it and reduces it
        gz, gx, gw, gbias = ext.batchnormAddReluBackward(
            mask, _aligned(ga), _aligned(gb) if gb is not None else None, save_mean, save_var, xt,
            wt, axes, train, epsilon, None)
        inputs[1].addGrad(gz)
        inputs[0].addGrad(gx)
        k = 2
        if weight is not None:
            inputs[k].addGrad(gw.reshape(wt.shape)); k += 1
        if bias is not None:
            inputs[k].addGrad(gbias.reshape(bt.shape))

    def grad_func(inputs, gy):
        grad_func2(inputs, gy, None)

    out = Variable(y, False, ins, grad_func)
    out.grad_func2 = grad_func2
    return out


def rnn(x: Variable, hx: Optional[Variable], cx: Optional[Variable], w: Variable, hidden: int,
        layers: int, mode: int, bidirectional: bool, dropout: float = 0.0):
    """fl::rnn (Functions.cpp:1606-1705): three outputs sharing one gradient computation."""
    ext = extension()
    payload = AutogradPayload()
    hxt = hx.tensor if hx is not None else None
    cxt = cx.tensor if cx is not None else None
    y, hy, cy = ext.rnn(x.tensor, hxt, cxt, w.tensor, hidden, layers, mode, bidirectional, dropout,
                        payload)
    grad_data = RNNGradData()
    xt, wt = x.tensor, w.tensor
    ins = [x, w] + ([hx] if hx is not None else []) + ([cx] if cx is not None else [])

    def dummy_grad(inputs, _g):
        dx, dhx, dcx, dw = ext.rnnBackward(xt, hxt, cxt, wt, grad_data, y, layers, hidden, mode,
                                           bidirectional, dropout, payload)
        inputs[0].addGrad(dx)
        inputs[1].addGrad(dw.reshape(wt.shape))
        k = 2
        if hx is not None:
            inputs[k].addGrad(dhx); k += 1
        if cx is not None and dcx is not None:
            inputs[k].addGrad(dcx)

    dummy = Variable(torch.empty(0, device=xt.device), False, ins, dummy_grad)

    def stash(name):
        def f(inputs, g):
            setattr(grad_data, name, g)
            if inputs[0].grad is None:
                inputs[0].grad = g.new_empty(0)  # marks the shared node as reached
        return f

    out_y = Variable(y, False, [dummy], stash("dy"))
    out_h = Variable(hy, False, [dummy], stash("dhy"))
    out_c = Variable(cy, False, [dummy], stash("dcy")) if cy is not None else None
    return out_y, out_h, out_c


def cast(x: Variable, dtype) -> Variable:
    """Variable::astype (flashlight/fl/autograd/Variable.cpp:160-175): the gradient is cast back
    to the input's type, which is how fp32 master weights receive the gradients of their bf16
    copies.  The conversions run on the library's kernel (flb200_astype) for f32 <-> f16 / bf16
    and fall back to torch for other types."""
    src = x.tensor.dtype
    if src == dtype:
        return x

    def to(t, d):
        out = F.astype(t, d) if t.is_cuda else None
        return out if out is not None else t.to(d)

    return glue(x, lambda t: to(t, dtype), lambda g: to(g, src))


def _linear_bf16(x: Variable, w: Variable, b: Optional[Variable], gelu: bool = False) -> Variable:
    """fl::linear on bf16 tensors: the three contractions go to flb200_matmul as strided views
    (bf16 operands, fp32 accumulation); bias (fp32) and an optional gelu in the forward
    contraction's epilogue where the library fuses them, else through the channel kernels."""
    xt, wt = x.tensor.contiguous(), w.tensor.contiguous()
    I, O = wt.shape
    rows = xt.numel() // I
    fused = None
    if (b is not None or gelu) and LINEAR_FUSED_ON:
        fused = F.linear_bias_act(xt, wt, b.tensor if b is not None else None, gelu)
    if fused is not None:
        y, pre = fused
    else:
        y = F.matmul(xt, wt, m=rows, n=O, k=I, a_strides=(I, 1), b_strides=(O, 1))
        y = y.reshape(tuple(xt.shape[:-1]) + (O,))
        if b is not None:
            F.channel_bias_add(y, b.tensor, rows, O, 1, out=y)
        pre = y
        if gelu:
            y = F.gelu(pre)

    def grad_func(inputs, gy):
        gy = gy.contiguous()
        if gelu:
            gy = F.gelu_backward(pre, gy)
        if inputs[0].isCalcGrad():   # dX (rows, I) = dY (rows, O) @ W^T (O, I)
            gx = F.matmul(gy, wt, m=rows, n=I, k=O, a_strides=(O, 1), b_strides=(1, O))
            inputs[0].addGrad(gx.reshape(xt.shape))
        if inputs[1].isCalcGrad():   # dW (I, O) = X^T (I, rows) @ dY (rows, O)
            inputs[1].addGrad(F.matmul(xt, gy, m=I, n=O, k=rows, a_strides=(1, I),
                                       b_strides=(O, 1)))
        if b is not None and inputs[2].isCalcGrad():
            inputs[2].addGrad(F.channel_sum(gy, rows, O, 1).reshape(b.tensor.shape))

    return Variable(y, False, [x, w] + ([b] if b is not None else []), grad_func)


def linear(x: Variable, w: Variable, b: Optional[Variable], gelu: bool = False) -> Variable:
    """fl::linear (Functions.cpp:1255-1309).  gelu=True: gelu(linear(x)) as one operator (the
    Linear + bias + GELU of a Transformer feed-forward block): bias and activation are applied
    where the contraction stores its result, and the pre-activation is kept for the gradient."""
    if x.tensor.dtype == torch.bfloat16:
        return _linear_bf16(x, w, b, gelu)
    mode = extension().math_mode
    bt = b.tensor if b is not None else None
    xt, wt = x.tensor, w.tensor
    fused = None
    if (b is not None or gelu) and LINEAR_FUSED_ON and xt.dtype == torch.float32:
        fused = F.linear_bias_act(xt, wt, bt, gelu, math_mode=mode)
    if fused is not None:
        y, pre = fused
    else:
        pre = F.linear(xt, wt, bt, math_mode=mode)
        y = F.gelu(pre) if gelu else pre

    def grad_func(inputs, gy):
        if gelu:
            gy = F.gelu_backward(pre, gy)
        need_b = b is not None and inputs[2].isCalcGrad()
        gx, gw, gb = F.linear_backward(xt, wt, gy, need_b, inputs[0].isCalcGrad(),
                                       inputs[1].isCalcGrad(), math_mode=mode)
        if gx is not None:
            inputs[0].addGrad(gx)
        if gw is not None:
            inputs[1].addGrad(gw)
        if need_b:
            inputs[2].addGrad(gb.reshape(bt.shape))

    return Variable(y, False, [x, w] + ([b] if b is not None else []), grad_func)


def _unary(x: Variable, fwd, bwd, save_output: bool) -> Variable:
    y = fwd(x.tensor)
    saved = y if save_output else x.tensor

    def grad_func(inputs, gy):
        inputs[0].addGrad(bwd(saved, gy))

    return Variable(y, False, [x], grad_func)


def relu(x: Variable) -> Variable:
    """fl::relu.  For contiguous f32 tensors the forward kernel also writes the predicate x > 0
    as a bit mask and the gradient reads dy and the mask (a third less traffic than reading
    dy and y); otherwise the output is the saved tensor ((x > 0) equals (y > 0))."""
    t = x.tensor
    if t.dtype == torch.float32 and is_dense(t) and t.data_ptr() % 16 == 0:
        y, mask = F.relu_with_mask(t)

        def grad_func(inputs, gy):
            inputs[0].addGrad(F.relu_backward_mask(mask, _aligned(gy)))

        def grad_func2(inputs, ga, gb):
            inputs[0].addGrad(F.relu_backward_mask_sum(mask, _aligned(ga), _aligned(gb)))

        out = Variable(y, False, [x], grad_func)
        out.grad_func2 = grad_func2
        return out
    return _unary(x, F.relu, F.relu_backward, True)


def _aligned(g: torch.Tensor) -> torch.Tensor:
    return g if is_dense(g) and g.data_ptr() % 16 == 0 else g.contiguous().clone()


def add_relu(a: Variable, b: Variable) -> Variable:
    """relu(a + b), the residual join of a ResNet block (Resnet.cpp:67-121), as one kernel
    forward (sum, relu and the predicate bit mask) and one backward: both addends receive
    mask ? dy : 0, and when the output fed two consumers their two gradients are summed inside
    that kernel.  Falls back to add + relu for tensors the fused kernels do not take."""
    ta, tb = a.tensor, b.tensor
    if not (ta.dtype == torch.float32 and same_layout(ta, tb) and is_dense(ta) and
            is_dense(tb) and ta.data_ptr() % 16 == 0 and tb.data_ptr() % 16 == 0):
        return relu(add(a, b))
    y, mask = F.add_relu_with_mask(ta, tb)

    def grad_func(inputs, gy):
        gx = F.relu_backward_mask(mask, _aligned(gy))
        inputs[0].addGrad(gx)
        inputs[1].addGrad(gx)

    def grad_func2(inputs, ga, gb):
        gx = F.relu_backward_mask_sum(mask, _aligned(ga), _aligned(gb))
        inputs[0].addGrad(gx)
        inputs[1].addGrad(gx)

    out = Variable(y, False, [a, b], grad_func)
    out.grad_func2 = grad_func2
    return out


def gelu(x: Variable) -> Variable:
    return _unary(x, F.gelu, F.gelu_backward, False)


def tanh(x: Variable) -> Variable:
    return _unary(x, F.tanh, F.tanh_backward, True)


def dropout(x: Variable, p: float, mask: torch.Tensor) -> Variable:
    """fl::dropout with the Bernoulli mask supplied as data (Functions.cpp:1777-1785)."""
    y = F.dropout_apply(x.tensor, mask, p)

    def grad_func(inputs, gy):
        inputs[0].addGrad(F.dropout_apply(gy, mask, p))

    return Variable(y, False, [x], grad_func)


def add(a: Variable, b: Variable) -> Variable:
    """operator+ (Functions.cpp:114-123): both inputs receive the same gradient tensor."""
    y = F.add(a.tensor, b.tensor)

    def grad_func(inputs, gy):
        inputs[0].addGrad(gy)
        inputs[1].addGrad(gy)

    return Variable(y, False, [a, b], grad_func)


def view(x: Variable, shape) -> Variable:
    """moddims (Functions.cpp:969-1019): same bytes, new extents (torch order)."""
    old = x.tensor.shape

    def grad_func(inputs, gy):
        inputs[0].addGrad(gy.reshape(old))

    return Variable(x.tensor.reshape(shape), False, [x], grad_func)


def log_softmax(x: Variable) -> Variable:
    return _unary(x, F.log_softmax, F.log_softmax_backward, True)


def categorical_cross_entropy(logp: Variable, targets: torch.Tensor, reduction=L.REDUCE_MEAN,
                              ignore_index=-1, validate=False) -> Variable:
    """fl::categoricalCrossEntropy (Functions.cpp:1078-1154)."""
    loss, state = F.categorical_cross_entropy(logp.tensor, targets, reduction, ignore_index)
    if validate:
        F.check_targets(state)
    like, classes = logp.tensor, logp.tensor.shape[-1]

    def grad_func(inputs, gl):
        inputs[0].addGrad(F.categorical_cross_entropy_backward(gl, state, classes, like))

    return Variable(loss, False, [logp], grad_func)


def log_softmax_cross_entropy(x: Variable, targets: torch.Tensor, reduction=L.REDUCE_MEAN,
                              ignore_index=-1) -> Variable:
    """categoricalCrossEntropy(logSoftmax(x)) with the fused gradient kernel."""
    y = F.log_softmax(x.tensor)
    loss, state = F.categorical_cross_entropy(y, targets, reduction, ignore_index)

    def grad_func(inputs, gl):
        inputs[0].addGrad(F.log_softmax_cross_entropy_backward(y, gl, state))

    return Variable(loss, False, [x], grad_func)


# ------------------------------------------------ pieces of the Transformer workload
def glue(x: Variable, fwd, bwd) -> Variable:
    """A data-movement step that has no kernel in this library (permutations between the
    [rows, features] and [batch*heads, T, head] views, exp, the causal mask).  `fwd` maps the
    tensor, `bwd` maps the output gradient back; both are torch calls and are named as glue
    wherever a workload uses them."""
    y = fwd(x.tensor)

    def grad_func(inputs, gy):
        inputs[0].addGrad(bwd(gy))

    return Variable(y, False, [x], grad_func)


def unbind(x: Variable, fwd, bwd, n: int) -> List[Variable]:
    """One copy that brings `x` into n stacked parts (`fwd` maps its tensor to [n, ...]) and
    hands each part out as a Variable of its own — the q, k, v of a packed projection.  The
    reference indexes the packed tensor three times, and each index gradient is a zero tensor
    of the full size with one slice filled, summed by addGrad
    (flashlight/fl/autograd/Functions.cpp:1233-1263 `index`); here the parts' gradients are
    written into one buffer and `bwd` maps it back once, when the last of them has arrived.
    Every part must take part in the loss (a part without a gradient would leave the buffer
    waiting).  Data movement only: torch glue."""
    stacked = fwd(x.tensor)
    state = {"buf": None, "seen": 0}

    def part_grad(i):
        def grad_func(inputs, gy):
            if state["buf"] is None:
                state["buf"] = torch.empty_like(stacked)
            state["buf"][i].copy_(gy)
            state["seen"] += 1
            if state["seen"] == n:
                full, state["buf"], state["seen"] = state["buf"], None, 0
                inputs[0].addGrad(bwd(full))
        return grad_func

    return [Variable(stacked[i], False, [x], part_grad(i)) for i in range(n)]


def bmm(a: Variable, b: Variable, trans_b: bool = False) -> Variable:
    """Batched matmul (Functions.cpp:827-946): a (Z, M, K); b (Z, K, N), or (Z, N, K) when
    trans_b.  The three contractions of forward and backward are strided views of the same
    buffers handed to flb200_matmul — no transposed copies."""
    mode = extension().math_mode
    at, bt = a.tensor.contiguous(), b.tensor.contiguous()
    Z, M, K = at.shape
    N = bt.shape[1] if trans_b else bt.shape[2]
    bs = (1, K) if trans_b else (N, 1)           # strides of B viewed as (K, N)
    b_elems = bt.shape[1] * bt.shape[2]
    y = F.matmul(at, bt, m=M, n=N, k=K, a_strides=(K, 1), b_strides=bs, batch=Z,
                 batch_strides=(M * K, b_elems, 0), math_mode=mode)

    def grad_func(inputs, gy):
        gy = gy.contiguous()
        if inputs[0].isCalcGrad():
            # dA (M, K) = dY (M, N) @ B^T (N, K)
            bts = (K, 1) if trans_b else (1, N)  # strides of B viewed as (N, K)
            ga = F.matmul(gy, bt, m=M, n=K, k=N, a_strides=(N, 1), b_strides=bts, batch=Z,
                          batch_strides=(M * N, b_elems, 0), math_mode=mode)
            inputs[0].addGrad(ga)
        if inputs[1].isCalcGrad():
            if trans_b:
                # dB (N, K) = dY^T (N, M) @ A (M, K)
                gb = F.matmul(gy, at, m=N, n=K, k=M, a_strides=(1, N), b_strides=(K, 1), batch=Z,
                              batch_strides=(M * N, M * K, 0), math_mode=mode)
            else:
                # dB (K, N) = A^T (K, M) @ dY (M, N)
                gb = F.matmul(at, gy, m=K, n=N, k=M, a_strides=(1, K), b_strides=(N, 1), batch=Z,
                              batch_strides=(M * K, M * N, 0), math_mode=mode)
            inputs[1].addGrad(gb)

    return Variable(y, False, [a, b], grad_func)


def attention(q: Variable, k: Variable, v: Variable, scale: float, causal: bool) -> Variable:
    """softmax(scale * q k^T [+ causal mask]) v for (batch * heads, T, head dim) tensors — the
    chain matmulNT, softmax, matmul of flashlight/fl/autograd/Functions.cpp:1828-1891.  The
    forward pass runs that chain on the library's kernels but keeps only q, k, v, the output and
    the rows' log-sum-exp; the gradient is the fused kernel, which recomputes the probabilities
    block by block.  Shapes the fused kernel is not built for take the operator chain."""
    if not F.attention_backward_supported(q.tensor) or FUSED_ATTENTION_OFF:
        probs = softmax_rows(bmm(q, k, trans_b=True), scale, causal_period=q.tensor.shape[1] if causal else 0)
        return bmm(probs, v)
    mode = extension().math_mode
    qt, kt, vt = q.tensor.contiguous(), k.tensor.contiguous(), v.tensor.contiguous()
    Z, T, hd = qt.shape
    scores = F.matmul(qt, kt, m=T, n=T, k=hd, a_strides=(hd, 1), b_strides=(1, hd), batch=Z,
                      batch_strides=(T * hd, T * hd, 0), math_mode=mode)
    probs, lse = F.softmax_lse(scores, scale, T if causal else 0)
    del scores
    out = F.matmul(probs, vt, m=T, n=hd, k=T, a_strides=(T, 1), b_strides=(hd, 1), batch=Z,
                   batch_strides=(T * T, T * hd, 0), math_mode=mode)
    del probs

    def grad_func(inputs, gy):
        dq, dk, dv = F.attention_backward(qt, kt, vt, out, gy.contiguous(), lse, scale, causal)
        for inp, g in zip(inputs, (dq, dk, dv)):
            if inp.isCalcGrad():
                inp.addGrad(g)

    return Variable(out, False, [q, k, v], grad_func)


def softmax_rows(x: Variable, scale: float = 1.0, causal_period: int = 0) -> Variable:
    """softmax over the last dimension (Functions.cpp:1021-1042) of scale * x, with the causal
    mask of attention scores folded in when causal_period = T (x is a stack of T-row score
    matrices): one kernel forward, one backward (attention_softmax.cu)."""
    xt = x.tensor.contiguous()
    p = F.softmax(xt, scale, causal_period)

    def grad_func(inputs, gy):
        inputs[0].addGrad(F.softmax_backward(p, gy.contiguous(), scale))

    return Variable(p, False, [x], grad_func)


def affine_rows(x: Variable, w: Variable, b: Variable) -> Variable:
    """y = x * tile(w) + tile(b) over rows of features: the affine part of fl::LayerNorm
    (flashlight/fl/nn/modules/LayerNorm.cpp:99-128) as one kernel forward and two backward
    (parameter gradients from one pass over dy and x, then dx = dy * w).  w and b are the fp32
    parameters themselves, whatever the activations' dtype."""
    xt, wt, bt = x.tensor, w.tensor, b.tensor
    y = F.layernorm_affine(xt, wt, bt)

    def grad_func(inputs, gy):
        need_p = inputs[1].isCalcGrad() or inputs[2].isCalcGrad()
        gx, gw, gb = F.layernorm_affine_backward(gy, xt, wt, inputs[0].isCalcGrad(), need_p)
        if inputs[0].isCalcGrad():
            inputs[0].addGrad(gx.reshape(xt.shape))
        if inputs[1].isCalcGrad():
            inputs[1].addGrad(gw.reshape(wt.shape))
        if inputs[2].isCalcGrad():
            inputs[2].addGrad(gb.reshape(bt.shape))

    return Variable(y, False, [x, w, b], grad_func)


def layernorm(x: Variable, w: Variable, b: Variable, eps: float = 1e-5) -> Variable:
    """fl::LayerNorm over the last dimension (flashlight/fl/nn/modules/LayerNorm.cpp:66-128) as
    one operator: a single forward kernel (a warp per row) that keeps x_hat and the rows' inverse
    standard deviation, and a gradient of two kernels.  w and b are the fp32 parameters whatever
    the activations' dtype.  Rows of more than 2048 features take the operator chain."""
    xt, wt, bt = x.tensor, w.tensor, b.tensor
    if xt.shape[-1] > 2048 or LAYERNORM_FUSED_OFF:
        return None
    y, xhat, invstd = F.layernorm(xt, wt, bt, eps)

    def grad_func(inputs, gy):
        need_p = inputs[1].isCalcGrad() or inputs[2].isCalcGrad()
        gx, gw, gb = F.layernorm_backward(gy, xhat, wt, invstd, inputs[0].isCalcGrad(), need_p)
        if inputs[0].isCalcGrad():
            inputs[0].addGrad(gx.reshape(xt.shape))
        if inputs[1].isCalcGrad():
            inputs[1].addGrad(gw.reshape(wt.shape))
        if inputs[2].isCalcGrad():
            inputs[2].addGrad(gb.reshape(bt.shape))

    return Variable(y.reshape(xt.shape), False, [x, w, b], grad_func)


def embedding(table: Variable, ids: torch.Tensor) -> Variable:
    """fl::embedding (Functions.cpp:1707-1749): rows of the table picked by token id; the
    gradient is a scatter-add into the table, done without atomics (embedding.cu).  The table
    gradient is always f32: when the table is a bf16 copy of fp32 master weights (autograd.cast)
    the master receives it without a round trip through bf16."""
    vocab = table.tensor.shape[0]
    y = F.embedding(table.tensor, ids)

    def grad_func(inputs, gy):
        inputs[0].addGrad(F.embedding_backward(gy, ids, vocab))

    return Variable(y, False, [table], grad_func)
