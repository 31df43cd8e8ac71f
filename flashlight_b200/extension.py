"""Host-side mirror of fl::AutogradExtension over the flb200 C ABI.

`B200AutogradExtension` has the nine operator methods of the reference
interface (flashlight/fl/autograd/tensor/AutogradExtension.h:46-180) with the
same names, argument order and argument meaning; the C++ class of the same
name (csrc/fl/B200AutogradExtension.cpp) is the one a Flashlight build links.
This Python class exists so that the parity tests and the benchmark drive the
very same C entry points from device buffers that torch owns.

Tensor convention: a torch CUDA tensor of shape (d_{k-1}, ..., d_0), contiguous,
stands for the fl tensor [d_0, ..., d_{k-1}] — fl is column-major, so the bytes
are identical.  An image batch fl [W,H,C,N] is torch (N,C,H,W); `axes` and every
other dimension index are fl indices (0 = fastest).  An absent (empty) fl tensor
is None.  Out-parameters of the reference (saveMean, saveVar) are returned.

Channels-last storage: an image batch may also be a torch tensor in
torch.channels_last memory format (same logical (N,C,H,W) indexing, bytes laid out
[N][H][W][C]).  conv2d, pool2d and batchnorm over the channel axis take such tensors
as they are (FLB200_LAYOUT_NHWC), return their results in the same format, and the
element-wise functions work on any two tensors of equal layout, so a network whose
first convolution is called with channels_last_out=True keeps every activation in
the layout the tensor-core convolutions read natively and no layout copy is made.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from . import _lib as L

_DTYPES = {torch.float32: L.F32, torch.float16: L.F16, torch.bfloat16: L.BF16}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"dtype {t.dtype} is not supported by the B200 autograd extension") from None


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("the B200 autograd extension needs device (CUDA) tensors")
    if not is_dense(t):
        # fl::DevicePtr also refuses non-contiguous tensors (flashlight/fl/common/DevicePtr.cpp:16-33)
        raise ValueError("can't get device pointer of non-contiguous tensor")
    return t.data_ptr()


def is_channels_last(t: Optional[torch.Tensor]) -> bool:
    """True for a 4-d tensor stored [N][H][W][C] whose bytes differ from the [N][C][H][W] order
    (with one channel or 1x1 planes the two orders coincide and the tensor counts as the latter)."""
    return (t is not None and t.dim() == 4 and not t.is_contiguous()
            and t.is_contiguous(memory_format=torch.channels_last))


def is_dense(t: torch.Tensor) -> bool:
    """Contiguous in fl's order or in channels-last order."""
    return t.is_contiguous() or is_channels_last(t)


def same_layout(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.shape == b.shape and is_channels_last(a) == is_channels_last(b)


def empty_images(shape, like: torch.Tensor, channels_last: bool) -> torch.Tensor:
    fmt = torch.channels_last if channels_last else torch.contiguous_format
    return torch.empty(shape, dtype=like.dtype, device=like.device, memory_format=fmt)


def stream_handle() -> int:
    return torch.cuda.current_stream().cuda_stream


_mask_offset = 0


def bernoulli_mask(shape, keep_prob: float, device, dtype=torch.float32, seed: Optional[int] = None,
                   offset: Optional[int] = None) -> torch.Tensor:
    """A 0 / 1 mask with P(1) = keep_prob from the library's counter-based generator
    (flb200_bernoulli_mask).  Without an explicit (seed, offset) the stream continues from the
    last call, seeded by torch's CUDA generator seed."""
    global _mask_offset
    out = torch.empty(shape, dtype=dtype, device=device)
    n = out.numel()
    if seed is None:
        seed = torch.cuda.initial_seed() & ((1 << 64) - 1)
    if offset is None:
        offset = _mask_offset
        _mask_offset += (n + 3) // 4
    code = {torch.float32: L.F32, torch.float16: L.F16, torch.bfloat16: L.BF16}[dtype]
    L.check(L.lib.flb200_bernoulli_mask(ptr(out), n, float(keep_prob), seed, offset, code,
                                        stream_handle()))
    return out


def workspace(nbytes: int, like: torch.Tensor) -> Optional[torch.Tensor]:
    if nbytes <= 0:
        return None
    return torch.empty(int(nbytes), dtype=torch.uint8, device=like.device)


class _ConvLayoutCache:
    """flb200_conv2d_cache plus the tensors behind it.  A copy is only trusted for the very
    tensor it was made from: same storage address and same version counter."""

    def __init__(self, x_bytes: int, gy_bytes: int, like: torch.Tensor):
        self.c = L.Conv2dCache()
        self.x_bytes, self.gy_bytes, self.device = int(x_bytes), int(gy_bytes), like.device
        self.x_buf = self.gy_buf = None
        self.x_key = self.gy_key = None

    @staticmethod
    def _key(t: torch.Tensor):
        return (t.data_ptr(), t._version, tuple(t.shape))

    def bind_x(self, x: torch.Tensor) -> None:
        if self.x_bytes and self.x_buf is None:
            self.x_buf = torch.empty(self.x_bytes, dtype=torch.uint8, device=self.device)
            self.c.x_cl, self.c.x_cl_bytes = self.x_buf.data_ptr(), self.x_bytes
        self.c.x_cl_valid = 0
        self.x_key = self._key(x)

    def check_x(self, x: torch.Tensor) -> None:
        if self.x_key != self._key(x):
            self.bind_x(x)

    def bind_gy(self, gy: torch.Tensor) -> None:
        if self.gy_bytes and self.gy_buf is None:
            self.gy_buf = torch.empty(self.gy_bytes, dtype=torch.uint8, device=self.device)
            self.c.gy_cl, self.c.gy_cl_bytes = self.gy_buf.data_ptr(), self.gy_bytes
        self.c.gy_cl_valid = 0
        self.gy_key = self._key(gy)

    def check_gy(self, gy: torch.Tensor) -> None:
        if self.gy_key != self._key(gy):
            self.c.gy_cl_valid = 0

    def release_gy(self) -> None:
        """The copy of grad_y is dead after backward-filter; give its memory back."""
        self.gy_buf = None
        self.gy_key = None
        self.c.gy_cl, self.c.gy_cl_bytes, self.c.gy_cl_valid = None, 0, 0

    def ref(self):
        return C.byref(self.c)


class AutogradPayload:
    """detail::AutogradPayload: a nullable slot that forward fills and backward reads."""

    def __init__(self):
        self.data = None


@dataclass
class RNNGradData:
    """detail::RNNGradData (flashlight/fl/autograd/tensor/AutogradOps.h:356-360)."""
    dy: Optional[torch.Tensor] = None
    dhy: Optional[torch.Tensor] = None
    dcy: Optional[torch.Tensor] = None


@dataclass
class _PoolPayload:
    argmax: torch.Tensor


@dataclass
class _RnnPayload:
    reserve: torch.Tensor
    dropout_mask: Optional[torch.Tensor] = None


def _shape4(t: torch.Tensor):
    """torch (.., N, C, H, W) with missing leading dims = 1 -> (W, H, C, N)."""
    if t.dim() > 4:
        raise ValueError("expected at most 4 dimensions")
    s = (1,) * (4 - t.dim()) + tuple(t.shape)
    return s[3], s[2], s[1], s[0]


def default_math_mode() -> int:
    """FLB200_TF32=1 selects the tensor-core (TF32) kernels, FLB200_TF32=0 strict fp32."""
    if os.environ.get("FLB200_MATH", "") in L.MATH_BY_NAME:  # strict | tf32 | f32x3
        return L.MATH_BY_NAME[os.environ["FLB200_MATH"]]
    return L.MATH_TF32 if os.environ.get("FLB200_TF32", "0") not in ("0", "", "false") else L.MATH_STRICT_F32


class DynamicBenchmark:
    """fl::DynamicBenchmark with DynamicBenchmarkOptions<KernelMode>
    (flashlight/fl/common/DynamicBenchmark.h:60-263): while the class-wide benchmark mode is on,
    audit() times the call under the current option (device synchronised on both sides, as
    fl::sync() does there); every option is timed `count` times, then the fastest is kept."""

    _benchmark_mode = False

    def __init__(self, options: Sequence[int], count: int = 10):
        if not options:
            raise ValueError("Options must be passed vector with at least one element")
        self.options, self.count = list(options), int(count)
        self.reset()

    def reset(self) -> None:
        self.times = [0.0] * len(self.options)
        self.counts = [0] * len(self.options)
        self._complete, self._idx = False, 0

    @classmethod
    def setBenchmarkMode(cls, mode: bool) -> None:
        cls._benchmark_mode = bool(mode)

    @classmethod
    def getBenchmarkMode(cls) -> bool:
        return cls._benchmark_mode

    def _update(self) -> None:
        if self._complete:
            return
        for i, c in enumerate(self.counts):
            if c < self.count:
                self._idx = i
                return
        self._complete = True
        self._idx = min(range(len(self.options)), key=lambda i: self.times[i])

    def currentOption(self) -> int:
        self._update()
        return self.options[self._idx]

    def timingsComplete(self) -> bool:
        self._update()
        return self._complete

    def audit(self, function, incrementCount: bool = True):
        if self.timingsComplete() or not self._benchmark_mode:
            return function()
        import time
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = function()
        torch.cuda.synchronize()
        self.times[self._idx] += time.perf_counter() - t0
        if incrementCount:
            self.counts[self._idx] += 1
        return out


class B200AutogradExtension:
    """sm_100a implementation of the Flashlight autograd extension interface."""

    def __init__(self, math_mode: Optional[int] = None, cache_layouts: Optional[bool] = None):
        self.math_mode = default_math_mode() if math_mode is None else math_mode
        # Keep the channels-last copies of x and grad_y in the payload of each conv2d call
        # site (forward -> backward-filter, backward-data -> backward-filter).  Costs one
        # extra copy of x per convolution that uses one; FLB200_CACHE_LAYOUTS=0 turns it off.
        if cache_layouts is None:
            cache_layouts = os.environ.get("FLB200_CACHE_LAYOUTS", "1") != "0"
        self.cache_layouts = cache_layouts

    # ------------------------------------------------------------ registry
    def isDataTypeSupported(self, dtype) -> bool:
        """TensorExtension::isDataTypeSupported (flashlight/fl/tensor/TensorExtension.h:34)."""
        return dtype in _DTYPES

    def createBenchmarkOptions(self) -> DynamicBenchmark:
        """Options of a Conv2D module's run-time autotune: fp32 FMA, TF32 ("allow conversion")
        and the three-pass split, tried in that order (the counterpart of
        backend/cudnn/CudnnAutogradExtension.cpp:16-25)."""
        return DynamicBenchmark([L.MATH_STRICT_F32, L.MATH_TF32, L.MATH_F32X3])

    def _audited(self, bench: Optional[DynamicBenchmark], run):
        """run(math_mode) under the benchmark's current option while tuning is on, else in the
        configured mode (backend/cudnn/Conv2D.cpp:401-405,466-535)."""
        if bench is None or not DynamicBenchmark.getBenchmarkMode():
            return run(self.math_mode)
        mode = bench.currentOption()
        return bench.audit(lambda: run(mode))

    # --------------------------------------------------------------- conv2d
    def _conv_desc(self, input, weights, sx, sy, px, py, dx, dy, groups,
                   output_channels_last: Optional[bool] = None) -> L.Conv2dDesc:
        """output_channels_last: layout of y / grad_y; None = that of the input."""
        if input.dtype not in _DTYPES or weights.dtype != input.dtype:
            raise ValueError("conv2d: input and weights must share one of f32 / f16 / bf16")
        x_cl = is_channels_last(input)
        y_cl = x_cl if output_channels_last is None else bool(output_channels_last)
        if x_cl and not y_cl:
            raise ValueError("conv2d: a channels-last input gives a channels-last output")
        layout = L.LAYOUT_NHWC if x_cl else (L.LAYOUT_NCHW_IN_NHWC_OUT if y_cl else L.LAYOUT_NCHW)
        W, H, Cin, N = _shape4(input)
        kW, kH, Cg, Cout = _shape4(weights)
        if Cg * groups != Cin:
            raise ValueError(
                f"conv2d: weight has {Cg} input channels per group x {groups} groups, input has {Cin}")
        return L.Conv2dDesc(W, H, Cin, N, kW, kH, Cout, sx, sy, px, py, dx, dy, groups,
                            dtype_code(input), self.math_mode, layout)

    def _conv_cache(self, d, payload, like) -> Optional["_ConvLayoutCache"]:
        """The layout cache kept in the payload of one conv2d call site (None when the route
        keeps no channels-last copies, when there is no payload, or when caching is off)."""
        if payload is None or not self.cache_layouts:
            return None
        if isinstance(payload.data, _ConvLayoutCache):
            return payload.data
        nx = L.lib.flb200_conv2d_cache_bytes(C.byref(d), 0)
        ng = L.lib.flb200_conv2d_cache_bytes(C.byref(d), 1)
        if nx == 0 and ng == 0:
            return None
        payload.data = _ConvLayoutCache(nx, ng, like)
        return payload.data

    def conv2d(self, input, weights, bias, sx, sy, px, py, dx, dy, groups, payload=None,
               channels_last_out: Optional[bool] = None, stats_out: Optional[list] = None):
        """channels_last_out=True on an input in fl's order: the output (and from there the whole
        network) is stored channels-last; a channels-last input always gives such an output.
        stats_out: a list that receives (matrix, groups) — the batch-norm statistics of the result,
        taken in the convolution's epilogue (flb200_conv2d_forward_stats), for
        batchnorm(..., conv_stats=...) — where the library can do that; it stays empty otherwise."""
        d = self._conv_desc(input, weights, sx, sy, px, py, dx, dy, groups, channels_last_out)
        wo, ho = L.i32(), L.i32()
        L.check(L.lib.flb200_conv2d_output_dims(C.byref(d), C.byref(wo), C.byref(ho)))
        out = empty_images((d.N, d.Cout, ho.value, wo.value), input, d.layout != L.LAYOUT_NCHW)
        if bias is not None and bias.numel() != d.Cout:
            raise ValueError("conv2d: bias must have one element per output channel")
        nbytes = L.lib.flb200_conv2d_workspace_bytes(C.byref(d), 0)
        ws = workspace(nbytes, input)
        cache = self._conv_cache(d, payload, input)
        if cache is not None:
            cache.bind_x(input)
        if stats_out is not None:
            groups = L.i64()
            sbytes = L.lib.flb200_conv2d_stats_bytes(C.byref(d), C.byref(groups))
            if sbytes and all(t is None or t.data_ptr() % 16 == 0
                              for t in (input, weights, bias, out, ws)):
                stats = torch.empty(sbytes // 4, dtype=torch.float32, device=input.device)
                L.check(L.lib.flb200_conv2d_forward_stats(
                    C.byref(d), ptr(input), ptr(weights), ptr(bias), ptr(out), ptr(stats), sbytes,
                    ptr(ws), nbytes, cache.ref() if cache is not None else None, stream_handle()))
                stats_out.append((stats, groups.value))
                return out
        L.check(L.lib.flb200_conv2d_forward_cached(
            C.byref(d), ptr(input), ptr(weights), ptr(bias), ptr(out), ptr(ws), nbytes,
            cache.ref() if cache is not None else None, stream_handle()))
        return out

    def conv2dBackwardData(self, gradOutput, input, weight, sx, sy, px, py, dx, dy, groups,
                           dataGradBenchmark=None, payload=None):
        grad_in = torch.empty_like(input)

        def run(mode):
            d = self._conv_desc(input, weight, sx, sy, px, py, dx, dy, groups,
                                is_channels_last(gradOutput) or is_channels_last(input))
            d.math_mode = mode
            nbytes = L.lib.flb200_conv2d_workspace_bytes(C.byref(d), 1)
            ws = workspace(nbytes, input)
            cache = self._conv_cache(d, payload, input)
            if cache is not None:
                cache.bind_gy(gradOutput)
            L.check(L.lib.flb200_conv2d_backward_data_cached(
                C.byref(d), ptr(gradOutput), ptr(weight), ptr(grad_in), ptr(ws), nbytes,
                cache.ref() if cache is not None else None, stream_handle()))

        self._audited(dataGradBenchmark, run)
        return grad_in

    def conv2dBackwardFilterBias(self, gradOutput, input, weights, bias, sx, sy, px, py, dx, dy,
                                 groups, filterBench=None, biasBench=None, autogradPayload=None):
        grad_w = torch.empty_like(weights)
        grad_b = torch.empty_like(bias) if bias is not None else None

        def run(mode):
            d = self._conv_desc(input, weights, sx, sy, px, py, dx, dy, groups,
                                is_channels_last(gradOutput) or is_channels_last(input))
            d.math_mode = mode
            nbytes = L.lib.flb200_conv2d_workspace_bytes(C.byref(d), 2)
            ws = workspace(nbytes, input)
            cache = self._conv_cache(d, autogradPayload, input)
            if cache is not None:
                cache.check_x(input)
                cache.check_gy(gradOutput)
            L.check(L.lib.flb200_conv2d_backward_filter_bias_cached(
                C.byref(d), ptr(gradOutput), ptr(input), ptr(grad_w), ptr(grad_b), ptr(ws), nbytes,
                cache.ref() if cache is not None else None, stream_handle()))
            if cache is not None:
                cache.release_gy()

        self._audited(filterBench, run)   # the bias gradient is a reduction: nothing to choose
        return grad_w, grad_b

    # --------------------------------------------------------------- pool2d
    @staticmethod
    def _pool_desc(input, wx, wy, sx, sy, px, py, mode) -> L.Pool2dDesc:
        W, H, Cc, N = _shape4(input)
        return L.Pool2dDesc(W, H, Cc, N, wx, wy, sx, sy, px, py, int(mode), dtype_code(input),
                            L.LAYOUT_NHWC if is_channels_last(input) else L.LAYOUT_NCHW)

    def pool2d(self, input, wx, wy, sx, sy, px, py, mode, payload=None):
        d = self._pool_desc(input, wx, wy, sx, sy, px, py, mode)
        wo, ho = L.i32(), L.i32()
        L.check(L.lib.flb200_pool2d_output_dims(C.byref(d), C.byref(wo), C.byref(ho)))
        out = empty_images((d.N, d.C, ho.value, wo.value), input, d.layout == L.LAYOUT_NHWC)
        argmax = None
        if payload is not None and int(mode) == L.POOL_MAX:
            argmax = torch.empty_like(out, dtype=torch.uint8)
            payload.data = _PoolPayload(argmax)
        L.check(L.lib.flb200_pool2d_forward(C.byref(d), ptr(input), ptr(out), ptr(argmax),
                                            stream_handle()))
        return out

    def pool2dBackward(self, gradOutput, input, poolOutput, wx, wy, sx, sy, px, py, mode,
                       payload=None):
        d = self._pool_desc(input, wx, wy, sx, sy, px, py, mode)
        argmax = payload.data.argmax if payload is not None and payload.data is not None else None
        grad_in = torch.empty_like(input)
        L.check(L.lib.flb200_pool2d_backward(C.byref(d), ptr(gradOutput), ptr(input), ptr(argmax),
                                             ptr(grad_in), stream_handle()))
        return grad_in

    # ------------------------------------------------------------ batchnorm
    @staticmethod
    def _bn_desc(input, axes: Sequence[int]) -> L.BatchnormDesc:
        if is_channels_last(input):
            # stored [N][H][W][C]: statistics per channel are column sums of a [pixels][C] matrix
            if list(axes) != [2]:
                raise ValueError("batchnorm: a channels-last tensor is normalised over fl axis 2 only")
            n, c, h, w = input.shape
            return L.BatchnormDesc(n * h * w, c, 1, dtype_code(input))
        fl_shape = tuple(reversed(input.shape))
        shape = (L.i64 * len(fl_shape))(*fl_shape)
        ax = (L.i32 * len(axes))(*axes)
        d = L.BatchnormDesc()
        L.check(L.lib.flb200_batchnorm_geometry(shape, len(fl_shape), ax, len(axes), C.byref(d)))
        d.dtype = dtype_code(input)
        return d

    def batchnorm(self, input, weight, bias, runningMean, runningVar, axes, train, momentum,
                  epsilon, payload=None, relu=False, conv_stats=None):
        """Returns (output, saveMean, saveVar).  saveVar holds 1/sqrt(var + eps).
        runningMean / runningVar are updated in place when given.  relu=True returns
        relu(batchnorm(x)) from the same two passes (pair it with batchnormReluBackward)."""
        d = self._bn_desc(input, axes)
        for t in (weight, bias, runningMean, runningVar):
            if t is not None and t.dtype != torch.float32:
                raise ValueError("fl::batchnorm: non-input tensors must be of type f32")
        if weight is not None and weight.numel() != d.channels:
            raise ValueError("[BatchNorm] Invalid shape for weight.")
        if bias is not None and bias.numel() != d.channels:
            raise ValueError("[BatchNorm] Invalid shape for bias.")
        out = torch.empty_like(input)
        save_mean = save_var = None
        if train:
            save_mean = torch.empty(d.channels, dtype=torch.float32, device=input.device)
            save_var = torch.empty(d.channels, dtype=torch.float32, device=input.device)
        nbytes = L.lib.flb200_batchnorm_workspace_bytes(C.byref(d))
        ws = workspace(nbytes, input)
        if conv_stats is not None and train:
            # statistics from what the producing convolution took: no pass over x for them
            stats, groups = conv_stats
            nbytes = L.lib.flb200_batchnorm_from_stats_workspace_bytes(C.byref(d), groups)
            ws = workspace(nbytes, input)
            L.check(L.lib.flb200_batchnorm_forward_from_stats(
                C.byref(d), ptr(input), None, 1 if relu else 0, ptr(stats), groups, ptr(weight),
                ptr(bias), ptr(runningMean), ptr(runningVar), ptr(save_mean), ptr(save_var),
                float(momentum), float(epsilon), ptr(out), None, ptr(ws), nbytes, stream_handle()))
            return out, save_mean, save_var
        forward = L.lib.flb200_batchnorm_relu_forward if relu else L.lib.flb200_batchnorm_forward
        L.check(forward(
            C.byref(d), ptr(input), ptr(weight), ptr(bias), ptr(runningMean), ptr(runningVar),
            ptr(save_mean), ptr(save_var), 1 if train else 0, float(momentum), float(epsilon),
            ptr(out), ptr(ws), nbytes, stream_handle()))
        return out, save_mean, save_var

    def batchnormBackward(self, gradOutput, saveMean, saveVar, input, weight, axes, train, epsilon,
                          payload=None):
        if not train:
            # cudnn/BatchNorm.cpp:196-199
            raise RuntimeError("can't compute batchnorm grad when train was not specified")
        d = self._bn_desc(input, axes)
        grad_in = torch.empty_like(input)
        grad_w = torch.empty(d.channels, dtype=torch.float32, device=input.device)
        grad_b = torch.empty(d.channels, dtype=torch.float32, device=input.device)
        nbytes = L.lib.flb200_batchnorm_workspace_bytes(C.byref(d))
        ws = workspace(nbytes, input)
        L.check(L.lib.flb200_batchnorm_backward(
            C.byref(d), ptr(gradOutput), ptr(input), ptr(weight), ptr(saveMean), ptr(saveVar),
            ptr(grad_in), ptr(grad_w), ptr(grad_b), ptr(ws), nbytes, stream_handle()))
        return grad_in, grad_w, grad_b

    def batchnormAddReluSupported(self, input, addend, axes) -> bool:
        d = self._bn_desc(input, axes)
        shape_ok = d.inner > 1 or (is_channels_last(input) and d.channels % 8 == 0)
        return (input.dtype == torch.float32 and shape_ok and same_layout(input, addend)
                and addend.dtype == input.dtype and is_dense(input)
                and input.data_ptr() % 16 == 0 and addend.data_ptr() % 16 == 0)

    def batchnormAddRelu(self, input, addend, weight, bias, runningMean, runningVar, axes, train,
                         momentum, epsilon, payload=None, conv_stats=None):
        """relu(batchnorm(input) + addend) with the predicate's bit mask: returns
        (output, mask, saveMean, saveVar).  Check batchnormAddReluSupported first."""
        d = self._bn_desc(input, axes)
        out = torch.empty_like(input)
        # elements per mask byte: 8 consecutive channels of a pixel for channels-last tensors
        group = 8 if d.inner % 8 == 0 or d.inner == 1 else (4 if d.inner % 4 == 0 else 1)
        mask = torch.empty((input.numel() + group - 1) // group, dtype=torch.uint8,
                           device=input.device)
        save_mean = save_var = None
        if train:
            save_mean = torch.empty(d.channels, dtype=torch.float32, device=input.device)
            save_var = torch.empty(d.channels, dtype=torch.float32, device=input.device)
        nbytes = L.lib.flb200_batchnorm_workspace_bytes(C.byref(d))
        ws = workspace(nbytes, input)
        if conv_stats is not None and train:
            stats, groups = conv_stats
            nbytes = L.lib.flb200_batchnorm_from_stats_workspace_bytes(C.byref(d), groups)
            ws = workspace(nbytes, input)
            L.check(L.lib.flb200_batchnorm_forward_from_stats(
                C.byref(d), ptr(input), ptr(addend), 1, ptr(stats), groups, ptr(weight), ptr(bias),
                ptr(runningMean), ptr(runningVar), ptr(save_mean), ptr(save_var), float(momentum),
                float(epsilon), ptr(out), ptr(mask), ptr(ws), nbytes, stream_handle()))
            return out, mask, save_mean, save_var
        L.check(L.lib.flb200_batchnorm_add_relu_forward(
            C.byref(d), ptr(input), ptr(addend), ptr(weight), ptr(bias), ptr(runningMean),
            ptr(runningVar), ptr(save_mean), ptr(save_var), 1 if train else 0, float(momentum),
            float(epsilon), ptr(out), ptr(mask), ptr(ws), nbytes, stream_handle()))
        return out, mask, save_mean, save_var

    def batchnormAddReluBackward(self, mask, gradA, gradB, saveMean, saveVar, input, weight, axes,
                                 train, epsilon, payload=None):
        """Gradient of batchnormAddRelu: returns (gradSum, gradInput, gradWeight, gradBias) where
        gradSum = mask ? gradA + gradB : 0 is the addend's gradient (gradB may be None)."""
        if not train:
            raise RuntimeError("can't compute batchnorm grad when train was not specified")
        d = self._bn_desc(input, axes)
        grad_sum = torch.empty_like(input)
        grad_in = torch.empty_like(input)
        grad_w = torch.empty(d.channels, dtype=torch.float32, device=input.device)
        grad_b = torch.empty(d.channels, dtype=torch.float32, device=input.device)
        nbytes = L.lib.flb200_batchnorm_workspace_bytes(C.byref(d))
        ws = workspace(nbytes, input)
        L.check(L.lib.flb200_batchnorm_add_relu_backward(
            C.byref(d), ptr(mask), ptr(gradA), ptr(gradB), ptr(input), ptr(weight), ptr(saveMean),
            ptr(saveVar), ptr(grad_sum), ptr(grad_in), ptr(grad_w), ptr(grad_b), ptr(ws), nbytes,
            stream_handle()))
        return grad_sum, grad_in, grad_w, grad_b

    def batchnormReluBackward(self, gradOutput, saveMean, saveVar, input, weight, bias, axes, train,
                              epsilon, payload=None):
        """Gradient of relu(batchnorm(x)) given the gradient of the relu output: the predicate
        is rebuilt from the input, so no output tensor or mask is needed."""
        if not train:
            raise RuntimeError("can't compute batchnorm grad when train was not specified")
        d = self._bn_desc(input, axes)
        grad_in = torch.empty_like(input)
        grad_w = torch.empty(d.channels, dtype=torch.float32, device=input.device)
        grad_b = torch.empty(d.channels, dtype=torch.float32, device=input.device)
        nbytes = L.lib.flb200_batchnorm_workspace_bytes(C.byref(d))
        ws = workspace(nbytes, input)
        L.check(L.lib.flb200_batchnorm_relu_backward(
            C.byref(d), ptr(gradOutput), ptr(input), ptr(weight), ptr(bias), ptr(saveMean),
            ptr(saveVar), ptr(grad_in), ptr(grad_w), ptr(grad_b), ptr(ws), nbytes, stream_handle()))
        return grad_in, grad_w, grad_b

    # ------------------------------------------------------------------ rnn
    def _rnn_desc(self, input, hiddenSize, numLayers, mode, bidirectional) -> L.RnnDesc:
        if input.dtype != torch.float32:
            raise ValueError("rnn: only f32 tensors are supported")
        if input.dim() != 3:
            raise ValueError("rnn: input must be [inputSize, batch, seqLen]")
        T, B, I = input.shape
        return L.RnnDesc(I, hiddenSize, numLayers, B, T, int(mode), 1 if bidirectional else 0, L.F32,
                         self.math_mode)

    def rnn(self, input, hiddenState, cellState, weights, hiddenSize, numLayers, mode,
            bidirectional, dropout, payload=None, dropout_mask=None):
        """Returns (y, hy, cy); cy is None unless mode is LSTM.  dropout > 0 applies inter-layer
        dropout (backend/cudnn/RNN.cpp:83-85): the mask [numLayers - 1, T, B, H * dirs] of 0 / 1
        is drawn here (`bernoulli_mask`, a counter-based generator seeded from torch's) unless the
        caller supplies one, and is kept in the payload for the backward pass."""
        if not 0.0 <= dropout < 1.0:
            raise ValueError("rnn: dropout must be in [0, 1)")
        d = self._rnn_desc(input, hiddenSize, numLayers, mode, bidirectional)
        nparams = L.lib.flb200_rnn_num_params(C.byref(d))
        if weights.numel() != nparams:
            raise ValueError(f"rnn: weights has {weights.numel()} elements, expected {nparams}")
        dirs = 2 if bidirectional else 1
        T, B, _ = input.shape
        dev = input.device
        use_dropout = (dropout > 0.0 or dropout_mask is not None) and numLayers > 1
        mask = None
        if use_dropout:
            shape = (numLayers - 1, T, B, hiddenSize * dirs)
            if dropout_mask is not None:
                mask = dropout_mask
                if tuple(mask.shape) != shape or mask.dtype != torch.float32 or not mask.is_contiguous():
                    raise ValueError(f"rnn: dropout mask must be a dense float32 tensor {shape}")
            else:
                mask = bernoulli_mask(shape, 1.0 - dropout, dev)
        y = torch.empty((T, B, hiddenSize * dirs), dtype=torch.float32, device=dev)
        hy = torch.empty((numLayers * dirs, B, hiddenSize), dtype=torch.float32, device=dev)
        cy = torch.empty_like(hy) if int(mode) == L.RNN_LSTM else None
        reserve = None
        rbytes = 0
        if payload is not None:
            rbytes = (L.lib.flb200_rnn_reserve_bytes_dropout(C.byref(d)) if use_dropout
                      else L.lib.flb200_rnn_reserve_bytes(C.byref(d)))
            reserve = workspace(rbytes, input)
            payload.data = _RnnPayload(reserve)
            payload.data.dropout_mask = mask
        wbytes = L.lib.flb200_rnn_workspace_bytes(C.byref(d), 0 if reserve is not None else 2)
        if reserve is None and use_dropout:
            wbytes += L.lib.flb200_rnn_reserve_bytes_dropout(C.byref(d))
        ws = workspace(wbytes, input)
        if use_dropout:
            L.check(L.lib.flb200_rnn_forward_dropout(
                C.byref(d), ptr(input), ptr(hiddenState), ptr(cellState), ptr(weights), ptr(mask),
                float(dropout), ptr(y), ptr(hy), ptr(cy), ptr(reserve), rbytes, ptr(ws), wbytes,
                stream_handle()))
        else:
            L.check(L.lib.flb200_rnn_forward(
                C.byref(d), ptr(input), ptr(hiddenState), ptr(cellState), ptr(weights), ptr(y),
                ptr(hy), ptr(cy), ptr(reserve), rbytes, ptr(ws), wbytes, stream_handle()))
        return y, hy, cy

    def rnnBackward(self, input, hiddenState, cellState, weights, gradData: RNNGradData, output,
                    numLayers, hiddenSize, mode, bidirectional, dropProb, payload=None):
        """Returns (dx, dhx, dcx, dw)."""
        if payload is None or payload.data is None:
            raise ValueError("B200AutogradExtension::rnnBackward given null detail::AutogradPayload")
        d = self._rnn_desc(input, hiddenSize, numLayers, mode, bidirectional)
        reserve = payload.data.reserve
        mask = getattr(payload.data, "dropout_mask", None)
        dx = torch.empty_like(input)
        dirs = 2 if bidirectional else 1
        B = input.shape[1]
        dhx = torch.empty((numLayers * dirs, B, hiddenSize), dtype=torch.float32, device=input.device)
        dcx = torch.empty_like(dhx) if int(mode) == L.RNN_LSTM else None
        dw = torch.empty_like(weights)
        wbytes = L.lib.flb200_rnn_workspace_bytes(C.byref(d), 1)
        ws = workspace(wbytes, input)
        if mask is not None:
            L.check(L.lib.flb200_rnn_backward_dropout(
                C.byref(d), ptr(input), ptr(hiddenState), ptr(cellState), ptr(weights), ptr(mask),
                float(dropProb), ptr(output), ptr(gradData.dy), ptr(gradData.dhy),
                ptr(gradData.dcy), ptr(dx), ptr(dhx), ptr(dcx), ptr(dw), ptr(reserve),
                reserve.numel(), ptr(ws), wbytes, stream_handle()))
            return dx, dhx, dcx, dw
        L.check(L.lib.flb200_rnn_backward(
            C.byref(d), ptr(input), ptr(hiddenState), ptr(cellState), ptr(weights), ptr(output),
            ptr(gradData.dy), ptr(gradData.dhy), ptr(gradData.dcy), ptr(dx), ptr(dhx), ptr(dcx),
            ptr(dw), ptr(reserve), reserve.numel(), ptr(ws), wbytes, stream_handle()))
        return dx, dhx, dcx, dw
