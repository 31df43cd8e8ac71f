"""Per-operator roofline bench: times ONE operator of the backward hot path on a
ResNet-50-shaped (or named) input with CUDA events and prints one JSON line with the
achieved GB/s or TFLOP/s and the fraction of the measured peak.

    python -m flashlight_b200.opbench --op batchnormBackward --shape 64,64,112,112
    python -m flashlight_b200.opbench --op conv2dBackwardData --conv 256,64,56,56,64,3,1,1 --math tf32
    python -m flashlight_b200.opbench --suite resnet50 --batch 64

--shape is torch order (N,C,H,W); --conv is N,Cin,H,W,Cout,k,stride,pad.  Inputs are
larger than L2 for the default shapes, so no flush is needed between iterations.
Algorithmic bytes / flops follow the operator's interface tensors (fp32): relu / add /
batchnorm backward 12 B per element, batchnorm forward 8, pooling 4*(N_in+N_out) forward and
4*(2*N_in+N_out) backward, bias gradient 4 per dy element, convolutions 2*M*N*K flops.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from . import _lib as L
from . import functions as F
from .extension import AutogradPayload, B200AutogradExtension

ROOT = Path(__file__).resolve().parent.parent
CHANNELS_LAST = False  # --channels-last: image tensors stored [N][H][W][C]


def images(t):
    return t.contiguous(memory_format=torch.channels_last) if CHANNELS_LAST and t.dim() == 4 else t


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def time_op(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def report(op, desc, ms, nbytes=None, flops=None, math="strict", extra=None):
    hbm, bf16, src = peaks()
    line = {"op": op, "case": desc, "ms": ms, "math": math}
    if CHANNELS_LAST:
        line["layout"] = "channels_last"
    if flops:
        tf = flops / (ms * 1e-3) / 1e12
        peak = bf16 / 2  # tf32 tensor rate = half the bf16 rate
        line.update(bound="tensor", achieved=tf, unit="TFLOP/s", peak=peak, frac=tf / peak,
                    peak_source=f"{src} bf16 burst / 2")
    else:
        gbs = nbytes / (ms * 1e-3) / 1e9
        line.update(bound="hbm", achieved=gbs, unit="GB/s", peak=hbm, frac=gbs / hbm, peak_source=src)
    if extra:
        line.update(extra)
    print(json.dumps(line), flush=True)
    return line


def bench_eltwise(op, shape, iters):
    x = torch.randn(shape, device="cuda")
    g = torch.randn(shape, device="cuda")
    n = x.numel()
    if op == "relu":
        return report(op, list(shape), time_op(lambda: F.relu(x), iters), nbytes=8 * n)
    if op == "relu_backward":
        return report(op, list(shape), time_op(lambda: F.relu_backward(x, g), iters), nbytes=12 * n)
    if op == "add":
        return report(op, list(shape), time_op(lambda: F.add(x, g), iters), nbytes=12 * n)
    if op == "gelu_backward":
        return report(op, list(shape), time_op(lambda: F.gelu_backward(x, g), iters), nbytes=12 * n)
    raise SystemExit(f"unknown eltwise op {op}")


def bench_bn(op, shape, iters, axes=(2,)):
    ext = B200AutogradExtension(L.MATH_STRICT_F32)
    x = images(torch.randn(shape, device="cuda"))
    g = images(torch.randn(shape, device="cuda"))
    ch = shape[1]
    w = torch.rand(ch, device="cuda")
    b = torch.zeros(ch, device="cuda")
    rm, rv = torch.zeros(ch, device="cuda"), torch.ones(ch, device="cuda")
    n = x.numel()
    if op == "batchnorm":
        ms = time_op(lambda: ext.batchnorm(x, w, b, rm, rv, list(axes), True, 0.1, 1e-5), iters)
        return report(op, list(shape), ms, nbytes=8 * n)
    if op == "batchnormRelu":  # relu(batchnorm(x)): same bytes as batchnorm
        ms = time_op(lambda: ext.batchnorm(x, w, b, rm, rv, list(axes), True, 0.1, 1e-5, relu=True),
                     iters)
        return report(op, list(shape), ms, nbytes=8 * n)
    if op == "batchnormAddRelu":  # relu(batchnorm(x) + shortcut): reads x twice + shortcut, writes y
        ms = time_op(lambda: ext.batchnormAddRelu(x, g, w, b, rm, rv, list(axes), True, 0.1, 1e-5),
                     iters)
        return report(op, list(shape), ms, nbytes=12 * n)
    if op == "batchnormAddReluBackward":
        # two incoming gradients and the mask in; the join's gradient and dx out (20 B/elem of
        # interface traffic; the passes move 28)
        _, mask, sm, sv = ext.batchnormAddRelu(x, g, w, b, rm, rv, list(axes), True, 0.1, 1e-5)
        g2 = images(torch.randn(shape, device="cuda"))
        ms = time_op(lambda: ext.batchnormAddReluBackward(mask, g, g2, sm, sv, x, w, list(axes), True,
                                                          1e-5), iters)
        return report(op, list(shape), ms, nbytes=20 * n)
    _, sm, sv = ext.batchnorm(x, w, b, rm, rv, list(axes), True, 0.1, 1e-5)
    if op == "batchnormReluBackward":
        ms = time_op(lambda: ext.batchnormReluBackward(g, sm, sv, x, w, b, list(axes), True, 1e-5),
                     iters)
        return report(op, list(shape), ms, nbytes=12 * n)
    ms = time_op(lambda: ext.batchnormBackward(g, sm, sv, x, w, list(axes), True, 1e-5), iters)
    return report(op, list(shape), ms, nbytes=12 * n)


def bench_pool(op, shape, iters, geo=(3, 3, 2, 2, 1, 1), mode=L.POOL_MAX):
    ext = B200AutogradExtension(L.MATH_STRICT_F32)
    x = images(torch.randn(shape, device="cuda"))
    payload = AutogradPayload()
    y = ext.pool2d(x, *geo, mode, payload)
    g = torch.randn_like(y)
    if op == "pool2d":
        ms = time_op(lambda: ext.pool2d(x, *geo, mode, payload), iters)
        return report(op, list(shape), ms, nbytes=4 * (x.numel() + y.numel()))
    ms = time_op(lambda: ext.pool2dBackward(g, x, y, *geo, mode, payload), iters)
    return report(op, list(shape), ms, nbytes=4 * (2 * x.numel() + y.numel()))


def bench_bias_grad(shape, iters):
    g = torch.randn(shape, device="cuda")
    N, Cc, H, W = shape
    ms = time_op(lambda: F.channel_sum(g, N, Cc, H * W), iters)
    return report("conv2dBackwardBias", list(shape), ms, nbytes=4 * g.numel())


def bench_conv(op, conv, iters, math):
    N, Cin, H, W, Cout, k, s, p = conv
    mode = L.MATH_BY_NAME.get(math, L.MATH_TF32)
    ext = B200AutogradExtension(mode)
    x = torch.randn(N, Cin, H, W, device="cuda")
    first = CHANNELS_LAST and Cin <= 4  # a network's first layer: x in fl's order, y channels-last
    if not first:
        x = images(x)
    w = torch.randn(Cout, Cin, k, k, device="cuda") * (1.0 / (Cin * k * k) ** 0.5)
    args = (s, s, p, p, 1, 1, 1)
    y = ext.conv2d(x, w, None, *args, None, True if first else None)
    g = torch.randn_like(y)
    flops = 2.0 * y.numel() * Cin * k * k
    if op == "conv2d":
        fn = lambda: ext.conv2d(x, w, None, *args, None, True if first else None)
    elif op == "conv2dBackwardData":
        fn = lambda: ext.conv2dBackwardData(g, x, w, *args)
    else:
        fn = lambda: ext.conv2dBackwardFilterBias(g, x, w, None, *args)
    ms = time_op(fn, iters)
    nbytes = 4 * (x.numel() + y.numel() + w.numel())
    return report(op, list(conv), ms, flops=flops, math=math,
                  extra={"hbm_floor_ms": nbytes / (peaks()[0] * 1e9) * 1e3})


def measure_cublas_tf32(n=8192, burst_iters=20, sustained_s=3.0):
    """The denominator that TF32-mode fractions can be read against: cuBLAS (through
    torch.matmul, TF32 allowed) on n^3, as a short burst and as a seconds-long loop under
    the power cap.  Library code measuring the peak; never on an operator's path."""
    import time
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(n, n, device="cuda")
        b = torch.randn(n, n, device="cuda")
        for _ in range(5):
            a @ b
        burst_ms = time_op(lambda: a @ b, burst_iters)
        torch.cuda.synchronize()
        t0 = time.time()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        iters = 0
        e0.record()
        while time.time() - t0 < sustained_s:
            for _ in range(20):
                a @ b
            iters += 20
            torch.cuda.synchronize()
        e1.record()
        torch.cuda.synchronize()
        sustained_ms = e0.elapsed_time(e1) / iters
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    flops = 2.0 * n ** 3
    print(json.dumps({"op": "cublas_tf32_peak", "n": n,
                      "burst_tflops": flops / (burst_ms * 1e-3) / 1e12,
                      "sustained_tflops": flops / (sustained_ms * 1e-3) / 1e12}), flush=True)


# distinct ResNet-50 convolution shapes: Cin, H(=W), Cout, k, stride, pad
RESNET50_CONVS = [
    (3, 224, 64, 7, 2, 3), (64, 56, 64, 1, 1, 0), (64, 56, 64, 3, 1, 1), (64, 56, 256, 1, 1, 0),
    (256, 56, 64, 1, 1, 0), (256, 56, 128, 1, 1, 0), (128, 56, 128, 3, 2, 1),
    (128, 28, 512, 1, 1, 0), (256, 56, 512, 1, 2, 0), (512, 28, 128, 1, 1, 0),
    (128, 28, 128, 3, 1, 1), (512, 28, 256, 1, 1, 0), (256, 28, 256, 3, 2, 1),
    (256, 14, 1024, 1, 1, 0), (512, 28, 1024, 1, 2, 0), (1024, 14, 256, 1, 1, 0),
    (256, 14, 256, 3, 1, 1), (1024, 14, 512, 1, 1, 0), (512, 14, 512, 3, 2, 1),
    (512, 7, 2048, 1, 1, 0), (1024, 14, 2048, 1, 2, 0), (2048, 7, 512, 1, 1, 0),
    (512, 7, 512, 3, 1, 1),
]


# how often each shape above occurs in ResNet-50 (bottleneck blocks 3-4-6-3)
RESNET50_COUNTS = [1, 1, 3, 4, 2, 1, 1, 4, 1, 3, 3, 1, 1, 6, 1, 5, 5, 1, 1, 3, 1, 2, 2]


def suite_resnet50_step_convs(batch, math):
    """Every convolution call of one ResNet-50 training step, once, in the call pattern of
    the autograd tape (forward, backward-data, backward-filter sharing one payload) and with
    nothing else on the device: the command to put under a profiler when the per-step DRAM
    traffic of the convolution kernels is wanted at the full batch size."""
    mode = L.MATH_BY_NAME.get(math, L.MATH_TF32)
    ext = B200AutogradExtension(mode)
    flops = 0.0
    algo_bytes = 0
    for (ci, hw, co, k, s, p), count in zip(RESNET50_CONVS, RESNET50_COUNTS):
        x = torch.randn(batch, ci, hw, hw, device="cuda")
        first = CHANNELS_LAST and ci <= 4  # the network's first layer: x in fl's order
        if not first:
            x = images(x)
        w = torch.randn(co, ci, k, k, device="cuda") * (1.0 / (ci * k * k) ** 0.5)
        args = (s, s, p, p, 1, 1, 1)
        for _ in range(count):
            payload = AutogradPayload()
            y = ext.conv2d(x, w, None, *args, payload, True if first else None)
            g = torch.ones_like(y)
            n_pass = 2
            if ci != 3:
                ext.conv2dBackwardData(g, x, w, *args, None, payload)
                n_pass = 3
            ext.conv2dBackwardFilterBias(g, x, w, None, *args, None, None, payload)
            flops += n_pass * 2.0 * y.numel() * ci * k * k
            # interface tensors of the three calls: each reads two of {x, w, y} and writes one
            algo_bytes += n_pass * 4 * (x.numel() + y.numel() + w.numel())
            del y, g, payload
        torch.cuda.synchronize()
    print(json.dumps({"suite": "resnet50_step_convs", "batch": batch, "math": math,
                      "layout": "channels_last" if CHANNELS_LAST else "fl",
                      "conv_calls": int(sum(RESNET50_COUNTS) * 3 - 1), "flops": flops,
                      "algorithmic_bytes": algo_bytes}), flush=True)


def suite_resnet50(batch, iters, math):
    for (ci, hw, co, k, s, p) in RESNET50_CONVS:
        conv = (batch, ci, hw, hw, co, k, s, p)
        bench_conv("conv2d", conv, iters, math)
        if ci != 3:
            bench_conv("conv2dBackwardData", conv, iters, math)
        bench_conv("conv2dBackwardFilterBias", conv, iters, math)
    for shape in [(batch, 64, 112, 112), (batch, 256, 56, 56), (batch, 512, 28, 28),
                  (batch, 1024, 14, 14), (batch, 2048, 7, 7)]:
        bench_bn("batchnorm", shape, iters)
        bench_bn("batchnormBackward", shape, iters)
        bench_eltwise("relu_backward", shape, iters)
        bench_eltwise("add", shape, iters)
    bench_pool("pool2d", (batch, 64, 112, 112), iters)
    bench_pool("pool2dBackward", (batch, 64, 112, 112), iters)
    bench_bias_grad((batch, 64, 112, 112), iters)


def suite_workloads(iters, math, which):
    """Forward + backward step time of the other synthetic workloads at their full sizes
    (the ResNet-50 step is bench.py's job): MNIST convnet batch 64, conv-ASR 12 x 1024
    channels T=1000 batch 16, 3-layer bidirectional LSTM H=1024 T=500 batch 32."""
    from . import autograd as A
    from . import workloads
    A.set_math_mode(L.MATH_BY_NAME.get(math, L.MATH_TF32))
    g = torch.Generator().manual_seed(1234)

    def run(name, model, x, t, units, unit):
        x, t = x.cuda(), t.cuda()

        def step():
            model.zeroGrad()
            loss = model.loss(x, t)
            loss.backward()
            return loss

        ms = time_op(step, iters, warmup=2)
        print(json.dumps({"workload": name, "math": math, "ms_per_step": ms,
                          "value": units / (ms * 1e-3), "unit": unit,
                          "loss": float(step().tensor.cpu())}), flush=True)

    if which in ("all", "mnist"):
        run("mnist_convnet_b64", workloads.mnist_convnet(),
            torch.randn(64, 1, 28, 28, generator=g),
            torch.randint(0, 10, (64,), generator=g, dtype=torch.int32), 64, "images/s")
    if which in ("all", "asr"):
        B, T = 16, 1000
        run("conv_asr_b16_t1000", workloads.ConvAsr(),
            torch.randn(B, 80, 1, T, generator=g),
            torch.randint(0, 30, (B * T,), generator=g, dtype=torch.int32), B * T, "frames/s")
    if which in ("all", "transformer"):
        B, T = 8, 512
        dt = torch.bfloat16 if math == "bf16" else torch.float32
        run("transformer_lm_12x768_t512_b8", workloads.TransformerLM(compute_dtype=dt),
            torch.randint(0, 32000, (B, T), generator=g),
            torch.randint(0, 32000, (B * T,), generator=g, dtype=torch.int32), B * T, "tokens/s")
    if which in ("all", "bilstm"):
        T, B = 500, 32
        run("bilstm_h1024_t500_b32", workloads.BiLstm(),
            torch.randn(T, B, 80, generator=g), torch.randn(T, B, 2048, generator=g), B,
            "sequences/s")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op")
    ap.add_argument("--suite")
    ap.add_argument("--shape", default="64,64,112,112")
    ap.add_argument("--conv", default="64,64,56,56,64,3,1,1")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--channels-last", action="store_true",
                    help="image tensors stored channels-last ([N][H][W][C])")
    ap.add_argument("--math", default="strict", choices=["strict", "tf32", "f32x3", "bf16"],
                    help="bf16 only applies to the transformer workload")
    a = ap.parse_args()
    global CHANNELS_LAST
    CHANNELS_LAST = a.channels_last
    if not torch.cuda.is_available():
        raise SystemExit("opbench needs a CUDA device")
    shape = tuple(int(v) for v in a.shape.split(","))
    conv = tuple(int(v) for v in a.conv.split(","))
    if a.op == "cublas_tf32_peak":
        return measure_cublas_tf32()
    if a.suite and a.suite.startswith("workloads"):
        which = a.suite.split(":")[1] if ":" in a.suite else "all"
        return suite_workloads(a.iters, a.math, which)
    if a.suite == "resnet50_step_convs":
        return suite_resnet50_step_convs(a.batch, a.math)
    if a.suite == "resnet50":
        return suite_resnet50(a.batch, a.iters, a.math)
    if a.op in ("relu", "relu_backward", "add", "gelu_backward"):
        return bench_eltwise(a.op, shape, a.iters)
    if a.op in ("batchnorm", "batchnormBackward", "batchnormRelu", "batchnormReluBackward",
                "batchnormAddRelu", "batchnormAddReluBackward"):
        return bench_bn(a.op, shape, a.iters)
    if a.op in ("pool2d", "pool2dBackward"):
        return bench_pool(a.op, shape, a.iters)
    if a.op == "conv2dBackwardBias":
        return bench_bias_grad(shape, a.iters)
    if a.op in ("conv2d", "conv2dBackwardData", "conv2dBackwardFilterBias"):
        return bench_conv(a.op, conv, a.iters, a.math)
    raise SystemExit(f"unknown op {a.op}")


if __name__ == "__main__":
    main()
