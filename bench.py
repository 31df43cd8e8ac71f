#!/usr/bin/env python
"""Benchmark of the autograd-backward hot path: ResNet-50 training step (forward +
backward, data-parallel gradient all-reduce at N > 1) on synthetic inputs.

    python bench.py --gpus N --steps K --warmup W            # this library, B200
    python bench.py --impl reference --steps K --warmup W     # CPU stand-in of the reference

One JSON line on stdout (rank 0).  `value` = images/s over all ranks with inputs
resident in HBM; `e2e` = the same step with the host->device copy of each batch from
pinned memory and the device->host read of the loss inside the timed region;
`roofline` = the operator with the largest share of device time, timed with CUDA events
around its launches inside the timed steps; `cpu_baseline` = the CPU stand-in
(torch-CPU, same operator sequence) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from collections import defaultdict
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "resnet50_fwd_bwd_images_per_sec"
UNIT = "images/s"
WORKLOAD = "resnet50_train_step_224x224x3_fp32"


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


def cpu_model() -> str:
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


# ------------------------------------------------------------------ CPU arm
def cpu_sample(batch: int, steps: int, warmup: int, budget_s: float, seed: int = 1234):
    """Times the CPU stand-in on `batch` images per step; stops early once budget_s is spent."""
    import torch

    from oracle import cpu_workloads

    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(seed)
    params = _resnet50_params_cpu(g)
    x = torch.randn(batch, 3, 224, 224, generator=g)
    t = torch.randint(0, 1000, (batch,), generator=g)
    for _ in range(warmup):
        cpu_workloads.resnet50_step(params, x, t)
    done, t0 = 0, time.perf_counter()
    while done < steps:
        cpu_workloads.resnet50_step(params, x, t)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return {"value": batch * done / dt, "unit": UNIT, "cores": torch.get_num_threads(),
            "cpu_model": cpu_model(), "kind": "port",
            "sample": f"{done} steps of {batch} images (torch-CPU oneDNN stand-in, fp32), "
                      f"{dt:.1f} s"}, dt / done * 1e3, done


def _resnet50_params_cpu(gen):
    """Same shapes and initialisers as flashlight_b200.workloads.resnet50, built on the CPU."""
    import math

    import torch

    ps = []

    def conv(i, o, k):
        bound = math.sqrt(3.0 / (k * k * i))
        ps.append((torch.rand(o, i, k, k, generator=gen) * 2 - 1) * bound)
        ps.append(torch.rand(o, generator=gen))
        ps.append(torch.zeros(o))

    conv(3, 64, 7)
    in_c = 64
    for i, nb in enumerate((3, 4, 6, 3)):
        planes = 64 * 2 ** i
        for j in range(nb):
            stride = (1 if i == 0 else 2) if j == 0 else 1
            conv(in_c, planes, 1)
            conv(planes, planes, 3)
            conv(planes, planes * 4, 1)
            if in_c != planes * 4 or stride > 1:
                conv(in_c, planes * 4, 1)
            in_c = planes * 4
    ps.append((torch.rand(in_c, 1000, generator=gen) * 2 - 1) * math.sqrt(3.0 / in_c))
    ps.append((torch.rand(1000, generator=gen) * 2 - 1) * math.sqrt(1.0 / in_c))
    return ps


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    batch = args.cpu_batch
    warmup = min(args.warmup, 3)  # a CPU step of the sample takes about a second
    base, ms, done = cpu_sample(batch, args.steps, warmup, budget_s=150.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT,
        "n_gpus": args.gpus, "steps": done, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch_per_step": batch,
                   "stand_in": True, "stand_in_backend": "torch-cpu (oneDNN + MKL)",
                   "reference_buildable": False, "sample_scaled_from_batch": 256,
                   "note": "the reference's oneDNN CPU backend cannot be built in this image; "
                           "this arm times the torch-CPU stand-in (same oneDNN generation) on a "
                           "bounded sample of the workload"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------- GPU arm
class ClockSampler:
    """nvidia-smi samples of this GPU's clocks while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i",
                 str(self.index), "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


class OpTimer:
    """CUDA-event brackets around every operator call of the extension / function layer."""

    def __init__(self, torch):
        self.torch = torch
        self.enabled = False
        self.records = []  # (name, start, end, flops, bytes)

    def wrap(self, name, fn, work):
        def timed(*a, **k):
            if not self.enabled:
                return fn(*a, **k)
            s = self.torch.cuda.Event(enable_timing=True)
            e = self.torch.cuda.Event(enable_timing=True)
            s.record()
            out = fn(*a, **k)
            e.record()
            fl, by = work(out, *a, **k)
            self.records.append((name, s, e, fl, by))
            return out
        return timed

    def summary(self):
        agg = defaultdict(lambda: [0, 0.0, 0.0, 0.0])
        for name, s, e, fl, by in self.records:
            a = agg[name]
            a[0] += 1
            a[1] += s.elapsed_time(e)
            a[2] += fl
            a[3] += by
        return {k: {"calls": v[0], "ms": v[1], "flops": v[2], "bytes": v[3]} for k, v in agg.items()}

    def floor_ms(self, names, tflops, gbs):
        """Sum over the calls of `names` of max(flops / tensor peak, interface bytes / HBM peak):
        the time the calls would take if each ran at whichever of the two roofs bounds it."""
        total = 0.0
        for name, _, _, fl, by in self.records:
            if name in names:
                total += max(fl / (tflops * 1e12), by / (gbs * 1e9)) * 1e3
        return total


def _numel_bytes(*ts):
    return float(sum(t.numel() * t.element_size() for t in ts if t is not None))


def install_timers(timer: OpTimer, ext, F):
    def conv_flops(y, w):
        # 2 * M * N * K of the implicit GEMM: outputs x (Cin/g * kH * kW)
        return 2.0 * y.numel() * w.shape[1] * w.shape[2] * w.shape[3]

    ext.conv2d = timer.wrap("conv2d", ext.conv2d,
                            lambda out, x, w, b, *a, **k: (conv_flops(out, w), _numel_bytes(x, w, out)))
    ext.conv2dBackwardData = timer.wrap(
        "conv2dBackwardData", ext.conv2dBackwardData,
        lambda out, gy, x, w, *a, **k: (conv_flops(gy, w), _numel_bytes(gy, w, out)))
    ext.conv2dBackwardFilterBias = timer.wrap(
        "conv2dBackwardFilterBias", ext.conv2dBackwardFilterBias,
        lambda out, gy, x, w, *a, **k: (conv_flops(gy, w), _numel_bytes(gy, x, w)))
    ext.batchnorm = timer.wrap("batchnorm", ext.batchnorm,
                               lambda out, x, *a, **k: (0.0, 2 * _numel_bytes(x)))
    ext.batchnormBackward = timer.wrap("batchnormBackward", ext.batchnormBackward,
                                       lambda out, gy, sm, sv, x, *a, **k: (0.0, 3 * _numel_bytes(x)))
    ext.batchnormAddRelu = timer.wrap("batchnorm_add_relu", ext.batchnormAddRelu,
                                      lambda out, x, *a, **k: (0.0, 3 * _numel_bytes(x)))
    ext.batchnormAddReluBackward = timer.wrap(
        "batchnorm_add_relu_backward", ext.batchnormAddReluBackward,
        lambda out, mask, ga, gb, sm, sv, x, *a, **k: (0.0, 5 * _numel_bytes(x)))
    ext.batchnormReluBackward = timer.wrap(
        "batchnormBackward", ext.batchnormReluBackward,
        lambda out, gy, sm, sv, x, *a, **k: (0.0, 3 * _numel_bytes(x)))
    ext.pool2d = timer.wrap("pool2d", ext.pool2d, lambda out, x, *a, **k: (0.0, _numel_bytes(x, out)))
    ext.pool2dBackward = timer.wrap("pool2dBackward", ext.pool2dBackward,
                                    lambda out, gy, x, *a, **k: (0.0, 2 * _numel_bytes(x) + _numel_bytes(gy)))
    F.relu = timer.wrap("relu", F.relu, lambda out, x: (0.0, 2 * _numel_bytes(x)))
    F.relu_backward = timer.wrap("relu_backward", F.relu_backward,
                                 lambda out, x, gy: (0.0, 3 * _numel_bytes(x)))
    # the bit-mask variants keep the operator's algorithmic byte counts (8 and 12 B/elem) so
    # that the reported GB/s stays comparable; they move 8.1 B/elem each
    F.relu_with_mask = timer.wrap("relu", F.relu_with_mask,
                                  lambda out, x: (0.0, 2 * _numel_bytes(x)))
    F.relu_backward_mask = timer.wrap("relu_backward", F.relu_backward_mask,
                                      lambda out, mask, gy: (0.0, 3 * _numel_bytes(gy)))
    F.add = timer.wrap("add", F.add, lambda out, a, b, **k: (0.0, 3 * _numel_bytes(a)))
    # fused residual join (add + relu) and its two-addend gradient: bytes actually moved
    F.add_relu_with_mask = timer.wrap("add_relu", F.add_relu_with_mask,
                                      lambda out, a, b: (0.0, 3 * _numel_bytes(a)))
    F.relu_backward_mask_sum = timer.wrap("relu_backward_sum", F.relu_backward_mask_sum,
                                          lambda out, mask, ga, gb: (0.0, 3 * _numel_bytes(ga)))
    F.linear = timer.wrap("linear", F.linear,
                          lambda out, x, w, b=None, **k: (2.0 * out.numel() * w.shape[0],
                                                          _numel_bytes(x, w, out)))
    F.linear_backward = timer.wrap(
        "linear_backward", F.linear_backward,
        lambda out, x, w, gy, *a, **k: (4.0 * gy.numel() * w.shape[0], _numel_bytes(x, w, gy) * 2))



# ------------------------------------------------- reported-only side legs (N = 1)
def vendor_library_leg(torch, batch, steps=5, warmup=3):
    """The same ResNet-50 step through the vendor libraries (torch-CUDA: cuDNN / cuBLAS with
    TF32 allowed, channels-last tensors, cudnn.benchmark on) on the same GPU, for orientation
    only: none of this library's code runs here and nothing of it feeds `value`."""
    from oracle import cpu_workloads
    prev = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32,
            torch.backends.cudnn.benchmark)
    torch.backends.cudnn.allow_tf32 = torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.benchmark = True
    try:
        g = torch.Generator().manual_seed(1234)
        params = [p.cuda() for p in _resnet50_params_cpu(g)]
        params = [p.contiguous(memory_format=torch.channels_last) if p.dim() == 4 else p
                  for p in params]
        x = torch.randn(batch, 3, 224, 224, generator=g).cuda().contiguous(
            memory_format=torch.channels_last)
        t = torch.randint(0, 1000, (batch,), generator=g).cuda()
        for _ in range(warmup):
            cpu_workloads.resnet50_step(params, x, t)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            cpu_workloads.resnet50_step(params, x, t)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        return {"what": "torch-CUDA (cuDNN, TF32 allowed, channels_last, cudnn.benchmark) "
                        "forward + backward of the same network, reported only",
                "ms_per_step": ms, "value": batch / ms * 1e3, "unit": UNIT,
                "torch": torch.__version__, "cudnn": torch.backends.cudnn.version()}
    except Exception as exc:  # the side leg must never take the bench line down
        return {"error": f"{type(exc).__name__}: {exc}"[:200]}
    finally:
        (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32,
         torch.backends.cudnn.benchmark) = prev
        torch.cuda.empty_cache()


def _timed_steps(torch, step, warmup, steps):
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _cpu_timed(fn, budget_s, max_steps=5):
    fn()  # warm-up
    done, t0 = 0, time.perf_counter()
    while done < max_steps:
        fn()
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    return (time.perf_counter() - t0) / done, done


def other_workloads_leg(torch, peaks, steps=5, warmup=3, cpu_budget_s=5.0):
    """The four other synthetic configurations at their full sizes (forward + backward step,
    3 warm-up + 5 timed steps each), each with the whole-step contraction rate against the
    tensor peak of its arithmetic mode and a bounded CPU stand-in sample (torch-CPU on a
    reduced slice of the same workload, scaled linearly and labelled so)."""
    from flashlight_b200 import _lib as L
    from flashlight_b200 import autograd as A
    from flashlight_b200 import workloads
    from oracle import cpu_workloads as CW

    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(1234)
    out = {}
    tf32_peak, bf16_peak = peaks["bf16_tflops_sustained"] / 2, peaks["bf16_tflops_sustained"]

    def run(name, model, x, t, units, unit, flops, peak, dtype, cpu_fn, cpu_units, cpu_note):
        xd, td = x.cuda(), t.cuda()

        def step():
            model.zeroGrad()
            loss = model.loss(xd, td)
            loss.backward()
            return loss

        try:
            ms_eager = _timed_steps(torch, step, warmup, steps)
            # the same step captured once as a CUDA graph and replayed (as the ResNet-50 line
            # does): no host work between the kernels
            ms, captured, capture_error = ms_eager, False, None
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    step()
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    step()
                ms = _timed_steps(torch, graph.replay, warmup, steps)
                captured = True
                del graph
            except Exception as exc:  # capture refused: the eager time stands, the reason is kept
                capture_error = f"{type(exc).__name__}: {exc}"[:300]
                torch.cuda.synchronize()
            achieved = flops / (ms * 1e-3) / 1e12
            entry = {"ms_per_step": ms, "ms_per_step_eager": ms_eager, "graph_captured": captured,
                     "graph_error": capture_error,
                     "value": units / (ms * 1e-3), "unit": unit, "dtype": dtype,
                     "steps": steps, "warmup": warmup, "loss": float(step().tensor.float().cpu()),
                     "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak,
                                  "unit": "TFLOP/s", "frac": achieved / peak,
                                  "kernel": "tcgen05 contraction kernels, whole step "
                                            "(2*M*N*K of every contraction / step time)",
                                  "peak_source": f"{peaks['source']} bf16 sustained" +
                                                 ("" if dtype == "bf16" else " / 2 (tf32 rate)")}}
        except Exception as exc:
            out[name] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
            return
        try:
            sec, done = _cpu_timed(cpu_fn, cpu_budget_s)
            entry["cpu_baseline"] = {"value": cpu_units / sec, "unit": unit,
                                     "cores": torch.get_num_threads(), "cpu_model": cpu_model(),
                                     "kind": "port", "sample": f"{done} steps, {cpu_note}"}
        except Exception as exc:
            entry["cpu_baseline"] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
        out[name] = entry
        del xd, td
        torch.cuda.empty_cache()

    def host(model):
        return [p.tensor.detach().float().cpu() for p in model.parameters()]

    # C1: README MNIST convnet, batch 64, fp32 operands on the tensor cores (TF32)
    A.set_math_mode(L.MATH_TF32)
    m = workloads.mnist_convnet(device_dropout=True)  # masks from the device generator
    x, t = torch.randn(64, 1, 28, 28, generator=g), torch.randint(0, 10, (64,), generator=g, dtype=torch.int32)
    mask = (torch.rand(64, 1024, generator=g) > 0.5).float()
    ps = host(m)
    run("mnist_convnet_b64", m, x, t, 64, "images/s", 3 * 1.78e9, tf32_peak, "tf32",
        lambda: CW.mnist_convnet_step(ps, x, t, mask), 64, "full size (batch 64), torch-CPU fp32")
    # C3: conv-ASR 12 x 1024 channels, T = 1000, batch 16
    m = workloads.ConvAsr()
    B, T = 16, 1000
    x = torch.randn(B, 80, 1, T, generator=g)
    t = torch.randint(0, 30, (B * T,), generator=g, dtype=torch.int32)
    ps = host(m)
    xs, ts = x[:1, :, :, :250].contiguous(), t[:250].contiguous()
    run("conv_asr_b16_t1000", m, x, t, B * T, "frames/s", 3 * 4833e9, tf32_peak, "tf32",
        lambda: CW.conv_asr_step(ps, xs, ts), 250,
        "1 sequence of 250 frames (1/64 of the step), torch-CPU fp32, frames/s of the sample")
    # C4: 3-layer bidirectional LSTM, H = 1024, T = 500, batch 32
    m = workloads.BiLstm()
    T, B = 500, 32
    x, tgt = torch.randn(T, B, 80, generator=g), torch.randn(T, B, 2048, generator=g)
    lstm = torch.nn.LSTM(80, 1024, 3, bidirectional=True)
    xs, tgs = x[:25], tgt[:25]

    def lstm_cpu():
        lstm.zero_grad()
        y, _ = lstm(xs)
        ((y - tgs) ** 2).mean().backward()

    run("bilstm_h1024_t500_b32", m, x, tgt, B, "sequences/s", 3 * 1900e9, tf32_peak, "tf32", lstm_cpu,
        32 * 25 / 500.0,
        "25 of 500 time steps at batch 32, torch.nn.LSTM on the CPU: a restatement, not the "
        "reference (its oneDNN backend has no rnnBackward), scaled to whole sequences")
    # C5: Transformer LM 12 x 768, T = 512, batch 8, bf16 compute with fp32 master weights
    m = workloads.TransformerLM(compute_dtype=torch.bfloat16)
    B, T = 8, 512
    ids = torch.randint(0, 32000, (B, T), generator=g)
    t = torch.randint(0, 32000, (B * T,), generator=g, dtype=torch.int32)
    ps = host(m)
    ids1, t1 = ids[:1].contiguous(), t[:T].contiguous()
    run("transformer_lm_12x768_t512_b8_bf16", m, ids, t, B * T, "tokens/s", 3 * 974e9, bf16_peak,
        "bf16", lambda: CW.transformer_lm_step(ps, ids1, t1, heads=12, layers=12), T,
        "1 of 8 sequences (512 tokens), torch-CPU fp32, tokens/s of the sample")
    return out


TENSOR_OPS = {"conv2d", "conv2dBackwardData", "conv2dBackwardFilterBias", "linear", "linear_backward"}
CONV_OPS = ("conv2d", "conv2dBackwardData", "conv2dBackwardFilterBias")
CONV_KERNEL = "tc_persistent_kernel (conv2d + conv2dBackwardData + conv2dBackwardFilterBias)"
# dram__bytes_read.sum + dram__bytes_write.sum of every convolution kernel of one step at
# batch 256 in TF32 mode, from one ncu capture of
# `python -m flashlight_b200.opbench --suite resnet50_step_convs --batch 256 --math tf32`
# (summary under profiles/); algorithmic bytes of the same calls: 66.2e9.  With activations in
# fl's order the layout copies add to it; stored channels-last (`--channels-last`, the default of
# the workload) the kernels move less than the algorithmic figure (consecutive calls of one
# layer find part of their operands in L2).
CONV_DRAM_BYTES_PER_STEP_B256 = 75.2e9
CONV_DRAM_BYTES_PER_STEP_B256_CHANNELS_LAST = 63.8e9
FP32_FMA_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12


def run_gpu_arm(args) -> None:
    import torch

    from flashlight_b200 import _lib as L
    from flashlight_b200 import autograd as A
    from flashlight_b200 import distributed as D
    from flashlight_b200 import functions as F
    from flashlight_b200 import workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device — this library has no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        D.distributedInit("nccl")
    dev = torch.device("cuda", local)

    math_mode = L.MATH_BY_NAME[args.math]
    A.set_math_mode(math_mode)
    model = workloads.resnet50(seed=1234, device=dev)
    reducer = None
    if world > 1:
        D.allReduceParameters(model)
        if args.sync != "none":  # "none": a diagnostic without gradient synchronisation
            reducer = D.BucketReducer(model.parameters(), 1.0 / world, args.bucket_mb << 20,
                                      overlap=args.sync == "overlap")
            D.distributeModuleGrads(model, reducer)

    B = args.batch
    g = torch.Generator().manual_seed(1000 + rank)
    x_host = torch.randn(B, 3, 224, 224, generator=g).pin_memory()
    t_host = torch.randint(0, 1000, (B,), generator=g, dtype=torch.int32).pin_memory()
    x_dev, t_dev = x_host.to(dev), t_host.to(dev)

    timer = OpTimer(torch)
    install_timers(timer, A.extension(), F)

    def step(x, t):
        model.zeroGrad()
        loss = model.loss(x, t)
        loss.backward()
        if reducer is not None:
            reducer.finalize()
        return loss

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(x_dev, t_dev)
    barrier()

    # ---- timed region 1: inputs resident in HBM
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = L.kernel_launches()
    timer.enabled = True
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        loss = step(x_dev, t_dev)
    e1.record()
    barrier()
    timer.enabled = False
    launches = L.kernel_launches() - launches0
    ms_eager = e0.elapsed_time(e1)
    ms_total = ms_eager

    # ---- the same step captured once as a CUDA graph and replayed: no per-operator events, no
    # host work between kernels.  `value` is timed on the replays when capture works; the
    # eager pass above stays the source of the per-operator and roofline figures.
    graph, graph_loss, graph_note, graph_error = None, None, "disabled", None
    if args.graph:
        try:
            static_x, static_t = x_dev.clone(), t_dev.clone()
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step(static_x, static_t)
            torch.cuda.current_stream().wait_stream(side)
            barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                graph_loss = step(static_x, static_t)
            for _ in range(max(args.warmup, 3)):
                graph.replay()
            barrier()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            for _ in range(args.steps):
                graph.replay()
            g1.record()
            barrier()
            ms_total = g0.elapsed_time(g1)
            graph_note = "value and e2e are timed on replays of the step captured as one CUDA graph"
        except Exception as exc:  # capture refused: keep the eager timing
            graph, graph_note = None, "graph capture failed, eager timing kept"
            graph_error = f"{type(exc).__name__}: {exc}"[:300]
            ms_total = ms_eager
            torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None

    # ---- timed region 2: end to end (pinned host batch -> device, loss -> host).  Every step's
    # batch is copied from pinned host memory inside the timed region; the copy of step i + 1
    # runs on a second stream into the other of two device buffers while step i computes.  The
    # loss of step i goes to pinned host memory right behind the step and is read on the host
    # after step i + 1 has been submitted (every loss is read inside the timed region; the
    # host never idles the device while it waits for a number).
    copy_stream = torch.cuda.Stream(device=dev)
    bufs = [(torch.empty_like(x_dev), torch.empty_like(t_dev)) for _ in range(2)]
    consumed = [None, None]  # main-stream event: the last reader of the slot has taken its batch
    loss_host = [torch.empty(1, dtype=torch.float32).pin_memory() for _ in range(2)]

    def fetch(slot):
        with torch.cuda.stream(copy_stream):
            if consumed[slot] is not None:
                copy_stream.wait_event(consumed[slot])
            bufs[slot][0].copy_(x_host, non_blocking=True)
            bufs[slot][1].copy_(t_host, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(copy_stream)
        return ev

    def run_e2e(n):
        ev = fetch(0)
        pending = None  # (event, slot) of the previous step's loss copy
        main = torch.cuda.current_stream()
        for i in range(n):
            main.wait_event(ev)
            xb, tb = bufs[i % 2]
            if graph is not None:
                static_x.copy_(xb)
                static_t.copy_(tb)
                taken = torch.cuda.Event()
                taken.record(main)
                consumed[i % 2] = taken
                if i + 1 < n:
                    ev = fetch((i + 1) % 2)
                graph.replay()
                loss_dev = graph_loss.tensor
            else:
                if i + 1 < n:
                    ev = fetch((i + 1) % 2)
                loss_dev = step(xb, tb).tensor
                taken = torch.cuda.Event()
                taken.record(main)
                consumed[i % 2] = taken
            loss_host[i % 2].copy_(loss_dev.reshape(1), non_blocking=True)
            done = torch.cuda.Event()
            done.record(main)
            if pending is not None:  # the previous step's loss, now that this one is queued
                pending[0].synchronize()
                _ = float(loss_host[pending[1]][0])
            pending = (done, i % 2)
        pending[0].synchronize()
        return float(loss_host[pending[1]][0])

    run_e2e(1)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    last = run_e2e(args.steps)
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)

    # The product configuration takes the batch-norm statistics inside the forward convolutions'
    # epilogues, so their time (and the roofline line below) includes that work.  One more short
    # eager pass with the hand-over switched off times the contraction kernels on their own.
    conv_alone = None
    if world == 1 and A.CONV_STATS_ON and math_mode != L.MATH_STRICT_F32:
        main_records, timer.records = timer.records, []
        A.CONV_STATS_ON = False
        try:
            for _ in range(2):
                step(x_dev, t_dev)
            barrier()
            timer.enabled = True
            for _ in range(min(args.steps, 5)):
                step(x_dev, t_dev)
            barrier()
            timer.enabled = False
            alone = timer.summary()
            conv_alone = {key: sum(alone[k][key] for k in CONV_OPS if k in alone)
                          for key in ("ms", "flops")}
        finally:
            A.CONV_STATS_ON = True
            timer.records = main_records

    if world > 1:
        tt = torch.tensor([ms_total, ms_e2e, ms_eager], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(tt, op=torch.distributed.ReduceOp.MAX)
        ms_total, ms_e2e, ms_eager = float(tt[0]), float(tt[1]), float(tt[2])
    if rank != 0:
        return

    images = world * B * args.steps
    value = images / (ms_total * 1e-3)
    e2e_value = images / (ms_e2e * 1e-3)
    peaks = measured_peaks()
    ops = timer.summary()
    total_op_ms = sum(v["ms"] for v in ops.values()) or 1.0
    # The dominant kernel is the tcgen05 contraction (tc_persistent_kernel) behind the three
    # convolution operators; they are reported as one group, helpers (layout copies, split-K
    # reductions) included, because that is what one convolution call costs.
    conv_ops = [k for k in CONV_OPS if k in ops]
    groups = {k: v for k, v in ops.items() if k not in CONV_OPS}
    if conv_ops:
        groups[CONV_KERNEL] = {key: sum(ops[k][key] for k in conv_ops)
                               for key in ("ms", "flops", "bytes", "calls")}
    top = max(groups, key=lambda k: groups[k]["ms"])
    tv = groups[top]
    if top == CONV_KERNEL or top in TENSOR_OPS:
        achieved = tv["flops"] / (tv["ms"] * 1e-3) / 1e12
        if math_mode != L.MATH_STRICT_F32:
            # TF32 has half the tensor rate of bf16; the measured bf16 cuBLAS figure is the
            # only driver-measured tensor number, so the TF32 peak is taken as half of it.
            peak = peaks["bf16_tflops_sustained"] / 2
            src = f"{peaks['source']} bf16 sustained / 2 (tf32 rate)"
            traffic = None
            if top == CONV_KERNEL and B == 256:
                per_step = (CONV_DRAM_BYTES_PER_STEP_B256_CHANNELS_LAST if workloads.CHANNELS_LAST
                            else CONV_DRAM_BYTES_PER_STEP_B256)
                traffic = per_step * args.steps / max(tv["calls"], 1)
        else:
            peak = FP32_FMA_TFLOPS
            src = "nominal fp32 FMA rate (148 SMs x 128 lanes x 2 x 1.965 GHz): strict mode uses no tensor cores"
            traffic = None
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": traffic, "peak_source": src,
                "per": "convolution call (average over the step's calls)"}
        if top == CONV_KERNEL:
            # Many of the calls (1x1 layers on 56x56 and 28x28 planes) are bounded by HBM, not by
            # the tensor pipe: per call, the floor is the larger of the two roofs.
            floor = timer.floor_ms(CONV_OPS, peak, peaks["hbm_gbs"])
            roof["per_call_floor_ms"] = floor / args.steps
            roof["frac_of_per_call_floor"] = floor / tv["ms"]
            if conv_alone and conv_alone["ms"] > 0:
                a2 = conv_alone["flops"] / (conv_alone["ms"] * 1e-3) / 1e12
                roof["includes"] = ("the batch-norm statistics of the forward convolutions' outputs, "
                                    "taken in their epilogues (conv + batch-norm-statistics fusion)")
                roof["contraction_only"] = {
                    "achieved": a2, "frac": a2 / peak,
                    "what": "the same convolution calls in a short extra eager pass with the "
                            "statistics hand-over off (FLB200_CONV_STATS=0)"}
    else:
        achieved = tv["bytes"] / (tv["ms"] * 1e-3) / 1e9
        peak = peaks["hbm_gbs"]
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": None, "peak_source": peaks["source"]}
    roof["kernel"] = top
    roof["share_of_step"] = tv["ms"] / total_op_ms
    per_op = {}
    for k, v in sorted(ops.items(), key=lambda kv: -kv[1]["ms"]):
        per_op[k] = {"calls_per_step": v["calls"] / args.steps, "ms_per_step": v["ms"] / args.steps,
                     "share": v["ms"] / total_op_ms,
                     "tflops": v["flops"] / (v["ms"] * 1e-3) / 1e12 if v["flops"] else None,
                     "gbs": v["bytes"] / (v["ms"] * 1e-3) / 1e9}

    cpu_base = vendor = others = None
    graph_captured = graph is not None
    if world == 1 and not args.no_cpu_baseline:
        cpu_base, _, _ = cpu_sample(args.cpu_batch, 12, 1, budget_s=25.0)
    if world == 1 and not args.no_side_legs:
        # free the step's tensors first: the side legs build their own models
        del model, graph, timer, bufs
        torch.cuda.empty_cache()
        vendor = vendor_library_leg(torch, B)
        others = other_workloads_leg(torch, peaks)
        A.set_math_mode(math_mode)
    # the loss of this very step (seed 1234, rank 0's batch, initial weights) is a fixed
    # number: 7.0982 in every arithmetic mode to the bound below
    loss_expected = 7.0982 if (B == 256 and world == 1) else None

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": {L.MATH_TF32: "tf32", L.MATH_F32X3: "f32 (3xTF32 tensor-core products)"}.get(
            math_mode, "f32"), "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch_per_gpu": B, "global_batch": B * world,
                   "parallelism": f"dp{world}", "math_mode": args.math,
                   "gradient_sync": args.sync if world > 1 else "none",
                   "l2": "inputs and activations larger than L2 (no flush needed)",
                   "step": "zeroGrad + forward + loss + backward" +
                           (" + bucketed NCCL all-reduce" if world > 1 else ""),
                   "timed_region": graph_note,
                   "host_layer": "Python mirror of fl::AutogradExtension over the C ABI "
                                 "(flashlight_b200/extension.py); the C++ class runs the same "
                                 "entry points behind fl::Tensor in tests/test_fl_harness_gpu.py",
                   "activation_layout": "channels_last" if workloads.CHANNELS_LAST else "fl order (NCHW)",
                   "gpu_launches_counted": "kernel launches of the eager pass of the same K steps "
                                           "(a replay runs the same kernels as graph nodes)"},
        "value_eager": images / (ms_eager * 1e-3), "ms_per_step_eager": ms_eager / args.steps,
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": int(x_host.numel() * 4 + t_host.numel() * 4),
                "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e / args.steps,
                "pipeline": "batch i + 1 is copied host -> device on a second stream while step i "
                            "runs; the loss of step i is copied to pinned host memory behind the "
                            "step and read on the host after step i + 1 has been submitted"},
        "graph_captured": graph_captured, "graph_error": graph_error,
        "gpu_launches": int(launches),
        "clocks": clocks, "roofline": roof, "cpu_baseline": cpu_base, "per_op": per_op,
        "loss": last,
        "loss_check": None if loss_expected is None else {
            "expected": loss_expected, "tolerance": 2e-3,
            "ok": abs(last - loss_expected) <= 2e-3 * loss_expected},
        "vendor_library": vendor, "workloads": others,
    }
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=256, help="images per GPU per step")
    ap.add_argument("--math", default=os.environ.get("FLB200_MATH", "tf32"), choices=["tf32", "strict", "f32x3"])
    ap.add_argument("--bucket-mb", type=int, default=32)
    ap.add_argument("--sync", default="overlap", choices=["overlap", "end", "none"],
                    help="N > 1: gradient all-reduce overlapped with backward (the product), "
                         "all at the end of backward, or none (the last two are diagnostics of "
                         "what the overlap hides and costs)")
    ap.add_argument("--cpu-batch", type=int, default=32)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-side-legs", action="store_true",
                    help="skip the reported-only legs (vendor-library step, the other four workloads)")
    ap.add_argument("--no-graph", dest="graph", action="store_false",
                    help="time the eager step only (default: also capture it as a CUDA graph)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        try:
            run_gpu_arm(args)
        finally:
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized():
                dist.destroy_process_group()


if __name__ == "__main__":
    main()
