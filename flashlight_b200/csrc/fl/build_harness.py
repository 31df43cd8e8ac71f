"""Builds libflb200_fl.so: B200AutogradExtension + B200Tensor / B200Backend + harness.cpp linked
with the reference's own tensor, runtime and autograd-dispatch sources, compiled IN PLACE from
the flashlight checkout (FLASHLIGHT_REFERENCE, or a directory `reference` beside this
repository) with the stub tensor backend selected and every other backend off.  No reference
source is copied; the object files and the shared object stay out of version control.

The shared object links libflb200.so and libflb200_dist.so (the kernel and gradient-
synchronisation libraries, same directory tree) and the CUDA runtime.  Where the checkout is absent nothing is built and the harness test is skipped.
Usage: python build_harness.py [--force]
"""
from __future__ import annotations

import hashlib
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE.parent
ROOT = CSRC.parent.parent
OUT = HERE / "build"
LIB = HERE / "libflb200_fl.so"

REFERENCE_SOURCES = [
    "tensor/TensorBase.cpp", "tensor/TensorBackend.cpp", "tensor/TensorExtension.cpp",
    "tensor/Shape.cpp", "tensor/Types.cpp", "tensor/Index.cpp", "tensor/TensorAdapter.cpp",
    "tensor/Compute.cpp", "tensor/Random.cpp", "tensor/DefaultTensorType.cpp",
    "tensor/backend/stub/StubBackend.cpp", "tensor/backend/stub/StubTensor.cpp",
    "common/DevicePtr.cpp", "common/DynamicBenchmark.cpp", "common/Timer.cpp",
    "runtime/CUDADevice.cpp", "runtime/CUDAStream.cpp", "runtime/CUDAUtils.cpp",
    "runtime/Device.cpp", "runtime/DeviceManager.cpp", "runtime/DeviceType.cpp",
    "runtime/Stream.cpp", "runtime/SynchronousStream.cpp",
    "autograd/tensor/AutogradOps.cpp",
]
OWN_SOURCES = ["B200AutogradExtension.cpp", "B200Tensor.cpp", "B200DistributedBackend.cpp",
               "harness.cpp"]
FLAGS = [
    "-std=c++20", "-O2", "-fPIC", "-DFL_USE_TENSOR_STUB=1", "-DFL_USE_ARRAYFIRE=0",
    "-DFL_USE_ONEDNN=0", "-DFL_USE_JIT=0", "-DFL_USE_CUDNN=0", "-DFL_BACKEND_CUDA=1",
    "-DFL_BACKEND_CPU=0", "-DFL_USE_CUDA=1", "-Wno-unknown-pragmas", "-Wno-deprecated-declarations",
]


def cuda_home() -> Path:
    for cand in ("/usr/local/cuda",):
        if (Path(cand) / "include/cuda_runtime.h").exists():
            return Path(cand)
    raise RuntimeError("CUDA toolkit headers not found")


def build(force: bool = False) -> Path | None:
    sys.path.insert(0, str(ROOT))
    from flashlight_b200._reference import find_reference
    ref = find_reference()
    if ref is None:
        print("flashlight checkout not found (set FLASHLIGHT_REFERENCE): harness not built")
        return LIB if LIB.exists() else None
    from flashlight_b200.csrc import build as kernel_build
    kernel_build.build()
    kernel_build.build_dist()
    OUT.mkdir(exist_ok=True)
    cuda = cuda_home()
    inc = ["-I", str(ref), "-I", str(ROOT / "include"), "-I", str(HERE), "-I", str(cuda / "include")]
    jobs = [(ref / "flashlight/fl" / s, OUT / ("ref_" + s.replace("/", "_") + ".o"))
            for s in REFERENCE_SOURCES]
    jobs += [(HERE / s, OUT / (s + ".o")) for s in OWN_SOURCES]

    def compile_one(job):
        src, obj = job
        h = hashlib.sha256(" ".join(FLAGS).encode() + src.read_bytes())
        for hdr in sorted(HERE.glob("*.h")) + sorted((ROOT / "include").glob("*.h")):
            h.update(hdr.read_bytes())
        stamp = obj.with_suffix(".stamp")
        if not force and obj.exists() and stamp.exists() and stamp.read_text() == h.hexdigest():
            return obj
        res = subprocess.run(["g++", *FLAGS, *inc, "-c", str(src), "-o", str(obj)],
                             capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"g++ failed for {src}:\n{res.stdout}\n{res.stderr}")
        stamp.write_text(h.hexdigest())
        return obj

    with ThreadPoolExecutor(max_workers=8) as pool:
        objs = list(pool.map(compile_one, jobs))
    cmd = ["g++", "-shared", "-o", str(LIB), *map(str, objs), "-L", str(CSRC), "-lflb200",
           "-L", str(CSRC / "dist"), "-lflb200_dist", "-Wl,-rpath,$ORIGIN/../dist",
           "-L", str(cuda / "lib64"), "-lcudart", "-Wl,-rpath,$ORIGIN/..",
           "-Wl,-rpath," + str(cuda / "lib64"), "-Wl,--no-undefined"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
