"""Compile check of B200AutogradExtension against the reference's own headers.

Compiles B200AutogradExtension.cpp to an object file with the flags under which the reference's
tensor / autograd headers build stand-alone (stub tensor backend, no ArrayFire / oneDNN / cuDNN),
so that a signature drift against fl::AutogradExtension is a build error here.  Linking a
Flashlight binary needs ArrayFire and cereal, which this image does not have.
Usage: python check_against_reference.py [reference_root]
"""
import subprocess
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent.parent


def main() -> int:
    sys.path.insert(0, str(ROOT))
    from flashlight_b200._reference import find_reference
    ref = Path(sys.argv[1]) if len(sys.argv) > 1 else find_reference()
    if ref is None or not (ref / "flashlight/fl/autograd/tensor/AutogradExtension.h").exists():
        print("reference headers not found (set FLASHLIGHT_REFERENCE): nothing checked")
        return 0
    out = HERE / "build"
    out.mkdir(exist_ok=True)
    cmd = [
        "g++", "-std=c++20", "-fPIC", "-c", str(HERE / "B200AutogradExtension.cpp"),
        "-o", str(out / "B200AutogradExtension.o"),
        "-I", str(ref), "-I", str(ROOT / "include"), "-I", "/usr/local/cuda/include",
        "-DFL_USE_TENSOR_STUB=1", "-DFL_USE_ARRAYFIRE=0", "-DFL_USE_ONEDNN=0", "-DFL_USE_JIT=0",
        "-DFL_USE_CUDNN=0", "-DFL_BACKEND_CUDA=1", "-DFL_BACKEND_CPU=0", "-DFL_USE_CUDA=1",
        "-Wall", "-Wno-unknown-pragmas",
    ]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        return res.returncode
    print("B200AutogradExtension.cpp compiles against the reference headers")
    return 0


if __name__ == "__main__":
    sys.exit(main())
