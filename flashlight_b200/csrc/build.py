"""Builds libflb200.so (the C-ABI kernel library) in-tree with nvcc for sm_100a.

Usage: python -m flashlight_b200.csrc.build [--force] [--verbose]
The shared object is written next to the sources so that it travels with a
snapshot of the repository; nothing is cached outside the tree.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
ROOT = CSRC.parent.parent
INCLUDE = ROOT / "include"
OBJ_DIR = CSRC / "build"
LIB = CSRC / "libflb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-DFLB200_BUILDING=1",
]
# Extra nvcc flags for one-off builds, e.g. FLB200_NVCC_EXTRA=-DFLB200_TC_PROFILE (per-role
# stall accounting of the tensor-core kernel, printed to stderr after every launch).
NVCC_FLAGS += os.environ.get("FLB200_NVCC_EXTRA", "").split()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the flb200 kernels cannot be built")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stamp(src: Path) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(src.read_bytes())
    for hdr in sorted(list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile(src: Path, verbose: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp_file = OBJ_DIR / (src.stem + ".stamp")
    stamp = _stamp(src)
    if obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(INCLUDE), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    stamp_file.write_text(stamp)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    if force:
        for f in OBJ_DIR.glob("*.stamp"):
            f.unlink()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), srcs))
    # The link step is cheap and depends on the SET of objects too (a removed source must
    # disappear from the library), so compare against a manifest rather than mtimes only.
    manifest = OBJ_DIR / "link.manifest"
    want = "\n".join(f"{o.name}:{o.stat().st_mtime_ns}" for o in objs)
    if force or not LIB.exists() or not manifest.exists() or manifest.read_text() != want:
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        manifest.write_text(want)
    return LIB


DIST_SRC = CSRC / "dist" / "dist.cpp"
DIST_LIB = CSRC / "dist" / "libflb200_dist.so"


def build_dist(force: bool = False) -> Path:
    """Builds libflb200_dist.so (gradient synchronisation over NCCL; host code only)."""
    h = hashlib.sha256(DIST_SRC.read_bytes())
    for hdr in sorted(INCLUDE.glob("*.h")):
        h.update(hdr.read_bytes())
    stamp_file = OBJ_DIR / "dist.stamp"
    OBJ_DIR.mkdir(exist_ok=True)
    if (not force and DIST_LIB.exists() and stamp_file.exists()
            and stamp_file.read_text() == h.hexdigest()):
        return DIST_LIB
    cmd = [_nvcc(), "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-I", str(INCLUDE),
           str(DIST_SRC), "-o", str(DIST_LIB), "-lnccl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building {DIST_LIB.name} failed:\n{res.stdout}\n{res.stderr}")
    stamp_file.write_text(h.hexdigest())
    return DIST_LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
    print(build_dist(force="--force" in sys.argv))
