"""ctypes binding of libflb200_dist.so — the C ABI declared in include/flb200_dist.h
(gradient synchronisation over NCCL, one process per GPU).  No fallback: a missing library
raises on import of this module."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import _lib as L

LIB_PATH = Path(__file__).resolve().parent / "csrc" / "dist" / "libflb200_dist.so"

F64, I32, I64 = 16, 17, 18
COALESCE_BYTES = 20 << 20

i64, vp, P = C.c_int64, C.c_void_p, C.POINTER

SIGNATURES = {
    "flb200_dist_init_file": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_double]),
    "flb200_dist_is_initialized": (C.c_int, []),
    "flb200_dist_world_rank": (C.c_int, []),
    "flb200_dist_world_size": (C.c_int, []),
    "flb200_dist_shutdown": (C.c_int, []),
    "flb200_dist_all_reduce": (C.c_int, [vp, i64, C.c_int, C.c_double, C.c_int, vp]),
    "flb200_dist_all_reduce_multiple": (C.c_int, [P(vp), P(i64), P(C.c_int), C.c_int, C.c_double,
                                                  C.c_int, C.c_int, vp]),
    "flb200_dist_sync": (C.c_int, [vp]),
    "flb200_dist_wait": (C.c_int, [C.c_double]),
    "flb200_dist_barrier": (C.c_int, []),
    "flb200_dist_last_error": (C.c_char_p, []),
    "flb200_reducer_arena_bytes": (i64, [P(i64), C.c_int, C.c_int, i64]),
    "flb200_reducer_create": (C.c_int, [P(i64), C.c_int, C.c_int, C.c_double, i64, vp, i64, P(vp)]),
    "flb200_reducer_slot": (vp, [vp, C.c_int]),
    "flb200_reducer_num_buckets": (C.c_int, [vp]),
    "flb200_reducer_bucket_of": (C.c_int, [vp, C.c_int]),
    "flb200_reducer_launched": (C.c_int, [vp]),
    "flb200_reducer_add": (C.c_int, [vp, C.c_int, vp, vp]),
    "flb200_reducer_finalize": (C.c_int, [vp, vp]),
    "flb200_reducer_destroy": (C.c_int, [vp]),
}


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is missing: build it with python -m flashlight_b200.csrc.build")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def check(status: int) -> None:
    if status == L.OK:
        return
    msg = lib.flb200_dist_last_error().decode(errors="replace")
    if status == L.INVALID_ARG:
        raise L.Flb200InvalidArgument(status, msg)
    if status == L.TIMEOUT:
        raise TimeoutError(msg)
    raise L.Flb200Error(status, msg)


def dtype_code(dtype) -> int:
    import torch
    table = {torch.float32: L.F32, torch.float16: L.F16, torch.bfloat16: L.BF16,
             torch.float64: F64, torch.int32: I32, torch.int64: I64}
    if dtype not in table:
        raise ValueError(f"unsupported element type for a reduction: {dtype}")
    return table[dtype]
