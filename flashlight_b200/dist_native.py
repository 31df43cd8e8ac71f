"""The fl::distributed surface (flashlight/fl/distributed/DistributedApi.h:33-136) over the
native backend libflb200_dist.so instead of torch.distributed: same names and argument meaning
as flashlight_b200.distributed, file-system rendezvous
(DistributedInit::FILE_SYSTEM, backend/cuda/DistributedBackend.cpp:443-487).  CUDA tensors only.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _dist as D

DEFAULT_BUCKET_BYTES = 32 << 20


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def distributedInit(file_path: str, world_rank: int, world_size: int,
                    device: Optional[int] = None, timeout_s: float = 600.0) -> None:
    if device is None:
        device = torch.cuda.current_device()
    torch.cuda.set_device(device)
    D.check(D.lib.flb200_dist_init_file(str(file_path).encode(), world_rank, world_size, device,
                                        float(timeout_s)))


def isDistributedInit() -> bool:
    return bool(D.lib.flb200_dist_is_initialized())


def getWorldRank() -> int:
    return D.lib.flb200_dist_world_rank()


def getWorldSize() -> int:
    return D.lib.flb200_dist_world_size()


def shutdown() -> None:
    D.check(D.lib.flb200_dist_shutdown())


def _dense(t: torch.Tensor) -> torch.Tensor:
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("the native backend reduces dense CUDA tensors in place")
    return t


def allReduce(t: torch.Tensor, scale: float = 1.0, async_: bool = False) -> None:
    _dense(t)
    D.check(D.lib.flb200_dist_all_reduce(t.data_ptr(), t.numel(), D.dtype_code(t.dtype),
                                         float(scale), int(async_), _stream()))


def allReduceMultiple(tensors: Sequence[torch.Tensor], scale: float = 1.0, async_: bool = False,
                      contiguous: bool = False) -> None:
    tensors = [_dense(t) for t in tensors]
    n = len(tensors)
    ptrs = (C.c_void_p * n)(*[t.data_ptr() for t in tensors])
    counts = (C.c_int64 * n)(*[t.numel() for t in tensors])
    dtypes = (C.c_int * n)(*[D.dtype_code(t.dtype) for t in tensors])
    D.check(D.lib.flb200_dist_all_reduce_multiple(ptrs, counts, dtypes, n, float(scale),
                                                  int(async_), int(contiguous), _stream()))


def syncDistributed() -> None:
    D.check(D.lib.flb200_dist_sync(_stream()))


def wait(timeout_s: float) -> None:
    """Host-side wait with a deadline; TimeoutError (and an aborted communicator) afterwards."""
    D.check(D.lib.flb200_dist_wait(float(timeout_s)))


def barrier() -> None:
    D.check(D.lib.flb200_dist_barrier())


class BucketReducer:
    """Reducer::add / finalize (flashlight/fl/distributed/reducers/Reducer.h:21-41) over the
    native bucketed reducer: gradients live inside one flat arena, laid out in REVERSE parameter
    order so that the first bucket fills first during the backward pass; buckets are reduced in
    index order on the backend's stream while the backward pass continues."""

    def __init__(self, params: Sequence, scale: Optional[float] = None,
                 bucket_bytes: int = DEFAULT_BUCKET_BYTES):
        self.params = list(params)[::-1]
        if not self.params:
            raise ValueError("no parameters")
        tensors = [p.tensor for p in self.params]
        dt = tensors[0].dtype
        if any(t.dtype != dt for t in tensors):
            raise ValueError("all parameters of one reducer must have the same type")
        self.scale = 1.0 / getWorldSize() if scale is None else float(scale)
        n = len(tensors)
        counts = (C.c_int64 * n)(*[t.numel() for t in tensors])
        code = D.dtype_code(dt)
        need = D.lib.flb200_reducer_arena_bytes(counts, n, code, bucket_bytes)
        if need < 0:
            D.check(1)
        self.arena = torch.zeros(max(need, 256) // tensors[0].element_size(), dtype=dt,
                                 device=tensors[0].device)
        handle = C.c_void_p()
        D.check(D.lib.flb200_reducer_create(counts, n, code, self.scale, bucket_bytes,
                                            self.arena.data_ptr(), need, C.byref(handle)))
        self.handle = handle
        self.index = {id(p): i for i, p in enumerate(self.params)}
        base = self.arena.data_ptr()
        self.views = []
        for i, t in enumerate(tensors):
            off = (D.lib.flb200_reducer_slot(handle, i) - base) // t.element_size()
            self.views.append(self.arena[off:off + t.numel()].view(t.shape))

    @property
    def num_buckets(self) -> int:
        return D.lib.flb200_reducer_num_buckets(self.handle)

    @property
    def launched(self) -> int:
        return D.lib.flb200_reducer_launched(self.handle)

    def bucket_view(self, p) -> torch.Tensor:
        """Where p's gradient lives: a backward pass that writes here needs no copy."""
        return self.views[self.index[id(p)]]

    def add(self, var) -> None:
        i = self.index[id(var)]
        g = var.grad
        if g is None:
            return
        view = self.views[i]
        src = None if g.data_ptr() == view.data_ptr() else _dense(g).data_ptr()
        D.check(D.lib.flb200_reducer_add(self.handle, i, src, _stream()))
        var.grad = view
        var._grad_owned = True

    def finalize(self) -> None:
        D.check(D.lib.flb200_reducer_finalize(self.handle, _stream()))
        for p, v in zip(self.params, self.views):
            p.grad = v
            p._grad_owned = True

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h and D is not None:  # module globals are gone at interpreter exit
            D.lib.flb200_reducer_destroy(h)
