"""Data-parallel gradient synchronisation: the fl::distributed API surface
(flashlight/fl/distributed/DistributedApi.h:33-136) and its reducers
(flashlight/fl/distributed/reducers/*.cpp, flashlight/fl/nn/DistributedUtils.cpp:16-43)
over torch.distributed — NCCL across the NVLink/NVSwitch domain of one box, gloo
on CPU for the host-logic tests.  One process per GPU.

What differs from the reference's NCCL backend
(flashlight/fl/distributed/backend/cuda/DistributedBackend.cpp:127-227):
  * gradients are packed into flat buckets laid out in REVERSE parameter order, so
    the bucket that fills first during backward is reduced while earlier layers are
    still computing; each bucket is one in-place all-reduce on the communication
    stream, ordered against the compute stream by events (async_op);
  * the 1/world scale rides on the collective (ncclAvg) instead of a second pass
    over every tensor (DistributedApi.cpp:44-46);
  * after finalize() each parameter's gradient IS its slice of the bucket: there is
    no scatter copy back.
"""
from __future__ import annotations

import os
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

DEFAULT_BUCKET_BYTES = 32 << 20
# flashlight/fl/common/Defines.h:97 — size of the reference's coalescing buffer
REFERENCE_CACHE_BYTES = 20 << 20

_pending: List = []


def distributedInit(backend: Optional[str] = None, world_rank: Optional[int] = None,
                    world_size: Optional[int] = None, init_method: Optional[str] = None,
                    timeout_s: float = 600.0) -> None:
    """fl::distributedInit: rendezvous from the launcher's environment (RANK, WORLD_SIZE,
    MASTER_ADDR, MASTER_PORT) or an explicit init_method such as a shared file, the
    counterpart of DistributedInit::FILE_SYSTEM."""
    if dist.is_initialized():
        return
    import datetime
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    kw = dict(backend=backend, timeout=datetime.timedelta(seconds=timeout_s))
    if init_method is not None:
        kw.update(init_method=init_method, rank=world_rank, world_size=world_size)
    elif world_rank is not None:
        kw.update(rank=world_rank, world_size=world_size)
    if backend == "nccl":
        local = int(os.environ.get("LOCAL_RANK", world_rank or 0))
        torch.cuda.set_device(local)
        kw["device_id"] = torch.device("cuda", local)
    dist.init_process_group(**kw)


def isDistributedInit() -> bool:
    return dist.is_initialized()


def getWorldRank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def getWorldSize() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def _require_init():
    if not dist.is_initialized():
        # backend/cuda/DistributedBackend.cpp:113-115
        raise RuntimeError("distributed environment not initialized")


def _supports_avg() -> bool:
    return dist.get_backend() == "nccl"


def _reduce(t: torch.Tensor, scale: float, async_: bool):
    """In-place sum all-reduce followed by `scale`; scale == 1/world folds into ncclAvg."""
    world = getWorldSize()
    use_avg = _supports_avg() and t.is_floating_point() and abs(scale * world - 1.0) < 1e-12
    op = dist.ReduceOp.AVG if use_avg else dist.ReduceOp.SUM
    work = dist.all_reduce(t, op=op, async_op=True)
    post = None if (use_avg or scale == 1.0) else scale
    if async_:
        _pending.append((work, t, post))
    else:
        work.wait()
        if post is not None:
            t.mul_(post)


def allReduce(t: torch.Tensor, scale: float = 1.0, async_: bool = False) -> None:
    """fl::allReduce(Variable&, scale, async) (DistributedApi.cpp:23-29)."""
    if getWorldSize() > 1:
        _require_init()
        _reduce(t, scale, async_)
    elif scale != 1.0:
        t.mul_(scale)


def allReduceMultiple(tensors: Sequence[torch.Tensor], scale: float = 1.0, async_: bool = False,
                      contiguous: bool = False) -> None:
    """fl::allReduceMultiple (DistributedApi.cpp:31-47).  contiguous=True coalesces the set into
    one flat buffer first; like the reference it refuses mixed dtypes and sets larger than the
    coalescing buffer (backend/cuda/DistributedBackend.cpp:148-155, 172-175)."""
    tensors = list(tensors)
    if not tensors:
        return
    if getWorldSize() <= 1:
        if scale != 1.0:
            for t in tensors:
                t.mul_(scale)
        return
    _require_init()
    if not contiguous:
        for t in tensors:
            _reduce(t, scale, async_)
        return
    dt = tensors[0].dtype
    if any(t.dtype != dt for t in tensors):
        raise RuntimeError("allReduceMultiple: all tensors in a contiguous set must have the same type")
    total = sum(t.numel() * t.element_size() for t in tensors)
    if total > REFERENCE_CACHE_BYTES:
        raise RuntimeError("allReduceMultiple: total size of the contiguous set exceeds the "
                           "coalescing buffer")
    flat = torch.cat([t.reshape(-1) for t in tensors])
    _reduce(flat, scale, False)
    off = 0
    for t in tensors:
        n = t.numel()
        t.copy_(flat[off:off + n].reshape(t.shape))
        off += n


def syncDistributed() -> None:
    """fl::syncDistributed: the compute stream waits for every outstanding collective
    (backend/cuda/DistributedBackend.cpp:233-245)."""
    while _pending:
        work, t, post = _pending.pop(0)
        work.wait()
        if post is not None:
            t.mul_(post)


def barrier() -> None:
    """fl::barrier: an all-reduce of one int (DistributedApi.cpp:49-56)."""
    if getWorldSize() > 1:
        t = torch.zeros(1, dtype=torch.int32,
                        device="cuda" if dist.get_backend() == "nccl" else "cpu")
        dist.all_reduce(t)
        t.item()


# ------------------------------------------------------------------ reducers
class Reducer:
    """flashlight/fl/distributed/reducers/Reducer.h:21-40."""

    def add(self, var) -> None:
        raise NotImplementedError

    def finalize(self) -> None:
        raise NotImplementedError


class InlineReducer(Reducer):
    """reducers/InlineReducer.cpp: reduce every gradient as it arrives."""

    def __init__(self, scale: float):
        self.scale = scale

    def add(self, var) -> None:
        if var.grad is not None:
            allReduce(var.grad, self.scale)

    def finalize(self) -> None:
        pass


class CoalescingReducer(Reducer):
    """reducers/CoalescingReducer.cpp:24-63 with the reference's semantics: cache gradients up to
    a threshold, flush through allReduceMultiple, oversize tensors go alone."""

    def __init__(self, scale: float, async_: bool = True, contiguous: bool = True,
                 cache_threshold_bytes: int = REFERENCE_CACHE_BYTES):
        self.scale, self.async_, self.contiguous = scale, async_, contiguous
        self.threshold = cache_threshold_bytes
        self.cache: List[torch.Tensor] = []
        self.cache_bytes = 0

    def add(self, var) -> None:
        g = var.grad
        if g is None:
            return
        nbytes = g.numel() * g.element_size()
        if self.cache_bytes + nbytes > self.threshold:
            self.flush()
        if nbytes > self.threshold:
            allReduce(g, self.scale, self.async_)
        else:
            self.cache.append(g)
            self.cache_bytes += nbytes

    def flush(self) -> None:
        allReduceMultiple(self.cache, self.scale, self.async_, self.contiguous)
        self.cache, self.cache_bytes = [], 0

    def finalize(self) -> None:
        self.flush()
        syncDistributed()


class BucketReducer(Reducer):
    """The B200 reducer: flat buckets in reverse parameter order, one in-place asynchronous
    all-reduce per bucket, no copy back.

    The collectives of a step are issued in bucket order on every rank, whatever order the
    gradients arrive in: a bucket whose last gradient has landed is reduced as soon as every
    bucket before it has been, and finalize() reduces the rest in the same order.  A parameter
    that received no gradient on this rank contributes zeros (its slice is cleared first, so that
    nothing of an earlier step is averaged in); ranks on which different parameters went unused
    therefore still pair the same buffers, and after finalize() every rank holds the same
    averaged gradient for every parameter of a reduced bucket."""

    def __init__(self, params: Sequence, scale: Optional[float] = None,
                 bucket_bytes: int = DEFAULT_BUCKET_BYTES, overlap: bool = True):
        self.params = list(params)
        # overlap=False: nothing is reduced before finalize() (same collectives, same order, no
        # overlap with the backward pass) — the comparison point for what the overlap costs the
        # compute kernels and what it hides
        self.overlap = overlap
        self.scale = (1.0 / getWorldSize()) if scale is None else scale
        self.slot = {}
        self.buckets: List[torch.Tensor] = []
        self.members: List[List] = []
        cur: List = []
        cur_bytes = 0
        groups: List[List] = []
        for p in reversed(self.params):
            nbytes = p.tensor.numel() * p.tensor.element_size()
            if cur and (cur_bytes + nbytes > bucket_bytes or cur[0].tensor.dtype != p.tensor.dtype):
                groups.append(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
        if cur:
            groups.append(cur)
        for bi, grp in enumerate(groups):
            n = sum(p.tensor.numel() for p in grp)
            flat = torch.zeros(n, dtype=grp[0].tensor.dtype, device=grp[0].tensor.device)
            off = 0
            for p in grp:
                self.slot[id(p)] = (bi, off, p.tensor.numel())
                off += p.tensor.numel()
            self.buckets.append(flat)
            self.members.append(list(grp))
        self.expected = [len(g) for g in self.members]
        self._reset()

    def _reset(self) -> None:
        self.remaining = list(self.expected)
        self.arrived = [set() for _ in self.members]
        self.next_bucket = 0  # buckets below this index have been reduced in this step

    def bucket_view(self, p) -> torch.Tensor:
        bi, off, n = self.slot[id(p)]
        return self.buckets[bi][off:off + n].view(p.tensor.shape)

    def _fire_ready(self) -> None:
        if not self.overlap:
            return
        while self.next_bucket < len(self.buckets) and self.remaining[self.next_bucket] == 0:
            allReduce(self.buckets[self.next_bucket], self.scale, True)
            self.next_bucket += 1

    def add(self, var) -> None:
        if var.grad is None:
            return
        bi, off, n = self.slot[id(var)]
        if id(var) in self.arrived[bi]:
            raise RuntimeError("BucketReducer: a parameter's gradient was added twice in one step")
        if bi < self.next_bucket:
            raise RuntimeError("BucketReducer: gradient arrived after its bucket was reduced")
        view = self.buckets[bi][off:off + n].view(var.tensor.shape)
        if var.grad.data_ptr() != view.data_ptr():
            view.copy_(var.grad)
            var.grad = view
            var._grad_owned = True
        self.arrived[bi].add(id(var))
        self.remaining[bi] -= 1
        self._fire_ready()

    def finalize(self) -> None:
        world = getWorldSize()
        for bi in range(self.next_bucket, len(self.buckets)):
            for p in self.members[bi]:
                if id(p) not in self.arrived[bi]:
                    # unused on this rank in this step: contribute zeros, not last step's values
                    self.bucket_view(p).zero_()
                    if world > 1:
                        p.grad = self.bucket_view(p)
                        p._grad_owned = True
            if world > 1:
                allReduce(self.buckets[bi], self.scale, True)
        self.next_bucket = len(self.buckets)
        syncDistributed()
        self._reset()


def distributeModuleGrads(module, reducer: Reducer) -> None:
    """flashlight/fl/nn/DistributedUtils.cpp:16-22: a grad hook per parameter."""
    for p in module.parameters():
        p.registerGradHook(lambda v, r=reducer: r.add(v))


def allReduceParameters(module) -> None:
    """DistributedUtils.cpp:24-32: average the replicas' parameters (initial sync)."""
    scale = 1.0 / getWorldSize()
    for p in module.parameters():
        allReduce(p.tensor, scale)


def allReduceGradients(module, scale: float = 1.0) -> None:
    for p in module.parameters():
        if p.grad is not None:
            allReduce(p.grad, scale)
