"""Host logic of the data-parallel gradient sync on CPU ranks (gloo, world size 2): value
patterns as flashlight/fl/test/distributed/AllReduceTest.cpp:23-183, the reference's guards
(mixed dtypes, oversize contiguous set, uninitialised use) and the bucket reducer."""
import os
import tempfile

import pytest
import torch
import torch.multiprocessing as mp


def _worker(rank, world, initfile, fn_name, q):
    try:
        os.environ.pop("MASTER_ADDR", None)
        from flashlight_b200 import distributed as D
        D.distributedInit("gloo", rank, world, init_method=f"file://{initfile}", timeout_s=60)
        globals()[fn_name](rank, world, D)
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover - reported to the parent
        import traceback
        q.put((rank, traceback.format_exc()))


def _run(fn_name, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        initfile = os.path.join(d, "rendezvous")
        procs = [ctx.Process(target=_worker, args=(r, world, initfile, fn_name, q)) for r in range(world)]
        for p in procs:
            p.start()
        results = [q.get(timeout=120) for _ in procs]
        for p in procs:
            p.join(timeout=60)
    for rank, res in results:
        assert res == "ok", f"rank {rank}:\n{res}"


def _values(rank, world, D):
    assert D.getWorldRank() == rank and D.getWorldSize() == world
    t = torch.full((3, 5), float(rank))
    D.allReduce(t, scale=2.0)
    expect = world * (world - 1) / 2 * 2.0
    assert torch.all(t == expect)
    # asynchronous set, then syncDistributed
    ts = [torch.full((4,), float(rank + i)) for i in range(6)]
    D.allReduceMultiple(ts, scale=1.0 / world, async_=True, contiguous=False)
    D.syncDistributed()
    for i, v in enumerate(ts):
        assert torch.allclose(v, torch.full((4,), (world - 1) / 2 + i))
    # contiguous set
    ts = [torch.full((7, 3), float(rank)), torch.full((2,), float(rank * 10))]
    D.allReduceMultiple(ts, scale=1.0, async_=False, contiguous=True)
    assert torch.all(ts[0] == world * (world - 1) / 2) and torch.all(ts[1] == 10 * world * (world - 1) / 2)
    D.barrier()


def _guards(rank, world, D):
    big = [torch.zeros(3 << 20) for _ in range(2)]  # 24 MB > 20 MB coalescing buffer
    with pytest.raises(RuntimeError, match="exceeds"):
        D.allReduceMultiple(big, contiguous=True)
    with pytest.raises(RuntimeError, match="same type"):
        D.allReduceMultiple([torch.zeros(2), torch.zeros(2, dtype=torch.float64)], contiguous=True)
    D.barrier()


class _Var:
    def __init__(self, t):
        self.tensor, self.grad, self._grad_owned, self.grad_hook = t, None, False, None

    def registerGradHook(self, h):
        self.grad_hook = h


class _Mod:
    def __init__(self, ps):
        self.ps = ps

    def parameters(self):
        return self.ps


def _reducers(rank, world, D):
    sizes = [(5, 3), (100,), (7, 7, 2), (1,), (64, 64)]
    # coalescing reducer, reference semantics (tiny threshold forces flushes and the oversize path)
    ps = [_Var(torch.zeros(s)) for s in sizes]
    red = D.CoalescingReducer(1.0 / world, True, True, cache_threshold_bytes=1024)
    D.distributeModuleGrads(_Mod(ps), red)
    for i, p in enumerate(reversed(ps)):
        p.grad = torch.full(p.tensor.shape, float(rank + 1) * (i + 1))
        p.grad_hook(p)
    red.finalize()
    for i, p in enumerate(reversed(ps)):
        assert torch.allclose(p.grad, torch.full(p.tensor.shape, (world + 1) / 2 * (i + 1)))
    # bucket reducer: gradients become views of the flat buckets, values averaged
    ps = [_Var(torch.zeros(s)) for s in sizes]
    red = D.BucketReducer(ps, bucket_bytes=4096)
    assert len(red.buckets) >= 2
    D.distributeModuleGrads(_Mod(ps), red)
    for step in range(2):
        for i, p in enumerate(reversed(ps)):
            p.grad = torch.full(p.tensor.shape, float(rank + 1) * (i + 1) + step)
            p.grad_hook(p)
        red.finalize()
        for i, p in enumerate(reversed(ps)):
            assert torch.allclose(p.grad, torch.full(p.tensor.shape, (world + 1) / 2 * (i + 1) + step))
            assert p.grad.data_ptr() == red.bucket_view(p).data_ptr()
    # One rank skips a parameter and the gradients arrive in another order than the buckets:
    # every rank still issues one collective per bucket, in bucket order, the skipped slice
    # contributes zeros (not the previous step's values), and both ranks end with the same
    # gradient for every parameter.
    skip = 1  # ps[1] gets no gradient on rank 1
    order = [0, 4, 2, 1, 3] if rank == 0 else [3, 0, 4, 2]
    for i in order:
        p = ps[i]
        p.grad = torch.full(p.tensor.shape, float(10 * (rank + 1) + i))
        p.grad_hook(p)
    if rank == 1:
        ps[skip].grad = None
    red.finalize()
    for i, p in enumerate(ps):
        ranks = [r for r in range(world) if not (r == 1 and i == skip)]
        want = sum(10 * (r + 1) + i for r in ranks) / world
        assert p.grad is not None and torch.allclose(p.grad, torch.full(p.tensor.shape, want)), (i, p.grad)
    # the same gradient twice in one step is a host-side error before any collective
    ps[0].grad = torch.ones(sizes[0])
    red.add(ps[0])
    with pytest.raises(RuntimeError, match="twice"):
        red.add(ps[0])
    for p in ps[1:]:
        p.grad = torch.ones(p.tensor.shape)
        red.add(p)
    red.finalize()
    D.barrier()


def test_allreduce_values_world2():
    _run("_values")


def test_reference_guards_world2():
    _run("_guards")


def test_reducers_world2():
    _run("_reducers")


def test_uninitialised_world_is_size_one():
    from flashlight_b200 import distributed as D
    assert D.getWorldSize() == 1 and D.getWorldRank() == 0
    t = torch.ones(4)
    D.allReduce(t, scale=0.5)  # world-size-1 fast path: scale only (DistributedApi.cpp:25-27)
    assert torch.all(t == 0.5)
    D.allReduceMultiple([t], scale=2.0)
    assert torch.all(t == 1.0)
    D.syncDistributed()
