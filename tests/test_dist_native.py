"""The native gradient-synchronisation backend (libflb200_dist.so, include/flb200_dist.h).

CPU part: the library loads and exports every declared symbol, and the guards that need neither
a GPU nor peers (not initialised, mixed types, oversize set, a rank 0 that never comes) answer
like the reference's NCCL backend (flashlight/fl/distributed/backend/cuda/DistributedBackend.cpp).
GPU part: one process is a communicator of size 1, which still runs every collective and the
stream ordering for real; two processes on two GPUs when the box has them."""
import ctypes as C
import os
import re
import subprocess
import sys
import time
from pathlib import Path

import pytest
import torch

from flashlight_b200 import _dist as D
from flashlight_b200 import _lib as L

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "flb200_dist.h"


def declared():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(flb200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared()
    assert len(names) == 20
    raw = C.CDLL(str(D.LIB_PATH))
    for n in names:
        assert hasattr(raw, n), n
    assert sorted(D.SIGNATURES) == names


def test_uninitialised_backend_answers_like_the_reference():
    assert D.lib.flb200_dist_is_initialized() == 0
    assert D.lib.flb200_dist_world_rank() == 0 and D.lib.flb200_dist_world_size() == 1
    st = D.lib.flb200_dist_all_reduce(None, 4, L.F32, 1.0, 0, None)
    assert st == L.INVALID_ARG
    assert D.lib.flb200_dist_last_error() == b"distributed environment not initialized"
    assert D.lib.flb200_dist_barrier() == L.INVALID_ARG
    assert D.lib.flb200_dist_sync(None) == L.OK and D.lib.flb200_dist_wait(1.0) == L.OK
    assert D.lib.flb200_dist_shutdown() == L.OK
    h = C.c_void_p()
    counts = (C.c_int64 * 1)(8)
    assert D.lib.flb200_reducer_create(counts, 1, L.F32, 1.0, 1024, None, 0, C.byref(h)) == L.INVALID_ARG


def _set(n, dtypes, counts):
    ptrs = (C.c_void_p * n)(*([0x1000] * n))
    return ptrs, (C.c_int64 * n)(*counts), (C.c_int * n)(*dtypes)


def test_contiguous_set_guards():
    p, c, d = _set(2, [L.F32, L.F16], [4, 4])
    assert D.lib.flb200_dist_all_reduce_multiple(p, c, d, 2, 1.0, 0, 1, None) == L.INVALID_ARG
    assert b"different types" in D.lib.flb200_dist_last_error()
    p, c, d = _set(2, [L.F32, L.F32], [3 << 20, 3 << 20])  # 24 MB > the 20 MB buffer
    assert D.lib.flb200_dist_all_reduce_multiple(p, c, d, 2, 1.0, 0, 1, None) == L.INVALID_ARG
    assert b"larger than existing buffer" in D.lib.flb200_dist_last_error()
    # the empty set is the reference's fast path: fine even before initialisation
    assert D.lib.flb200_dist_all_reduce_multiple(None, None, None, 0, 1.0, 0, 1, None) == L.OK
    # mixed types are allowed when not contiguous: the call gets as far as the init check
    p, c, d = _set(2, [L.F32, L.F16], [4, 4])
    assert D.lib.flb200_dist_all_reduce_multiple(p, c, d, 2, 1.0, 0, 0, None) == L.INVALID_ARG
    assert b"not initialized" in D.lib.flb200_dist_last_error()
    p, c, d = _set(1, [99], [4])
    assert D.lib.flb200_dist_all_reduce_multiple(p, c, d, 1, 1.0, 0, 0, None) == L.INVALID_ARG
    assert b"element type" in D.lib.flb200_dist_last_error()


def test_rendezvous_arguments_and_missing_rank_zero(tmp_path):
    f = str(tmp_path / "id").encode()
    assert D.lib.flb200_dist_init_file(b"", 0, 1, 0, 1.0) == L.INVALID_ARG
    assert b"FilePath" in D.lib.flb200_dist_last_error()
    assert D.lib.flb200_dist_init_file(f, 2, 2, 0, 1.0) == L.INVALID_ARG
    assert D.lib.flb200_dist_init_file(f, 1, 2, 0, 0.0) == L.INVALID_ARG
    t0 = time.time()
    st = D.lib.flb200_dist_init_file(f, 1, 2, 0, 0.3)  # rank 0 never publishes the id
    assert st == L.TIMEOUT and 0.25 < time.time() - t0 < 5
    assert b"did not publish" in D.lib.flb200_dist_last_error()
    with pytest.raises(TimeoutError):
        D.check(st)
    assert D.lib.flb200_dist_is_initialized() == 0


def test_reducer_plan_sizes():
    counts = (C.c_int64 * 4)(100, 3, 1000, 64)
    # every slot is padded to 256 bytes: 512 + 256 + 4096 + 256
    assert D.lib.flb200_reducer_arena_bytes(counts, 4, L.F32, 1 << 20) == 5120
    assert D.lib.flb200_reducer_arena_bytes(counts, 4, L.F16, 1 << 20) == 256 + 256 + 2048 + 256
    assert D.lib.flb200_reducer_arena_bytes(counts, 0, L.F32, 1 << 20) == 0
    assert D.lib.flb200_reducer_arena_bytes(counts, 4, 99, 1 << 20) == -1
    assert D.lib.flb200_reducer_arena_bytes(counts, 4, L.F32, 0) == -1


# ------------------------------------------------------------------------------------- GPU
WORKER = r"""
import sys, torch
sys.path.insert(0, {root!r})
from flashlight_b200 import dist_native as N
from flashlight_b200 import _dist as D, _lib as L
from flashlight_b200.autograd import Variable
rank, world, path = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
dev = rank % torch.cuda.device_count()
N.distributedInit(path, rank, world, device=dev, timeout_s=60)
assert N.isDistributedInit() and N.getWorldRank() == rank and N.getWorldSize() == world
N.distributedInit(path, rank, world, device=dev)          # second call: warning, no error
tot = sum(range(1, world + 1))
x = torch.full((1 << 20,), float(rank + 1), device="cuda")
N.allReduce(x)
assert torch.all(x == tot)
x = torch.arange(4096, device="cuda", dtype=torch.float32) * (rank + 1)
N.allReduce(x, 0.5, True)
N.syncDistributed()
assert torch.equal(x, torch.arange(4096, device="cuda", dtype=torch.float32) * tot * 0.5)
for dt in (torch.float16, torch.bfloat16, torch.float64):
    h = torch.full((1000,), rank + 1.0, device="cuda", dtype=dt)
    N.allReduce(h, 0.25)
    assert torch.all(h == tot * 0.25), dt
i = torch.full((77,), rank + 1, device="cuda", dtype=torch.int64)
N.allReduce(i)
assert torch.all(i == tot)
try:
    N.allReduce(i, 0.5)
    raise SystemExit("scaled integer reduction accepted")
except ValueError as e:
    assert "integer" in str(e)
# sets: grouped with mixed types, packed with one type
a = torch.full((300,), rank + 1.0, device="cuda")
b = torch.full((17, 5), rank + 2.0, device="cuda", dtype=torch.float16)
N.allReduceMultiple([a, b], 1.0, False, False)
assert torch.all(a == tot) and torch.all(b == tot + world)
a = torch.full((300,), rank + 1.0, device="cuda")
c = torch.full((7, 9), rank + 3.0, device="cuda")
e = torch.empty(0, device="cuda")
N.allReduceMultiple([a, e, c], 1.0 / world, True, True)
N.syncDistributed()
assert torch.allclose(a, torch.full_like(a, tot / world)) and torch.allclose(c, torch.full_like(c, tot / world + 2))
N.barrier()
# bucketed reducer: gradients arrive in a rank-dependent order, one never arrives
shapes = [(64, 33), (33,), (128, 64), (64,), (10, 10)]
params = [Variable(torch.zeros(s, device="cuda"), True) for s in shapes]
red = N.BucketReducer(params, bucket_bytes=512)
assert red.num_buckets == 3
for step in range(2):
    order = list(range(len(params)))
    if rank % 2:
        order = order[::-1]
    launched0 = red.launched
    for k in order:
        if k == 3:
            continue                                   # unused parameter
        g = torch.full(shapes[k], float((rank + 1) * (k + 1) + step), device="cuda")
        if k == 2:                                      # written in place: no copy
            red.bucket_view(params[k]).copy_(g)
            params[k].grad = red.bucket_view(params[k])
        else:
            params[k].grad = g
        red.add(params[k])
    try:
        red.add(params[0])
        raise SystemExit("double add accepted")
    except ValueError as e:
        assert "twice" in str(e)
    red.finalize()
    assert red.launched - launched0 == red.num_buckets
    for k, p in enumerate(params):
        want = 0.0 if k == 3 else (tot * (k + 1) + world * step) / world
        assert torch.allclose(p.grad, torch.full(shapes[k], want, device="cuda")), (k, step)
N.wait(30.0)
torch.cuda.synchronize()
N.shutdown()
assert not N.isDistributedInit()
print("ok", rank)
"""


def _run_world(world, tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=str(ROOT)))
    path = str(tmp_path / "nccl_id")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(world), path],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
             for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timed out]"
        outs.append((p.returncode, out))
    for r, (rc, out) in enumerate(outs):
        assert rc == 0 and f"ok {r}" in out, f"rank {r} rc={rc}\n{out[-3000:]}"


@pytest.mark.gpu
def test_native_backend_single_rank(tmp_path):
    _run_world(1, tmp_path)


@pytest.mark.gpu
def test_native_backend_two_ranks(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run_world(2, tmp_path)
