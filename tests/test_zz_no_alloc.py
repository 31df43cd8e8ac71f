"""The channel sum that brings its own scratch (flb200_channel_sum_static_scratch).

It exists for callers that cannot allocate device memory at the moment they need the sum — code
inside a memory-manager callback or an out-of-memory handler, or a host whose device budget was
handed out at start-up — so this test calls it through the C ABI with nothing but the input and
the output, twice in a row (the calls share one built-in array and must not be disturbed by what
the previous call left there), and compares with the entry point that takes caller scratch.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(L, x, outer, channels, inner):
    stream = torch.cuda.current_stream().cuda_stream
    nbytes = L.lib.flb200_channel_sum_workspace_bytes(outer, channels, inner)
    ws = torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device="cuda")
    want = torch.empty(channels, dtype=torch.float32, device="cuda")
    L.check(L.lib.flb200_channel_sum(x.data_ptr(), want.data_ptr(), outer, channels, inner, L.F32,
                                     ws.data_ptr(), nbytes, stream))
    got = torch.full((channels,), float("nan"), dtype=torch.float32, device="cuda")
    L.check(L.lib.flb200_channel_sum_static_scratch(x.data_ptr(), got.data_ptr(), outer, channels,
                                                    inner, L.F32, stream))
    torch.cuda.synchronize()
    return got, want


def test_static_scratch_matches_caller_scratch_on_two_calls_in_a_row():
    from flashlight_b200 import _lib as L
    g = torch.Generator().manual_seed(5)
    # conv bias gradient shape (batch, Cout, Ho*Wo), then a different geometry that reuses the
    # same built-in array with other split counts, then the first one again
    cases = [(16, 64, 56 * 56), (300, 130, 1), (16, 64, 56 * 56)]
    for outer, channels, inner in cases:
        x = torch.randn(outer, channels, inner, generator=g).cuda()
        got, want = _both(L, x, outer, channels, inner)
        # same kernels, same split plan, same order of additions: the results are identical
        assert torch.equal(got, want), (outer, channels, inner)
        ref = x.double().sum(dim=(0, 2)).cpu()
        err = float((got.cpu().double() - ref).abs().max() / ref.abs().max())
        assert err <= 1e-4


def test_static_scratch_refuses_shapes_beyond_its_array():
    from flashlight_b200 import _lib as L
    outer, channels, inner = 4096, 40000, 1   # 40000 channels x 64 splits x 8 B > 1 MiB
    assert L.lib.flb200_channel_sum_workspace_bytes(outer, channels, inner) > (1 << 20)
    x = torch.zeros(8, device="cuda")  # never read: the call must be refused before any launch
    out = torch.zeros(8, device="cuda")
    before = L.lib.flb200_kernel_launches()
    st = L.lib.flb200_channel_sum_static_scratch(x.data_ptr(), out.data_ptr(), outer, channels,
                                                 inner, L.F32, None)
    assert st == L.INVALID_ARG
    assert b"built-in scratch" in L.lib.flb200_last_error()
    assert L.lib.flb200_kernel_launches() == before
