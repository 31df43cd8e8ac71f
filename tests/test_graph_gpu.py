"""The training step captured as one CUDA graph replays to the same loss and gradients as the
eager step: nothing in the library synchronises, allocates outside the caller's allocator or
keeps host-side state that a replay would miss (tensor maps are kernel arguments, workspaces
come from the caller)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode_name", ["tf32", "strict"])
def test_resnet_step_replays_bit_for_bit(mode_name):
    from flashlight_b200 import _lib as L
    from flashlight_b200 import autograd as A
    from flashlight_b200 import workloads
    A.set_math_mode(L.MATH_BY_NAME[mode_name])
    try:
        model = workloads.resnet50(seed=5, blocks=(1, 1, 1), classes=10, width=16)
        g = torch.Generator().manual_seed(3)
        x = torch.randn(4, 3, 112, 112, generator=g).cuda()
        t = torch.randint(0, 10, (4,), generator=g, dtype=torch.int32).cuda()

        def step():
            model.zeroGrad()
            loss = model.loss(x, t)
            loss.backward()
            return loss.tensor

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            want_loss = step().clone()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        want = [p.grad.clone() for p in model.parameters()]

        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            got_loss = step()
        for _ in range(2):  # a replay leaves the same result every time
            for p in model.parameters():
                p.grad.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(got_loss, want_loss)
            for p, w in zip(model.parameters(), want):
                assert torch.equal(p.grad, w)
        # new inputs in the captured buffers give the new step's result
        x.copy_(torch.randn(4, 3, 112, 112, generator=g))
        graph.replay()
        replayed = [p.grad.clone() for p in model.parameters()]
        fresh_loss = step()
        torch.cuda.synchronize()
        assert torch.equal(got_loss, fresh_loss) or abs(float(got_loss) - float(fresh_loss)) < 1e-6
        for r, p in zip(replayed, model.parameters()):
            assert torch.equal(r, p.grad)
    finally:
        A.set_math_mode(L.MATH_STRICT_F32)
    assert L.lib.flb200_tc_poll_status(None) == 0
