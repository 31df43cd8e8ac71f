"""Fused attention backward (flb200_attention_backward) against the operator chain of
flashlight/fl/autograd/Functions.cpp:1828-1891 (matmulNT, softmax, matmul) restated in fp64 with
torch autograd on the bf16-rounded inputs.  bf16 operands, fp32 accumulation: errors are bounded
relative to each tensor's largest magnitude (the probabilities and dS are rounded to bf16 before
they enter the second group of contractions, as in the unfused bf16 chain)."""
import math

import pytest
import torch

from tests.parity import assert_close_scaled, randn

pytestmark = pytest.mark.gpu


def reference(q, k, v, go, scale, causal):
    q, k, v = (t.double().requires_grad_(True) for t in (q, k, v))
    s = scale * q @ k.transpose(1, 2)
    if causal:
        T = s.shape[-1]
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
    o = torch.softmax(s, -1) @ v
    o.backward(go.double())
    return o.detach(), q.grad, k.grad, v.grad


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("Z,T", [(3, 128), (2, 256), (5, 512)])
def test_attention_backward_matches_the_operator_chain(Z, T, causal):
    from flashlight_b200 import functions as F
    hd, scale = 64, 1.0 / math.sqrt(64)
    q = randn(Z, T, hd, seed=90).bfloat16()
    k = randn(Z, T, hd, seed=91).bfloat16()
    v = randn(Z, T, hd, seed=92).bfloat16()
    go = randn(Z, T, hd, seed=93).bfloat16()
    assert F.attention_backward_supported(q.cuda())
    wo, wdq, wdk, wdv = reference(q, k, v, go, scale, causal)
    # forward through the library's kernels: scores, softmax + lse, context
    scores = torch.bmm(q.cuda().float(), k.cuda().float().transpose(1, 2)).bfloat16()
    probs, lse = F.softmax_lse(scores, scale, T if causal else 0)
    s64 = scale * scores.double().cpu()
    if causal:
        s64 = s64.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
    assert_close_scaled(lse.view(Z, T), torch.logsumexp(s64, -1), 1e-5, "lse")
    o = torch.bmm(probs.float(), v.cuda().float()).bfloat16()
    assert_close_scaled(o.float(), wo, 1.6e-2, "attention output")
    dq, dk, dv = F.attention_backward(q.cuda(), k.cuda(), v.cuda(), o, go.cuda(), lse, scale, causal)
    assert dq.dtype == torch.bfloat16
    assert_close_scaled(dv.float(), wdv, 1.6e-2, "attention dv")
    assert_close_scaled(dk.float(), wdk, 1.6e-2, "attention dk")
    assert_close_scaled(dq.float(), wdq, 1.6e-2, "attention dq")


def test_attention_op_fused_and_chain_agree():
    """The tape's attention(): fused gradient where it is built, the operator chain elsewhere
    (fp32 tensors, other head sizes); both against the fp64 reference."""
    from flashlight_b200 import autograd as A
    from flashlight_b200 import functions as F
    Z, T, hd, scale = 4, 256, 64, 0.125
    q, k, v, go = (randn(Z, T, hd, seed=94 + i).bfloat16() for i in range(4))
    _, wdq, wdk, wdv = reference(q, k, v, go, scale, True)
    vars_ = [A.Variable(t.cuda(), True) for t in (q, k, v)]
    out = A.attention(*vars_, scale, causal=True)
    out.backward(go.cuda())
    for var, want, what in zip(vars_, (wdq, wdk, wdv), ("dq", "dk", "dv")):
        assert_close_scaled(var.grad.float(), want, 1.6e-2, f"attention op {what}")
    # a shape the fused kernel is not built for (head dim 32) takes the chain
    q2, k2, v2, go2 = (randn(2, 96, 32, seed=98 + i) for i in range(4))
    assert not F.attention_backward_supported(q2.cuda())
    _, wdq, wdk, wdv = reference(q2, k2, v2, go2, 0.2, True)
    vars2 = [A.Variable(t.cuda(), True) for t in (q2, k2, v2)]
    A.attention(*vars2, 0.2, causal=True).backward(go2.cuda())
    for var, want, what in zip(vars2, (wdq, wdk, wdv), ("dq", "dk", "dv")):
        assert_close_scaled(var.grad, want, 2e-4, f"attention chain {what}")


def test_attention_backward_rejects_what_it_is_not_built_for():
    from flashlight_b200 import _lib as L
    assert L.lib.flb200_attention_backward_supported(512, 64, L.BF16) == 1
    assert L.lib.flb200_attention_backward_supported(500, 64, L.BF16) == 0
    assert L.lib.flb200_attention_backward_supported(512, 128, L.BF16) == 0
    assert L.lib.flb200_attention_backward_supported(512, 64, L.F32) == 0
    st = L.lib.flb200_attention_backward(None, None, None, None, None, None, None, None, None, 1, 128,
                                         64, 1.0, 1, L.BF16, None, 0, None)
    assert st == L.INVALID_ARG
