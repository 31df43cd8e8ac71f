"""Pins the CPU oracle (oracle/flref.py) before anything is compared against it.

* the reference's own forward goldens for RNN / LSTM / GRU are parsed from its test
  file at run time (skipped where the reference checkout is absent);
* the torch-backed oracle functions are checked against plain fp64 loops;
* the closed-form and finite-difference protocols of the reference's tests are
  replayed on the oracle (AutogradTestUtils.h:33-70, AutogradNormalizationTest.cpp).
"""
import re

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import flref as R
from tests.parity import randn, rel_err


# ------------------------------------------------ reference goldens (RNN)
def _grab(src: str, test: str):
    body = re.search(r"TEST\(ModuleTest, %s\)(.*?)\n}\n" % test, src, re.S).group(1)
    geti = lambda k: int(re.search(r"int %s = (\d+);" % k, body).group(1))
    cfg = dict(L=geti("num_layers"), H=geti("hidden_size"), I=geti("input_size"),
               B=geti("batch_size"), T=geti("seq_length"))
    cfg["n"] = int(re.search(r"n_params = (\d+);", body).group(1))
    scales = [float(x) for x in re.findall(r"\(i \+ 1\) \* ([0-9.]+);", body)]
    cfg["sin"], cfg["sw"] = scales[0], scales[1]
    arr = re.search(r"expected_dims,\s*\{(.*?)\}\)", body, re.S).group(1)
    cfg["vals"] = np.array([float(x) for x in re.findall(r"-?\d+\.\d+(?:[eE]-?\d+)?", arr)])
    return cfg


@pytest.mark.parametrize("test,mode", [("RNNFwd", R.RNN_RELU), ("LSTMFwd", R.RNN_LSTM),
                                       ("GRUFwd", R.RNN_GRU)])
def test_rnn_forward_matches_reference_goldens(reference_root, test, mode):
    src = (reference_root / "flashlight/fl/test/nn/ModuleTest.cpp").read_text()
    c = _grab(src, test)
    assert R.rnn_num_params(c["I"], c["H"], c["L"], mode, False) == c["n"]
    w = torch.arange(1, c["n"] + 1, dtype=torch.float64) * c["sw"]
    x = (torch.arange(1, c["I"] * c["B"] * c["T"] + 1, dtype=torch.float64) * c["sin"]).reshape(
        c["T"], c["B"], c["I"])
    y, _, _ = R.rnn(x, None, None, w, c["H"], c["L"], mode, False)
    got = y.numpy().reshape(-1)
    assert got.shape == c["vals"].shape
    # goldens carry 4 decimals; the reference test itself uses allClose(1e-4)
    assert np.abs(got - c["vals"]).max() < 1e-4


# ------------------------- reference goldens (Embedding, Linear, LogSoftmax, LayerNorm)
def _literals(src: str, test: str):
    """Every Tensor::fromVector<float>({shape}, {values}) literal of one TEST body, in order, as
    fp64 tensors in torch order (reversed fl shape; the flat value order is the same bytes)."""
    body = re.search(r"TEST\(ModuleTest, %s\)(.*?)\n}\n" % test, src, re.S).group(1)
    out = []
    for m in re.finditer(r"fromVector<float>\(\s*\{([^}]*)\},\s*\{([^}]*)\}\)", body, re.S):
        names = dict(re.findall(r"(\w+) = (\d+)", body))
        shape = [int(names.get(t.strip(), t.strip())) for t in m.group(1).split(",")]
        vals = [float(v) for v in re.findall(r"-?\d+\.?\d*(?:[eE]-?\d+)?", m.group(2))]
        out.append(torch.tensor(vals, dtype=torch.float64).reshape(list(reversed(shape))))
    return out


def _module_tests(reference_root):
    return (reference_root / "flashlight/fl/test/nn/ModuleTest.cpp").read_text()


def test_committed_fixture_equals_the_checkout(reference_root):
    """tests/golden/reference_module_goldens.npz (what the GPU tests read) holds exactly what a
    fresh parse of the checkout gives."""
    import importlib.util
    from pathlib import Path
    path = Path(__file__).resolve().parent / "golden" / "make_reference_goldens.py"
    spec = importlib.util.spec_from_file_location("make_reference_goldens", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    fresh = mod.collect(reference_root)
    stored = np.load(mod.OUT)
    assert sorted(stored.files) == sorted(fresh)
    for k, v in fresh.items():
        assert np.array_equal(stored[k], v), k


def test_embedding_matches_reference_golden(reference_root):
    """ModuleTest EmbeddingFwd: table [embDim, nEmb], ids [nQuery, batch] -> [embDim, nQuery, batch]."""
    table, ids, want = _literals(_module_tests(reference_root), "EmbeddingFwd")[:3]
    got = R.embedding(table, ids.to(torch.int64)).reshape(want.shape)
    assert torch.equal(got, want)


def test_linear_matches_reference_goldens(reference_root):
    """ModuleTest LinearFwd: fl weight [n_out, n_in] (torch (n_in, n_out)), with and without bias."""
    w, x, want, bias, want_b = _literals(_module_tests(reference_root), "LinearFwd")[:5]
    assert torch.equal(R.linear(x, w, None), want)
    assert torch.equal(R.linear(x, w, bias), want_b)


def test_log_softmax_matches_reference_goldens(reference_root):
    """ModuleTest LogSoftmaxFwd: over fl dim 0 (the oracle's own axis) and over fl dim 1 (the
    same function on the transposed view); goldens carry 6 digits, the test uses allClose(1e-4)."""
    x, want0, want1 = _literals(_module_tests(reference_root), "LogSoftmaxFwd")[:3]
    assert (R.log_softmax(x) - want0).abs().max() < 1e-4
    assert (R.log_softmax(x.t()).t() - want1).abs().max() < 1e-4


def test_layer_norm_matches_reference_closed_form(reference_root):
    """ModuleTest LayerNormFwd holds no literal output: it compares the module with
    (x - mean) / sqrt(var_biased + eps) over the normalised axis.  Replayed on the oracle with the
    reference's shapes, axis and eps (read from the test), for its three module variants."""
    body = re.search(r"TEST\(ModuleTest, LayerNormFwd\)(.*?)\n}\n", _module_tests(reference_root), re.S).group(1)
    eps = float(re.search(r"double eps = ([0-9.eE-]+);", body).group(1))
    axis = int(re.search(r"feat_axes = \{(\d+)\}", body).group(1))
    feat = int(re.search(r"int F = (\d+);", body).group(1))
    shape = [int(v) for v in re.search(r"fl::rand\(\{([^}]*)\}\)", body).group(1).replace("F", str(feat)).split(",")]
    assert (eps, axis, shape) == (1e-5, 3, [4, 4, 3, 10])
    x = randn(*reversed(shape), seed=7, dtype=torch.float64)   # torch view of fl [4, 4, 3, F]
    tdim = len(shape) - 1 - axis                               # fl axis 3 = torch dim 0
    true_out = (x - x.mean(tdim, keepdim=True)) / torch.sqrt(x.var(tdim, unbiased=False, keepdim=True) + eps)
    assert (R.layer_norm(x, [axis], eps) - true_out).abs().max() < eps
    ones = torch.ones(feat, dtype=torch.float64).reshape(-1, 1, 1, 1)
    zeros = torch.zeros(feat, dtype=torch.float64).reshape(-1, 1, 1, 1)
    assert (R.layer_norm(x, [axis], eps, ones, zeros) - true_out).abs().max() < eps
    x3 = randn(3, 4, 4, seed=8, dtype=torch.float64)           # fl [4, 4, 3], axes {0}
    want3 = (x3 - x3.mean(-1, keepdim=True)) / torch.sqrt(x3.var(-1, unbiased=False, keepdim=True) + eps)
    assert (R.layer_norm(x3, [0], eps) - want3).abs().max() < eps


def test_conv_padding_shapes_of_reference_module_test(reference_root):
    """ModuleTest ConvPadding pins SAME padding and the output-extent formula: the three output
    shapes are read from the test and reproduced with derive_padding + conv_out_dim."""
    from flashlight_b200.nn import SAME, derive_padding
    body = re.search(r"TEST\(ModuleTest, ConvPadding\)(.*?)\n}\n", _module_tests(reference_root), re.S).group(1)
    shapes = [[int(v) for v in m.split(",")] for m in re.findall(r"Shape\(\{([^}]*)\}\)", body)]
    assert len(shapes) == 3
    # Conv2D(30, 100, wx, wy, sx, sy, px, py, [dx, dy]) on a 32 x 32 x 30 x 2 input
    cases = [(3, 5, 2, 1, SAME, 0, 1, 1), (3, 5, 2, 1, SAME, SAME, 1, 1), (10, 10, 1, 1, SAME, SAME, 4, 4)]
    for (wx, wy, sx, sy, px, py, dx, dy), want in zip(cases, shapes):
        pxx, pyy = derive_padding(32, wx, sx, px, dx), derive_padding(32, wy, sy, py, dy)
        got = [R.conv_out_dim(32, wx, sx, pxx, dx), R.conv_out_dim(32, wy, sy, pyy, dy), 100, 2]
        assert got == want, (got, want)


def test_rnn_param_counts_of_reference_backward_test(reference_root):
    """AutogradRnnTest.cpp pins the flat weight size for 2 layers, H=2, in=2, bidirectional."""
    src = (reference_root / "flashlight/fl/test/autograd/AutogradRnnTest.cpp").read_text()
    counts = [int(v) for v in re.findall(r"testRnnImpl\(RnnMode::\w+[^;]*?(\d+)\)?;", src)]
    ours = {R.rnn_num_params(2, 2, 2, m, True) for m in (R.RNN_RELU, R.RNN_LSTM, R.RNN_GRU)}
    assert ours == {56, 224, 168}
    for v in (56, 224, 168):
        assert str(v) in src


def test_oracle_rnn_matches_torch_modules():
    """Bidirectional multi-layer: the oracle's own recurrence equals torch.nn.LSTM / GRU with the
    flat vector unpacked in (layer, direction) order — the cuDNN order adopted for parity."""
    I, H, L, B, T = 3, 4, 2, 2, 5
    for mode, mod in ((R.RNN_LSTM, torch.nn.LSTM), (R.RNN_GRU, torch.nn.GRU)):
        n = R.rnn_num_params(I, H, L, mode, True)
        w = randn(n, seed=3, dtype=torch.float64) * 0.3
        x = randn(T, B, I, seed=4, dtype=torch.float64)
        net = mod(I, H, L, bidirectional=True).double()
        params = R.rnn_unpack(w, I, H, L, mode, True)
        with torch.no_grad():
            for l in range(L):
                for d, suf in enumerate(("", "_reverse")):
                    wih, whh, bih, bhh = params[l * 2 + d]
                    getattr(net, f"weight_ih_l{l}{suf}").copy_(wih)
                    getattr(net, f"weight_hh_l{l}{suf}").copy_(whh)
                    getattr(net, f"bias_ih_l{l}{suf}").copy_(bih)
                    getattr(net, f"bias_hh_l{l}{suf}").copy_(bhh)
        want, _ = net(x)
        got, hy, cy = R.rnn(x, None, None, w, H, L, mode, True)
        assert rel_err(got, want) < 1e-10


# ------------------------------------------------------ conv / pool loops
@pytest.mark.parametrize("cfg", [
    dict(N=2, C=4, H=7, W=6, Cout=6, kH=3, kW=2, sx=1, sy=2, px=1, py=0, dx=1, dy=1, groups=2),
    dict(N=1, C=3, H=9, W=8, Cout=4, kH=3, kW=3, sx=2, sy=1, px=2, py=1, dx=2, dy=1, groups=1),
])
def test_conv_oracle_matches_loops(cfg):
    c = cfg
    x = randn(c["N"], c["C"], c["H"], c["W"], seed=1, dtype=torch.float64)
    w = randn(c["Cout"], c["C"] // c["groups"], c["kH"], c["kW"], seed=2, dtype=torch.float64)
    b = randn(c["Cout"], seed=3, dtype=torch.float64)
    args = (c["sx"], c["sy"], c["px"], c["py"], c["dx"], c["dy"], c["groups"])
    want = R.conv2d_naive(x.numpy(), w.numpy(), b.numpy(), *args)
    got = R.conv2d(x, w, b, *args)
    assert tuple(got.shape) == want.shape
    assert rel_err(got, want) < 1e-12


def test_conv_backward_oracle_is_the_jacobian():
    """Finite differences as in AutogradTestUtils.h:33-70 (central, +-1e-4) on a small conv."""
    x = randn(1, 2, 5, 4, seed=5, dtype=torch.float64)
    w = randn(3, 2, 3, 2, seed=6, dtype=torch.float64)
    args = (1, 2, 1, 1, 1, 1, 1)
    y = R.conv2d(x, w, None, *args)
    gy = randn(*y.shape, seed=7, dtype=torch.float64)
    gx = R.conv2d_backward_data(gy, x.shape, w, *args)
    gw, gb = R.conv2d_backward_filter_bias(gy, x, w.shape, True, *args)
    eps = 1e-4
    fd = torch.zeros_like(x)
    for i in range(x.numel()):
        xp, xm = x.clone().reshape(-1), x.clone().reshape(-1)
        xp[i] += eps
        xm[i] -= eps
        fd.reshape(-1)[i] = ((R.conv2d(xp.reshape(x.shape), w, None, *args) -
                              R.conv2d(xm.reshape(x.shape), w, None, *args)) * gy).sum() / (2 * eps)
    assert rel_err(gx, fd) < 1e-6
    fdw = torch.zeros_like(w)
    for i in range(w.numel()):
        wp, wm = w.clone().reshape(-1), w.clone().reshape(-1)
        wp[i] += eps
        wm[i] -= eps
        fdw.reshape(-1)[i] = ((R.conv2d(x, wp.reshape(w.shape), None, *args) -
                               R.conv2d(x, wm.reshape(w.shape), None, *args)) * gy).sum() / (2 * eps)
    assert rel_err(gw, fdw) < 1e-6
    assert rel_err(gb, gy.sum(dim=(0, 2, 3))) < 1e-12


@pytest.mark.parametrize("mode", [R.POOL_MAX, R.POOL_AVG_INCLUDE_PAD, R.POOL_AVG_EXCLUDE_PAD])
@pytest.mark.parametrize("geo", [(2, 2, 2, 2, 0, 0), (3, 3, 2, 2, 1, 1), (3, 2, 1, 2, 1, 0)])
def test_pool_oracle_matches_loops(mode, geo):
    wx, wy, sx, sy, px, py = geo
    x = randn(2, 3, 9, 8, seed=11, dtype=torch.float64)
    want, _ = R.pool2d_naive(x.numpy(), wx, wy, sx, sy, px, py, mode)
    got = R.pool2d(x, wx, wy, sx, sy, px, py, mode)
    assert tuple(got.shape) == want.shape
    assert rel_err(got, want) < 1e-12


def test_max_pool_ties_go_to_first_in_scan_order():
    """All-equal windows (the post-ReLU case): the whole gradient lands on the first in-bounds
    element, y outer / x inner.  No reference test pins this; the stand-in's rule is adopted."""
    x = torch.zeros(1, 1, 4, 4, dtype=torch.float64)
    gy = torch.ones(1, 1, 2, 2, dtype=torch.float64)
    gx = R.pool2d_backward(gy, x, 2, 2, 2, 2, 0, 0, R.POOL_MAX)
    want = torch.zeros_like(x)
    want[0, 0, 0::2, 0::2] = 1
    assert torch.equal(gx, want)
    _, arg = R.pool2d_naive(x.numpy(), 2, 2, 2, 2, 0, 0, R.POOL_MAX)
    assert (arg == 0).all()
    # 3x3 stride 2 pad 1: window (0,0) starts out of bounds, first in-bounds element is (0,0)
    gy3 = torch.ones(1, 1, 2, 2, dtype=torch.float64)
    gx3 = R.pool2d_backward(gy3, x, 3, 3, 2, 2, 1, 1, R.POOL_MAX)
    assert gx3[0, 0, 0, 0] == 1 and gx3[0, 0, 0, 1] == 1 and gx3[0, 0, 1, 0] == 1 and gx3[0, 0, 1, 1] == 1


# ------------------------------------------------------------- batchnorm
def test_batchnorm_geometry_rule():
    # spatial: fl [W,H,C,N] axes {2}
    assert R.batchnorm_geometry((5, 6, 7, 8), [2]) == (8, 7, 30)
    # per-activation: axes {0,1,2}
    assert R.batchnorm_geometry((5, 6, 7, 8), [0, 1, 2]) == (8, 210, 1)
    # LayerNorm as the reference maps it (nn/modules/LayerNorm.cpp:88-97): fl [C,T,B], normalise
    # axis 0 -> batchnorm over axes {1,2}
    assert R.batchnorm_geometry((768, 512, 8), [1, 2]) == (1, 4096, 768)
    with pytest.raises(ValueError):
        R.batchnorm_geometry((5, 6, 7, 8), [0, 2])
    with pytest.raises(ValueError):
        R.batchnorm_geometry((5, 6, 7), [3])


def test_batchnorm_matches_torch_and_layernorm():
    x = randn(4, 5, 3, 6, seed=21, dtype=torch.float64)  # fl [6,3,5,4]
    g = randn(5, seed=22, dtype=torch.float64)
    b = randn(5, seed=23, dtype=torch.float64)
    y, mean, invstd, rm, rv = R.batchnorm(x, g, b, torch.zeros(5, dtype=torch.float64),
                                          torch.ones(5, dtype=torch.float64), [2], True, 0.1, 1e-5)
    trm, trv = torch.zeros(5, dtype=torch.float64), torch.ones(5, dtype=torch.float64)
    want = F.batch_norm(x, trm, trv, g, b, True, 0.1, 1e-5)
    assert rel_err(y, want) < 1e-12
    assert rel_err(rm, trm) < 1e-12 and rel_err(rv, trv) < 1e-12
    # backward against autograd
    xr = x.clone().requires_grad_(True)
    gr = g.clone().requires_grad_(True)
    br = b.clone().requires_grad_(True)
    out = F.batch_norm(xr, None, None, gr, br, True, 0.0, 1e-5)
    gy = randn(*x.shape, seed=24, dtype=torch.float64)
    wx, wg, wb = torch.autograd.grad(out, (xr, gr, br), gy)
    dx, dg, db = R.batchnorm_backward(gy, x, g, [2], 1e-5)
    assert rel_err(dx, wx) < 1e-10 and rel_err(dg, wg) < 1e-10 and rel_err(db, wb) < 1e-10
    # layer norm over fl axis 0 of fl [C,T,B] == batchnorm over axes {1,2}
    z = randn(3, 7, 16, seed=25, dtype=torch.float64)  # torch (B,T,C)
    yl, *_ = R.batchnorm(z, None, None, None, None, [1, 2], True, 0.0, 1e-5)
    assert rel_err(yl, F.layer_norm(z, (16,), eps=1e-5)) < 1e-12


# ---------------------------------------------------- gradFunc restatements
def test_eltwise_and_loss_oracles_match_autograd():
    x = randn(5, 7, seed=31, dtype=torch.float64)
    gy = randn(5, 7, seed=32, dtype=torch.float64)
    xr = x.clone().requires_grad_(True)
    (want,) = torch.autograd.grad(F.gelu(xr, approximate="tanh"), xr, gy)
    assert rel_err(R.gelu_backward(x, gy), want) < 1e-7  # constants 0.7978845608 vs sqrt(2/pi)
    assert rel_err(R.tanh_backward(torch.tanh(x), gy), gy * (1 - torch.tanh(x) ** 2)) < 1e-12
    assert rel_err(R.log_softmax(x), F.log_softmax(x, -1)) < 1e-12
    xr = x.clone().requires_grad_(True)
    (want,) = torch.autograd.grad(F.log_softmax(xr, -1), xr, gy)
    assert rel_err(R.log_softmax_backward(F.log_softmax(x, -1), gy), want) < 1e-12
    t = torch.tensor([0, 3, -1, 6, 2], dtype=torch.int32)
    lp = F.log_softmax(x, -1)
    loss, denom = R.categorical_cross_entropy(lp, t, R.REDUCE_MEAN, -1)
    assert denom == 4
    want = F.nll_loss(lp, t.long(), ignore_index=-1)
    assert rel_err(loss, want.reshape(1)) < 1e-12
    lpr = lp.clone().requires_grad_(True)
    (wg,) = torch.autograd.grad(F.nll_loss(lpr, t.long(), ignore_index=-1), lpr)
    got = R.categorical_cross_entropy_backward(torch.ones(1, dtype=torch.float64), lp.shape, t,
                                               R.REDUCE_MEAN, -1, torch.float64)
    assert rel_err(got, wg) < 1e-12
    with pytest.raises(ValueError):
        R.categorical_cross_entropy(lp, torch.tensor([0, 1, 2, 3, 7]), R.REDUCE_MEAN, -1)


def test_linear_oracle():
    x = randn(3, 4, 6, seed=41, dtype=torch.float64)
    w = randn(6, 5, seed=42, dtype=torch.float64)  # fl [O=5, I=6]
    b = randn(5, seed=43, dtype=torch.float64)
    y = R.linear(x, w, b)
    assert rel_err(y, F.linear(x, w.t(), b)) < 1e-12
    gy = randn(*y.shape, seed=44, dtype=torch.float64)
    xr, wr, br = (t.clone().requires_grad_(True) for t in (x, w, b))
    wx, ww, wb = torch.autograd.grad(F.linear(xr, wr.t(), br), (xr, wr, br), gy)
    gx, gw, gb = R.linear_backward(x, w, gy, True)
    assert rel_err(gx, wx) < 1e-12 and rel_err(gw, ww) < 1e-12 and rel_err(gb, wb) < 1e-12


def test_sgd_rule_matches_the_torch_optimizer():
    """fl::SGDOptimizer's update (weight decay added to the gradient, momentum buffer without
    dampening, optional Nesterov) is torch.optim.SGD's; three steps must agree."""
    import torch
    from oracle import flref as R
    for nesterov in (False, True):
        g = torch.Generator().manual_seed(3)
        p = torch.randn(257, generator=g, dtype=torch.float64)
        tp = p.clone().requires_grad_(True)
        opt = torch.optim.SGD([tp], lr=0.1, momentum=0.9, weight_decay=0.1, nesterov=nesterov)
        v = torch.zeros_like(p)
        for _ in range(3):
            grad = torch.randn(257, generator=g, dtype=torch.float64)
            tp.grad = grad.clone()
            opt.step()
            p, v = R.sgd_step(p, grad, v, 0.1, 0.9, 0.1, nesterov)
        assert torch.allclose(p, tp.detach(), rtol=0, atol=1e-12)
