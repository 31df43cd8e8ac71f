"""Generates tests/golden/*.npz: small seeded input / expected-output vectors for the operators of
the backward hot path, computed by the CPU oracle (oracle/flref.py) in fp64.  The reference
itself is C++ and cannot be built or imported in this environment, so these vectors pin the
ORACLE (a later change to it shows up as a fixture mismatch in the CPU suite) and give the GPU
suite inputs that do not depend on any random-number generator on the box.

    python tests/golden/make_golden.py          # rewrites the fixtures
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import flref as R  # noqa: E402

OUT = Path(__file__).resolve().parent


def rnd(*shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float64)


def conv_case():
    x, w, b = rnd(2, 8, 9, 10, seed=1), rnd(6, 4, 3, 4, seed=2) * 0.2, rnd(6, seed=3)
    args = (1, 2, 2, 1, 1, 1, 2)  # sx, sy, px, py, dx, dy, groups
    y = R.conv2d(x, w, b, *args)
    gy = rnd(*y.shape, seed=4)
    gx = R.conv2d_backward_data(gy, x.shape, w, *args)
    gw, gb = R.conv2d_backward_filter_bias(gy, x, w.shape, True, *args)
    return dict(x=x, w=w, b=b, args=np.array(args), y=y, gy=gy, gx=gx, gw=gw, gb=gb)


def pool_case():
    x = torch.clamp_min(rnd(2, 3, 9, 8, seed=5) - 0.3, 0)  # post-ReLU: exact ties at zero
    geo = (3, 3, 2, 2, 1, 1)
    y = R.pool2d(x, *geo, R.POOL_MAX)
    gy = rnd(*y.shape, seed=6)
    gx = R.pool2d_backward(gy, x, *geo, R.POOL_MAX)
    _, arg = R.pool2d_naive(x.numpy(), *geo, R.POOL_MAX)
    ya = R.pool2d(x, *geo, R.POOL_AVG_EXCLUDE_PAD)
    gxa = R.pool2d_backward(gy, x, *geo, R.POOL_AVG_EXCLUDE_PAD)
    return dict(x=x, geo=np.array(geo), y=y, gy=gy, gx=gx, argmax=arg, y_avg=ya, gx_avg=gxa)


def bn_case():
    x = rnd(4, 6, 5, 7, seed=7) * 1.5 + 0.3
    g, b = rnd(6, seed=8).abs() + 0.5, rnd(6, seed=9)
    y, mean, invstd, rm, rv = R.batchnorm(x, g, b, torch.zeros(6, dtype=torch.float64),
                                          torch.ones(6, dtype=torch.float64), [2], True, 0.1, 1e-5)
    gy = rnd(*x.shape, seed=10)
    gx, gg, gb = R.batchnorm_backward(gy, x, g, [2], 1e-5)
    return dict(x=x, g=g, b=b, y=y, mean=mean, invstd=invstd, rm=rm, rv=rv, gy=gy, gx=gx, gg=gg,
                gb=gb)


def rnn_case():
    I, H, L, B, T = 3, 4, 2, 2, 5
    n = R.rnn_num_params(I, H, L, R.RNN_LSTM, True)
    w, x = rnd(n, seed=11) * 0.3, rnd(T, B, I, seed=12)
    hx, cx = rnd(L * 2, B, H, seed=13) * 0.5, rnd(L * 2, B, H, seed=14) * 0.5
    y, hy, cy = R.rnn(x, hx, cx, w, H, L, R.RNN_LSTM, True)
    gy = rnd(*y.shape, seed=15)
    dx, dhx, dcx, dw = R.rnn_backward(x, hx, cx, w, H, L, R.RNN_LSTM, True, gy, None, None)
    return dict(x=x, w=w, hx=hx, cx=cx, y=y, hy=hy, cy=cy, gy=gy, dx=dx, dhx=dhx, dcx=dcx, dw=dw,
                dims=np.array([I, H, L, B, T]))


def loss_case():
    x = rnd(7, 10, seed=16) * 2
    t = torch.tensor([0, 9, 3, -1, 5, 5, 2], dtype=torch.int32)
    lp = R.log_softmax(x)
    loss, denom = R.categorical_cross_entropy(lp, t, R.REDUCE_MEAN, -1)
    gl = torch.ones(1, dtype=torch.float64)
    glp = R.categorical_cross_entropy_backward(gl, lp.shape, t, R.REDUCE_MEAN, -1, torch.float64)
    gx = R.log_softmax_backward(lp, glp)
    return dict(x=x, t=t, lp=lp, loss=loss, denom=np.array(denom), gx=gx)


def main():
    for name, fn in (("conv", conv_case), ("pool", pool_case), ("batchnorm", bn_case),
                     ("rnn_lstm", rnn_case), ("loss", loss_case)):
        d = {k: (v.numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in fn().items()}
        np.savez_compressed(OUT / f"{name}.npz", **d)
        print(name, {k: v.shape for k, v in d.items()})


if __name__ == "__main__":
    main()
