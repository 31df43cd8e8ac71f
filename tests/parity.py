"""Shared helpers of the parity tests: the error metric and seeded inputs."""
import numpy as np
import torch

# Bars from the build's north star: strict fp32 gradients within 1e-4; the TF32
# tensor-core mode has a looser, stated bound (10-bit mantissa inputs).
STRICT_TOL = 1e-4
TF32_TOL = 5e-3


REL_FLOOR = 1e-2
TIGHT_FLOOR = 1e-3


def rel_err(got, want, floor: float = REL_FLOOR) -> float:
    """max_i |got_i - want_i| / max(|want_i|, floor * max|want|): element-wise relative
    error with a floor at a fraction of the tensor's largest magnitude, so that entries that
    are tiny through cancellation are measured against the tensor's scale (an fp32 sum of K
    products carries an absolute error of order eps * sqrt(K) * scale whatever its own size)."""
    g = torch.as_tensor(got).detach().double().cpu().reshape(-1)
    w = torch.as_tensor(want).detach().double().cpu().reshape(-1)
    assert g.shape == w.shape, (g.shape, w.shape)
    if w.numel() == 0:
        return 0.0
    if not bool(torch.isfinite(g).all()):
        return float("inf")
    scale = float(w.abs().max())
    if scale == 0.0:
        return float(g.abs().max())
    den = torch.clamp(w.abs(), min=floor * scale)
    return float(((g - w).abs() / den).max())


WORST = {}  # what -> largest error seen at the tight floor (printed by conftest at session end)


def assert_close(got, want, tol, what=""):
    """Two bars: the element-wise relative error with the floor at 1 % of the tensor's largest
    magnitude must be within `tol`, and with the floor at 0.1 % within 10 * tol (an absolute
    error of tol * 1e-2 * scale is allowed on the smallest entries in both)."""
    e = rel_err(got, want)
    assert e <= tol, f"{what}: relative error {e:.3e} > {tol:.1e}"
    e2 = rel_err(got, want, TIGHT_FLOOR)
    WORST[what] = max(WORST.get(what, 0.0), e2)
    assert e2 <= 10 * tol, f"{what}: relative error at the 0.1 % floor {e2:.3e} > {10 * tol:.1e}"


def randn(*shape, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float64).to(dtype)


def randint(lo, hi, *shape, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi, shape, generator=g, dtype=torch.int32)


# TF32 mode: operands are read with a 10-bit mantissa, so single products carry ~1e-3
# relative error and entries that are small through cancellation cannot be matched
# element-wise; the bound is on the error relative to the tensor's largest magnitude.
TF32_SCALED_TOL = 2e-3


def scaled_err(got, want) -> float:
    """max_i |got_i - want_i| / max_i |want_i|."""
    g = torch.as_tensor(got).detach().double().cpu().reshape(-1)
    w = torch.as_tensor(want).detach().double().cpu().reshape(-1)
    assert g.shape == w.shape, (g.shape, w.shape)
    if w.numel() == 0:
        return 0.0
    if not bool(torch.isfinite(g).all()):
        return float("inf")
    scale = float(w.abs().max()) or 1.0
    return float((g - w).abs().max()) / scale


def assert_close_scaled(got, want, tol, what=""):
    e = scaled_err(got, want)
    assert e <= tol, f"{what}: error relative to the tensor scale {e:.3e} > {tol:.1e}"
