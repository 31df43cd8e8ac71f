"""Shared helpers of the parity tests: the error metric and seeded inputs."""
import numpy as np
import torch

# Bars from the build's north star: strict fp32 gradients within 1e-4; the TF32
# tensor-core mode has a looser, stated bound (10-bit mantissa inputs).
STRICT_TOL = 1e-4
TF32_TOL = 5e-3


def rel_err(got, want) -> float:
    """max_i |got_i - want_i| / max(|want_i|, 1e-2 * max|want|): element-wise relative
    error with a floor at 1% of the tensor's largest magnitude, so that entries that are
    tiny through cancellation are measured against the tensor's scale."""
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
    den = torch.clamp(w.abs(), min=1e-2 * scale)
    return float(((g - w).abs() / den).max())


def assert_close(got, want, tol, what=""):
    e = rel_err(got, want)
    assert e <= tol, f"{what}: relative error {e:.3e} > {tol:.1e}"


def randn(*shape, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float64).to(dtype)


def randint(lo, hi, *shape, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi, shape, generator=g, dtype=torch.int32)
