import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from flashlight_b200._reference import find_reference  # noqa: E402

# checkout of the flashlight project, where present (FLASHLIGHT_REFERENCE, or a directory
# `reference` beside the repository)
REFERENCE = find_reference()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    # GPU tests must never run (and silently pass) on a box without a GPU.
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def reference_root():
    if REFERENCE is None:
        pytest.skip("reference checkout not present on this machine")
    return REFERENCE


@pytest.fixture(autouse=True)
def _no_expired_device_waits(request):
    """Every wait inside the tensor-core kernels is bounded; one that runs out only raises a
    device flag.  After each GPU test the flag must be clear, so that a wait that expired can
    never pass as a slow success."""
    yield
    if "gpu" not in request.keywords:
        return
    import torch
    if not torch.cuda.is_available():
        return
    from flashlight_b200 import _lib
    assert _lib.lib.flb200_tc_poll_status(None) == 0, "a bounded device wait ran out in this test"


def pytest_sessionfinish(session, exitstatus):
    """Largest element-wise relative errors (floor at 0.1 % of the tensor scale) seen by
    tests/parity.assert_close in this session: the measured worst cases behind the bounds."""
    try:
        from tests.parity import WORST
    except Exception:  # pragma: no cover
        return
    if not WORST:
        return
    top = sorted(WORST.items(), key=lambda kv: -kv[1])[:12]
    print("\nworst relative errors at the 0.1 % floor: " +
          ", ".join(f"{k or '?'} {v:.2e}" for k, v in top))
