"""Writes tests/golden/reference_module_goldens.npz: the known-answer vectors of the flashlight
project's own module tests (flashlight/fl/test/nn/ModuleTest.cpp: EmbeddingFwd, LinearFwd,
LogSoftmaxFwd, RNNFwd, LSTMFwd, GRUFwd), parsed from a checkout of the project.  The GPU tests
read the fixture, so they also run where no checkout is present; tests/test_oracle_pins.py
re-parses the checkout where there is one and checks the fixture against it.

    python tests/golden/make_reference_goldens.py [path of the flashlight checkout]
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

from flashlight_b200._reference import find_reference  # noqa: E402
from tests.test_oracle_pins import _grab, _literals  # noqa: E402

OUT = Path(__file__).resolve().parent / "reference_module_goldens.npz"


def collect(reference_root: Path) -> dict:
    src = (reference_root / "flashlight/fl/test/nn/ModuleTest.cpp").read_text()
    out = {}
    for test, count in (("EmbeddingFwd", 3), ("LinearFwd", 5), ("LogSoftmaxFwd", 3)):
        for i, t in enumerate(_literals(src, test)[:count]):
            out[f"{test}_{i}"] = t.numpy()
    for test in ("RNNFwd", "LSTMFwd", "GRUFwd"):
        c = _grab(src, test)
        out[f"{test}_dims"] = np.array([c[k] for k in ("L", "H", "I", "B", "T", "n")], dtype=np.int64)
        out[f"{test}_scales"] = np.array([c["sin"], c["sw"]], dtype=np.float64)
        out[f"{test}_vals"] = c["vals"]
    return out


def main() -> None:
    root = Path(sys.argv[1]) if len(sys.argv) > 1 else find_reference()
    if root is None:
        raise SystemExit("no flashlight checkout found: pass its path")
    np.savez_compressed(OUT, **collect(Path(root)))
    print(OUT, OUT.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
