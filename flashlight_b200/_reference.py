"""Where the flashlight checkout is, for the build-time checks and tests that read it.

The library never needs it at run time.  FLASHLIGHT_REFERENCE names the checkout; without
the variable a directory called `reference` beside this repository is used when it exists.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Optional

_REPO = Path(__file__).resolve().parent.parent
_MARKER = "flashlight/fl/autograd/tensor/AutogradExtension.h"


def find_reference() -> Optional[Path]:
    cands = []
    env = os.environ.get("FLASHLIGHT_REFERENCE")
    if env:
        cands.append(Path(env))
    cands.append(_REPO.parent / "reference")
    for c in cands:
        if (c / _MARKER).exists():
            return c
    return None
