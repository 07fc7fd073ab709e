"""Loads the compiled torch binding ``ops3d_b200._C`` (built in-tree by ``ops3d_b200.build``).

Mirrors the reference loader's contract (``ops3d/_extension.py:13-16``): ``_C`` is ``None`` when
the binding cannot be imported, and the operator then raises instead of computing anything else --
there is no CPU or PyTorch fallback in this package.  ``_C_IMPORT_ERROR`` keeps the reason.
"""
from __future__ import annotations

import torch  # noqa: F401  (libtorch must be loaded before the binding)

_C_IMPORT_ERROR = None
try:
    from . import _C  # type: ignore[attr-defined]
except ImportError as exc:  # not built, or built for another torch / python
    _C = None
    _C_IMPORT_ERROR = exc
