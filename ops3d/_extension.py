"""``ops3d._C``: the compiled binding, or ``None`` when it is not built (same contract as the reference
loader, ``ops3d/_extension.py:13-16``).  One binary serves both package names, so the module object
of ``ops3d_b200._C`` is registered as ``ops3d._C`` as well (``import ops3d._C`` works)."""
import sys

from ops3d_b200._extension import _C, _C_IMPORT_ERROR  # noqa: F401

if _C is not None:
    sys.modules.setdefault(__package__ + "._C", _C)
