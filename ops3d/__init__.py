"""``ops3d`` import surface for Flash Deformable 3D Attention on B200.

Code written against cell-observatory/ops3d keeps its imports:

    from ops3d import FlashDeformAttnFunction, _C
    from ops3d.flash_deform_attn import findspec, findspec_bwd
    import ops3d._C

(reference ``ops3d/__init__.py:3-6``, ``ops3d/_extension.py:13-16``).  The implementation is the
``ops3d_b200`` package: hand-written sm_100a kernels behind ``libfda_b200.so`` and the torch binding
that this package re-exports as ``ops3d._C``.  Only the deformable-attention entry points exist here;
the reference's other operators (ROI-Align 3D, NMS) are not part of this build, and there is no
CPU or PyTorch implementation of the operator in this package.
"""
from ._extension import _C
from .flash_deform_attn import FlashDeformAttnFunction

__all__ = ["FlashDeformAttnFunction", "_C"]
