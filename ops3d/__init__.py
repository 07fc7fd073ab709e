"""``ops3d`` import surface for Flash Deformable 3D Attention on B200.

Code written against cell-observatory/ops3d keeps its imports:

    from ops3d import FlashDeformAttnFunction, _C
    from ops3d.flash_deform_attn import findspec, findspec_bwd
    import ops3d._C

(reference ``ops3d/__init__.py:3-6``, ``ops3d/_extension.py:13-16``).  The implementation is the
``ops3d_b200`` package: hand-written sm_100a kernels behind ``libfda_b200.so`` and the torch binding
that this package re-exports as ``ops3d._C``.  Beside deformable attention, the reference's other operators are here
under their own names too: ROI-Align 3D (``RoIAlign3DFunction``, ``RoIAlign``, ``roi_align_3d``), NMS 3D (``nms_nd``) and
the DCNv4-3D binding functions (``_C.dcnv4_forward`` / ``_C.dcnv4_backward``).  There is no CPU or PyTorch implementation
of any operator in this package (the reference's debug function ``ms_deform_attn_core_pytorch_3d`` is not exported).
"""
from ._extension import _C
from .flash_deform_attn import FlashDeformAttnFunction
from .nms_nd import nms_nd
from .roi_align_nd import RoIAlign, RoIAlign3DFunction, roi_align_3d

__all__ = ["FlashDeformAttnFunction", "RoIAlign3DFunction", "RoIAlign", "roi_align_3d", "nms_nd", "_C"]
