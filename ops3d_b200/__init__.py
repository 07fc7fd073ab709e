"""ops3d_b200 -- Flash Deformable 3D Attention for NVIDIA B200 (sm_100a).

Drop-in for the ``ops3d.flash_deform_attn`` entry points of cell-observatory/ops3d: hand-written
CUDA kernels behind a C ABI (``include/fda_b200.h``, ``libfda_b200.so``), a thin torch binding
(``ops3d_b200._C``) and the autograd wrapper ``FlashDeformAttnFunction``.  CUDA only.
"""
from ._extension import _C
from .flash_deform_attn import FlashDeformAttnFunction, findspec, findspec_bwd

__all__ = ["FlashDeformAttnFunction", "findspec", "findspec_bwd", "_C"]
# The layer around the operator lives in ops3d_b200.msda3d (MSDeformAttn3D); imported on demand.
