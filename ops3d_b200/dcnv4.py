"""DCNv4-3D (volumetric deformable convolution v4) as an autograd function over the B200 kernels.

The reference exposes this operator only through its binding (``_C.dcnv4_forward`` / ``_C.dcnv4_backward``,
reference ``csrc/dcnv4.h:7-61``); the same two functions, with the same positional arguments, are part of
``ops3d._C`` here.  ``DCNv4Function`` is the autograd wrapper a layer would put around them.

    value     [B, D, H, W, group*group_channels]
    p_offset  [B, D_out, H_out, W_out, padded]    per group: K*3 offsets (x, y, z per stencil point), then K masks,
                                                  at g*K*4; ``padded`` >= group*K*4 (a multiple of 8 in the reference)
    output    [B, D_out, H_out, W_out, group*group_channels]
"""
from __future__ import annotations

from torch.autograd import Function
from torch.autograd.function import once_differentiable

from ._extension import _C, _C_IMPORT_ERROR


def _ext():
    if _C is None:
        raise RuntimeError(f"ops3d_b200._C extension not built; DCNv4Function requires it: {_C_IMPORT_ERROR}")
    return _C


class DCNv4Function(Function):
    """``apply(value, p_offset, kernel, stride, pad, dilation, group, group_channels, offset_scale, im2col_step,
    remove_center, softmax)``; ``kernel`` .. ``dilation`` are (d, h, w) triples."""

    @staticmethod
    def forward(ctx, value, p_offset, kernel, stride, pad, dilation, group, group_channels, offset_scale, im2col_step=64,
                remove_center=0, softmax=False):
        ctx.cfg = (tuple(kernel), tuple(stride), tuple(pad), tuple(dilation), group, group_channels, float(offset_scale),
                   im2col_step, int(remove_center), bool(softmax))
        out = _ext().dcnv4_forward(value, p_offset, *kernel, *stride, *pad, *dilation, group, group_channels, float(offset_scale),
                                   im2col_step, int(remove_center), 8, 0, bool(softmax))
        ctx.save_for_backward(value, p_offset)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        value, p_offset = ctx.saved_tensors
        kernel, stride, pad, dilation, group, group_channels, offset_scale, im2col_step, remove_center, softmax = ctx.cfg
        grad_value, grad_offset = _ext().dcnv4_backward(value, p_offset, *kernel, *stride, *pad, *dilation, group, group_channels,
                                                        offset_scale, im2col_step, grad_output.contiguous(), remove_center, 8, 0,
                                                        softmax)
        return (grad_value, grad_offset) + (None,) * 10
