"""ROI-Align 3D with the call surface of the reference module ``ops3d/roi_align_nd.py`` (``RoIAlign3DFunction``,
``roi_align_3d``, ``RoIAlign``), over the B200 kernels behind ``ops3d._C.roi_align_3d_forward / _backward``.

features ``[N, C, D, H, W]``; rois ``[n, 7]`` = (batch index, x1, y1, z1, x2, y2, z2); output
``[n, C, out_d, out_h, out_w]``.  Gradients flow to ``features`` only (as in the reference); they are accumulated in
fp32 and returned in the dtype of ``features``.
"""
import torch
import torch.nn as nn
from torch.autograd import Function

from ._extension import _C


def _require():
    if _C is None:
        raise RuntimeError("ops3d._C extension not built; RoIAlign requires it.")
    return _C


class RoIAlign3DFunction(Function):
    @staticmethod
    def forward(ctx, features, rois, output_size, spatial_scale, sampling_ratio=0, order=1):
        if isinstance(output_size, int):
            out_d = out_h = out_w = output_size
        elif isinstance(output_size, tuple):
            assert len(output_size) == 3 and all(isinstance(v, int) for v in output_size)
            out_d, out_h, out_w = output_size
        else:
            raise TypeError('"output_size" must be an integer or tuple of integers')
        ctx.spatial_scale, ctx.sampling_ratio, ctx.order = spatial_scale, sampling_ratio, order
        ctx.save_for_backward(rois)
        ctx.feature_size, ctx.feature_dtype = features.size(), features.dtype
        output = features.new_empty(rois.size(0), features.size(1), out_d, out_h, out_w)
        _require().roi_align_3d_forward(features.contiguous(), rois.to(features.dtype).contiguous(), output, out_d, out_h, out_w,
                                        spatial_scale, sampling_ratio, order)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        (rois,) = ctx.saved_tensors
        grad_input = None
        if ctx.needs_input_grad[0]:
            out_d, out_h, out_w = grad_output.shape[2:]
            accum = torch.zeros(ctx.feature_size, dtype=torch.float32, device=grad_output.device)
            _require().roi_align_3d_backward(grad_output.contiguous(), rois.float().contiguous(), accum, out_d, out_h, out_w,
                                             ctx.spatial_scale, ctx.sampling_ratio, ctx.order)
            grad_input = accum.to(ctx.feature_dtype)
        return grad_input, None, None, None, None, None


roi_align_3d = RoIAlign3DFunction.apply


class RoIAlign(nn.Module):
    """RoI align pooling layer for 3D proposals: ``output_size`` = (d, h, w); rois scaled by ``spatial_scale``;
    ``sampling_ratio`` samples per bin and axis (<= 0: adaptive); ``order`` 0 = nearest, 1 = trilinear."""

    def __init__(self, output_size: tuple, spatial_scale: float, sampling_ratio: int = -1):
        super().__init__()
        assert iter(output_size)
        self.output_size = output_size
        self.spatial_scale = float(spatial_scale)
        self.sampling_ratio = int(sampling_ratio)
        self.dim = len(self.output_size)
        if self.dim != 3:
            raise Exception("Tried to init RoIAlign module with incorrect output size: {}".format(self.output_size))
        self.roi_align = roi_align_3d

    def forward(self, features, rois, order=1):
        assert order in [0, 1], "only support order = 0 (nearest) or 1 (linear)"
        sampling_ratio = 1 if order == 0 else self.sampling_ratio
        return self.roi_align(features, rois, self.output_size, self.spatial_scale, sampling_ratio, order)
