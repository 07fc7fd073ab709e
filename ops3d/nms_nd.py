"""3D non-maximum suppression with the call surface of the reference module ``ops3d/nms_nd.py``."""
import torch

from ._extension import _C


def nms_nd(dets: torch.Tensor, iou_threshold: float):
    """``dets`` ``[N, 6 + 1]`` = (x1, y1, z1, x2, y2, z2, score).  Removes boxes whose IoU with a higher-scoring kept
    box exceeds ``iou_threshold``.  Returns ``(keep, dets)`` like the reference: ``keep`` = int64 indices of the kept
    boxes in decreasing score order."""
    if _C is None:
        raise RuntimeError("ops3d._C extension not built; nms_nd requires it.")
    boxes = dets[:, :-1]
    scores = dets[:, -1]
    return _C.nms_3d(boxes, scores, iou_threshold), dets
