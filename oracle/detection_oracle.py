"""CPU oracles for ROI-Align 3D and NMS 3D.  TEST INFRASTRUCTURE ONLY (never imported by the product packages).

Plain-Python / numpy restatements of the reference's CUDA kernels (the reference has no CPU path for either):

* ``roi_align3d_forward`` / ``roi_align3d_backward``: ``csrc/cuda/roi_align_3d_cuda_kernel.cuh:31-107`` and ``:110-221``
  with the interpolation rules of ``csrc/cuda/interpolation_helpers_3d.h`` (samples more than one voxel outside the
  volume contribute nothing, coordinates clamp to ``[0, size-1]``, order 0 = nearest corner with ties to the lower one).
  Loops over every output element: for small cases only.
* ``nms3d``: IoU of ``csrc/cuda/nms_3d_cuda.cu:16-27`` and the greedy sweep of ``:133-157`` (score order, a box is
  dropped when its IoU with an earlier kept box exceeds the threshold).

Parity pin: PINNED to outputs of the reference's own CUDA kernels.  ``tests/golden/roi_align3d_*.npz`` and
``tests/golden/nms3d_*.npz`` were produced by ``tests/golden/make_golden_detection.py`` on a B200 from the reference
sources compiled unmodified (``baseline/build_ref_cuda.sh <checkout> --detection``); ``tests/test_oracle.py`` checks this
module against them, and restates the reference's own known-answer NMS tests (``tests/test_nms.py:17-50``).
"""
from __future__ import annotations

import math

import numpy as np


def _axis(v, size):
    if v <= 0:
        v = 0.0
    i0 = int(v)
    if i0 >= size - 1:
        i0 = i1 = size - 1
        v = float(i0)
    else:
        i1 = i0 + 1
    l = v - i0
    return i0, i1, l, 1.0 - l


def _sample(depth, height, width, z, y, x, order):
    """[(index tuple, weight)] of the up to eight corners, or [] when the sample is outside."""
    if y < -1.0 or y > height or x < -1.0 or x > width or z < -1.0 or z > depth:
        return []
    z0, z1, lz, hz = _axis(z, depth)
    y0, y1, ly, hy = _axis(y, height)
    x0, x1, lx, hx = _axis(x, width)
    if order == 0:
        lz, ly, lx = (1.0 if lz > 0.5 else 0.0), (1.0 if ly > 0.5 else 0.0), (1.0 if lx > 0.5 else 0.0)
        hz, hy, hx = 1.0 - lz, 1.0 - ly, 1.0 - lx
    return [((z0, y0, x0), hz * hy * hx), ((z0, y0, x1), hz * hy * lx), ((z0, y1, x0), hz * ly * hx), ((z0, y1, x1), hz * ly * lx),
            ((z1, y0, x0), lz * hy * hx), ((z1, y0, x1), lz * hy * lx), ((z1, y1, x0), lz * ly * hx), ((z1, y1, x1), lz * ly * lx)]


def _bins(roi, spatial_scale, sampling_ratio, pooled):
    pd, ph, pw = pooled
    b = int(roi[0])
    sw, sh, sd, ew, eh, ed = [np.float32(v) * np.float32(spatial_scale) for v in roi[1:7]]
    rw, rh, rd = max(ew - sw, np.float32(1)), max(eh - sh, np.float32(1)), max(ed - sd, np.float32(1))
    bd, bh, bw = rd / np.float32(pd), rh / np.float32(ph), rw / np.float32(pw)
    gd = sampling_ratio if sampling_ratio > 0 else int(math.ceil(rd / pd))
    gh = sampling_ratio if sampling_ratio > 0 else int(math.ceil(rh / ph))
    gw = sampling_ratio if sampling_ratio > 0 else int(math.ceil(rw / pw))
    return b, (sd, sh, sw), (bd, bh, bw), (gd, gh, gw), max(gd * gh * gw, 1)


def _points(start, bins, grid, idx):
    f32 = np.float32
    (sd, sh, sw), (bd, bh, bw), (gd, gh, gw), (id_, ih, iw) = start, bins, grid, idx
    for iz in range(gd):
        z = sd + f32(id_) * bd + f32(iz + .5) * bd / f32(gd)
        for iy in range(gh):
            y = sh + f32(ih) * bh + f32(iy + .5) * bh / f32(gh)
            for ix in range(gw):
                x = sw + f32(iw) * bw + f32(ix + .5) * bw / f32(gw)
                yield float(z), float(y), float(x)


def roi_align3d_forward(features, rois, output_size, spatial_scale, sampling_ratio, order):
    features = np.asarray(features, dtype=np.float64)
    rois = np.asarray(rois, dtype=np.float32)
    N, C, D, H, W = features.shape
    pd, ph, pw = output_size
    out = np.zeros((rois.shape[0], C, pd, ph, pw))
    for n, roi in enumerate(rois):
        b, start, bins, grid, count = _bins(roi, spatial_scale, sampling_ratio, output_size)
        for id_ in range(pd):
            for ih in range(ph):
                for iw in range(pw):
                    acc = np.zeros(C)
                    for z, y, x in _points(start, bins, grid, (id_, ih, iw)):
                        for (cz, cy, cx), w in _sample(D, H, W, z, y, x, order):
                            acc += w * features[b, :, cz, cy, cx]
                    out[n, :, id_, ih, iw] = acc / count
    return out


def roi_align3d_backward(grad_output, rois, feature_shape, spatial_scale, sampling_ratio, order):
    grad_output = np.asarray(grad_output, dtype=np.float64)
    rois = np.asarray(rois, dtype=np.float32)
    N, C, D, H, W = feature_shape
    n_rois, _, pd, ph, pw = grad_output.shape
    grad = np.zeros(feature_shape)
    for n, roi in enumerate(rois):
        b, start, bins, grid, count = _bins(roi, spatial_scale, sampling_ratio, (pd, ph, pw))
        for id_ in range(pd):
            for ih in range(ph):
                for iw in range(pw):
                    g = grad_output[n, :, id_, ih, iw] / count
                    for z, y, x in _points(start, bins, grid, (id_, ih, iw)):
                        for (cz, cy, cx), w in _sample(D, H, W, z, y, x, order):
                            grad[b, :, cz, cy, cx] += w * g
    return grad


def iou3d(a, b):
    a, b = np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32)
    w = max(min(a[3], b[3]) - max(a[0], b[0]), np.float32(0))
    h = max(min(a[4], b[4]) - max(a[1], b[1]), np.float32(0))
    d = max(min(a[5], b[5]) - max(a[2], b[2]), np.float32(0))
    inter = w * h * d
    sa = (a[3] - a[0]) * (a[4] - a[1]) * (a[5] - a[2])
    sb = (b[3] - b[0]) * (b[4] - b[1]) * (b[5] - b[2])
    with np.errstate(divide="ignore", invalid="ignore"):
        return inter / (sa + sb - inter)


def nms3d(boxes, scores, threshold):
    """Indices of the kept boxes in decreasing score order (ties: earlier box first)."""
    boxes, scores = np.asarray(boxes, dtype=np.float32), np.asarray(scores, dtype=np.float32)
    order = np.argsort(-scores, kind="stable")
    keep = []
    for i in order:
        if all(not (iou3d(boxes[j], boxes[i]) > threshold) for j in keep):
            keep.append(int(i))
    return keep
