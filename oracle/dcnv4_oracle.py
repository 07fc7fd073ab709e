"""CPU oracle for DCNv4-3D.  TEST INFRASTRUCTURE ONLY (never imported by the product packages).

Restates in plain PyTorch what the reference's CUDA kernels compute (the reference has no Python or
CPU implementation of this operator):

* sampling positions, stencil order, offset-row layout, mask soft-max:
  ``csrc/cuda/dcnv4_im2col_cuda.cuh:49-256`` (``forward_kernel_dcn``), in particular ``:118`` (row layout
  ``offset + (b*Q + q)*padded + g*K*4``: K*3 offsets then K masks), ``:178-216`` (positions
  ``p0 - half_span*scale + (i*dilation + offset)*scale``, loops w outermost / d innermost, centre skipped
  with ``remove_center``) and ``:147-170`` (soft-max over the K masks);
* trilinear sampling with zero padding: ``csrc/cuda/common.h:52-138`` -- voxel coordinates, corners outside
  the volume contribute nothing; expressed here through ``F.grid_sample(align_corners=False)`` on the
  normalised position ``(2*(p + 0.5)/size - 1)``, which un-normalises back to ``p``;
* gradients (``csrc/cuda/dcnv4_col2im_cuda.cuh:48-245``): autograd through the same expression.

Parity pin: PINNED to outputs of the reference's own CUDA kernels.  ``tests/golden/dcnv4_*.npz`` were produced by
``tests/golden/make_golden_dcnv4.py`` on a B200 from the reference sources compiled unmodified
(``baseline/build_ref_cuda.sh <checkout> --dcnv4``); ``tests/test_oracle.py`` checks this module against them:
``out`` in all five cases, ``grad_value`` and ``grad_offset`` in four.  The fifth (soft-maxed masks, 16 channels per
group) would go through the reference's ``backward_kernel_dcn_warp_primitive``, whose soft-max backward block is
misplaced inside the outermost stencil loop (``csrc/cuda/dcnv4_col2im_cuda.cuh:520-533``): it writes garbage and stores
past the end of ``grad_offset``, so the generator does not run the reference's backward on it; the soft-max
backward is pinned instead by two cases with 48 channels per group, which take ``backward_kernel_dcn`` (``:225-237``).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def output_size(size_in, kernel, stride, pad, dilation):
    return tuple((s + 2 * p - (d * (k - 1) + 1)) // st + 1 for s, k, st, p, d in zip(size_in, kernel, stride, pad, dilation))


def stencil_points(kernel, remove_center):
    """Stencil indices (i_w, j_h, k_d) in the kernels' order."""
    kd, kh, kw = kernel
    pts = []
    for i in range(kw):
        for j in range(kh):
            for k in range(kd):
                if remove_center and (i, j, k) == (kw // 2, kh // 2, kd // 2):
                    continue
                pts.append((i, j, k))
    return pts


def sampling_positions(p_offset, size_in, kernel, stride, pad, dilation, group, offset_scale, remove_center):
    """Voxel coordinates ``[B, Q, G, K, 3]`` (w, h, d) of every sampling point, and the raw masks ``[B, Q, G, K]``."""
    B = p_offset.shape[0]
    G = group
    Do, Ho, Wo = output_size(size_in, kernel, stride, pad, dilation)
    pts = stencil_points(kernel, remove_center)
    K = len(pts)
    Q = Do * Ho * Wo
    rows = p_offset.reshape(B, Q, -1)[..., : G * K * 4].reshape(B, Q, G, K * 4)
    off = rows[..., : K * 3].reshape(B, Q, G, K, 3)          # (x, y, z) = (w, h, d)
    mask = rows[..., K * 3:]                                   # [B, Q, G, K]
    dev, dt = p_offset.device, p_offset.dtype
    zz, yy, xx = torch.meshgrid(torch.arange(Do, device=dev), torch.arange(Ho, device=dev), torch.arange(Wo, device=dev), indexing="ij")
    (kd, kh, kw), (sd, sh, sw), (pd, ph, pw), (dd, dh, dw) = kernel, stride, pad, dilation
    half = ((dw * (kw - 1)) >> 1, (dh * (kh - 1)) >> 1, (dd * (kd - 1)) >> 1)
    p0 = torch.stack([half[0] - pw + xx * sw, half[1] - ph + yy * sh, half[2] - pd + zz * sd], -1).reshape(1, Q, 1, 1, 3).to(dt)
    p0 = p0 - torch.tensor(half, device=dev, dtype=dt) * offset_scale
    st = torch.tensor([(i * dw, j * dh, k * dd) for i, j, k in pts], device=dev, dtype=dt).reshape(1, 1, 1, K, 3)
    return p0 + (st + off) * offset_scale, mask


def dcnv4_forward(value, p_offset, kernel, stride, pad, dilation, group, group_channels, offset_scale, remove_center, softmax):
    """value ``[B, Din, Hin, Win, G*Dg]``, p_offset ``[B, Do, Ho, Wo, padded]`` -> ``[B, Do, Ho, Wo, G*Dg]``.
    Triples are in (d, h, w) order.  Differentiable w.r.t. ``value`` and ``p_offset``."""
    B, Din, Hin, Win, C = value.shape
    G, Dg = group, group_channels
    Do, Ho, Wo = output_size((Din, Hin, Win), kernel, stride, pad, dilation)
    Q = Do * Ho * Wo
    pos, mask = sampling_positions(p_offset, (Din, Hin, Win), kernel, stride, pad, dilation, G, offset_scale, remove_center)
    K = pos.shape[3]
    if softmax:
        mask = F.softmax(mask, dim=-1)
    dev, dt = value.device, value.dtype
    size = torch.tensor([Win, Hin, Din], device=dev, dtype=dt)
    grid = 2 * (pos + 0.5) / size - 1                          # grid_sample un-normalises this back to pos
    vol = value.reshape(B, Din, Hin, Win, G, Dg).permute(0, 4, 5, 1, 2, 3).reshape(B * G, Dg, Din, Hin, Win)
    grid = grid.permute(0, 2, 1, 3, 4).reshape(B * G, 1, Q, K, 3)
    sampled = F.grid_sample(vol, grid, mode="bilinear", padding_mode="zeros", align_corners=False)  # [B*G, Dg, 1, Q, K]
    w = mask.permute(0, 2, 1, 3).reshape(B * G, 1, Q, K)
    out = (sampled[:, :, 0] * w).sum(-1)                        # [B*G, Dg, Q]
    return out.reshape(B, G, Dg, Q).permute(0, 3, 1, 2).reshape(B, Do, Ho, Wo, G * Dg)


def dcnv4_forward_backward(value, p_offset, grad_out, *args):
    """fp32 forward + autograd backward; returns ``(out, grad_value, grad_offset)`` (padding of the offset rows gets 0)."""
    v = value.detach().float().clone().requires_grad_(True)
    o = p_offset.detach().float().clone().requires_grad_(True)
    out = dcnv4_forward(v, o, *args)
    out.backward(grad_out.detach().float())
    return out.detach(), v.grad, o.grad


def make_inputs(B, size_in, G, Dg, kernel, stride, pad, dilation, remove_center, seed=0, offset_std=0.7):
    """Seeded fp32 CPU inputs: value ~ N(0,1), offsets ~ N(0, offset_std) voxels, masks ~ N(0,1); offset rows padded
    to a multiple of 8 elements (the reference's requirement, ``csrc/cuda/dcnv4_cuda.cu:40-42``) with junk in the padding."""
    gen = torch.Generator().manual_seed(seed)
    Do, Ho, Wo = output_size(size_in, kernel, stride, pad, dilation)
    K = kernel[0] * kernel[1] * kernel[2] - (1 if remove_center else 0)
    padded = -(-(G * K * 4) // 8) * 8
    value = torch.randn(B, *size_in, G * Dg, generator=gen)
    rows = torch.randn(B, Do, Ho, Wo, padded, generator=gen)
    body = rows[..., : G * K * 4].reshape(B, Do, Ho, Wo, G, K * 4)
    body[..., : K * 3] *= offset_std
    grad_out = torch.randn(B, Do, Ho, Wo, G * Dg, generator=torch.Generator().manual_seed(seed + 1))
    return value, rows, grad_out


def keep_positions_off_the_grid(p_offset, size_in, kernel, stride, pad, dilation, group, offset_scale, remove_center, margin=2e-3):
    """Returns ``p_offset`` (same dtype) with the offsets nudged wherever a sampling position would land within
    ``margin`` of an integer voxel coordinate.  Trilinear interpolation has a left and a right derivative there; with
    16-bit offsets exact hits are common (offset == stencil centre - stencil index), and which side an implementation
    takes is not part of the operator's contract."""
    out = p_offset.clone()
    dt = out.dtype
    G = group
    K = kernel[0] * kernel[1] * kernel[2] - (1 if remove_center else 0)
    B = out.shape[0]
    for _ in range(4):
        pos, _ = sampling_positions(out.float(), size_in, kernel, stride, pad, dilation, G, offset_scale, remove_center)
        near = (pos - pos.round()).abs() < margin
        if not bool(near.any()):
            break
        body = out.reshape(B, -1, out.shape[-1])[..., : G * K * 4].reshape(B, -1, G, K * 4)
        off = body[..., : K * 3].reshape(B, -1, G, K, 3)
        off += (near.to(dt) * 0.171).to(dt)   # views into `out`
    return out
