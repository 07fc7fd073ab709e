"""Python entry points of Flash Deformable 3D Attention, same names and call signatures as the
reference module ``ops3d/flash_deform_attn.py``.

``FlashDeformAttnFunction.apply(value, spatial_shapes, level_start_index, sampling_loc_attn,
im2col_step, K=8, use_reg=True)`` -> ``[B, Lq, G*D]``; backward returns gradients for ``value``
and ``sampling_loc_attn`` (positions 0 and 3 of the 7 inputs), reference ``:68-136``.

    value              [B, N, G, D]      float32 / float16 / bfloat16, CUDA, contiguous
    spatial_shapes     [L, 3] int64      (D_l, H_l, W_l) per level, CUDA
    level_start_index  [L]    int64      CUDA
    sampling_loc_attn  [B, Lq, G, L*K*4] planar: L*K*3 normalised (x,y,z) coordinates, then L*K raw
                                          logits (soft-max happens inside the operator); dtype of
                                          ``value``, or float32 beside a 16-bit ``value``

``findspec`` / ``findspec_bwd`` are kept because callers import them (reference ``:26-62``; its
wrapper test calls ``_C`` directly with their results).  They return the same numbers as the
reference's but in O(sqrt(B*Q)) host time instead of a Python loop over every integer up to B*Q;
the kernels treat the results as hints and ignore them.
"""
from __future__ import annotations

import torch
from torch.autograd import Function
from torch.autograd.function import once_differentiable

from ._extension import _C, _C_IMPORT_ERROR


def _require_extension():
    if _C is None:
        raise RuntimeError(
            "ops3d_b200._C extension not built; FlashDeformAttnFunction requires it "
            f"(run `python -m ops3d_b200.build`): {_C_IMPORT_ERROR}"
        )
    return _C


def _largest_divisor(n: int, fits) -> int:
    """Largest divisor m of n with fits(m) true, 1 if none; ``fits`` must be monotone (true for small m)."""
    best = 1
    i = 1
    while i * i <= n:
        if n % i == 0:
            for m in (i, n // i):
                if m > best and fits(m):
                    best = m
        i += 1
    return best


def findspec(B, Q, G, C):
    """Forward launch hint ``(d_stride, threads_per_block)``: 8 channels per thread and the largest
    divisor m <= 64 of B*Q with m*G*C/8 <= 512 threads (reference ``:26-41``)."""
    d_stride = 8
    multiplier = _largest_divisor(B * Q, lambda m: m <= 64 and (m * G * C // d_stride) <= 512)
    return d_stride, multiplier * G * C // d_stride


def findspec_bwd(B, Q, G, C, max_tpb=256, max_mult=64):
    """Backward launch hint: smallest power-of-two ``d_stride`` dividing C with G*C/d_stride <= max_tpb,
    then the largest divisor m <= max_mult of B*Q that keeps the block within max_tpb (reference ``:44-62``)."""
    for d in (1, 2, 4, 8, 16, 32):
        if C % d == 0 and G * (C // d) <= max_tpb:
            d_stride = d
            break
    else:
        raise RuntimeError(f"Cannot fit G={G}, C={C} into {max_tpb} threads")
    lanes = G * (C // d_stride)
    mult = _largest_divisor(B * Q, lambda m: m <= max_mult and m * lanes <= max_tpb)
    return d_stride, mult * lanes


class FlashDeformAttnFunction(Function):
    @staticmethod
    def forward(ctx, value, value_spatial_shapes, value_level_start_index, sampling_loc_attn, im2col_step,
                K=8, use_reg=True):
        ext = _require_extension()
        ctx.K = K
        ctx.im2col_step = im2col_step

        L = value_spatial_shapes.shape[0]
        expected_last = L * K * 3 + L * K
        if sampling_loc_attn.shape[-1] != expected_last:
            raise ValueError(
                "sampling_loc_attn last dimension ({}) does not match value_spatial_shapes level count "
                "L={} and K={} (expected {})".format(sampling_loc_attn.shape[-1], L, K, expected_last)
            )

        B, Q, G, C = value.shape[0], sampling_loc_attn.shape[1], value.shape[2], value.shape[3]
        d_stride, blockthread = findspec(B, Q, G, C)
        ctx.d_stride_backward, ctx.blockthread_backward = findspec_bwd(B, Q, G, C)

        output = ext.flash_deform_attn_forward(
            value, value_spatial_shapes, value_level_start_index, sampling_loc_attn,
            ctx.im2col_step, K, d_stride, blockthread, use_reg,
        )
        ctx.save_for_backward(value, value_spatial_shapes, value_level_start_index, sampling_loc_attn)
        return output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        value, value_spatial_shapes, value_level_start_index, sampling_loc_attn = ctx.saved_tensors
        grad_value, grad_sampling_loc_attn = _require_extension().flash_deform_attn_backward(
            value, value_spatial_shapes, value_level_start_index, sampling_loc_attn,
            grad_output.contiguous(), ctx.im2col_step, ctx.K, ctx.d_stride_backward, ctx.blockthread_backward,
        )
        return grad_value, None, None, grad_sampling_loc_attn, None, None, None
