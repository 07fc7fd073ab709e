"""Multi-scale deformable 3D attention layer around the operator (the operator's usual caller).

The reference repository ships only the operator; its callers (MaskDINO-style encoder/decoder
layers) live elsewhere and build the packed input with separate divide / add / concatenate kernels.
``MSDeformAttn3D`` is that layer with the packing done in one fused kernel:

    value   = value_proj(input_flatten)                       [B, N, G, D]
    offsets = sampling_offsets(query)                          [B, Q, G, L, K, 3]   (x, y, z in cells)
    logits  = attention_weights(query)                         [B, Q, G, L, K]      (soft-max inside the operator)
    packed  = pack(reference_points + offsets / (W,H,D)_l, logits)
    out     = output_proj(FlashDeformAttnFunction(value, shapes, level_start_index, packed))

``reference_points`` are normalised ``(x, y, z)`` per level, ``[B, Q, L, 3]``.
"""
from __future__ import annotations

import math

import torch
from torch import nn
from torch.autograd import Function
from torch.autograd.function import once_differentiable

from .flash_deform_attn import FlashDeformAttnFunction


class PackSamplingFunction(Function):
    """``packed = pack(offsets, reference_points, logits, spatial_shapes)`` (fused CUDA kernel, fp32 output);
    gradients flow to ``offsets`` (divided by the level extent), ``reference_points`` (summed over heads
    and points) and ``logits`` (unchanged) through one fused CUDA kernel as well."""

    @staticmethod
    def forward(ctx, offsets, reference_points, logits, spatial_shapes):
        from . import capi

        dtype = offsets.dtype
        ctx.save_for_backward(spatial_shapes)
        ctx.meta = (offsets.shape, dtype, reference_points.dtype, logits.dtype)
        return capi.pack_sampling(offsets.contiguous(), reference_points.to(dtype).contiguous(),
                                  logits.to(dtype).contiguous(), spatial_shapes)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_packed):
        from . import capi

        (spatial_shapes,) = ctx.saved_tensors
        (B, Q, G, L, K, _), dtype, ref_dtype, logit_dtype = ctx.meta
        g_off, g_ref, g_logit = capi.pack_sampling_backward(grad_packed.float().contiguous(), spatial_shapes, B, Q, G, L, K, dtype)
        return g_off, g_ref.to(ref_dtype), g_logit.to(logit_dtype), None


class MSDeformAttn3D(nn.Module):
    def __init__(self, d_model: int = 256, n_levels: int = 3, n_heads: int = 8, n_points: int = 4, im2col_step: int = 64):
        super().__init__()
        if d_model % n_heads:
            raise ValueError("d_model must be divisible by n_heads")
        if n_points not in (4, 8) or not 1 <= n_levels <= 5:
            raise ValueError("the operator supports 1..5 levels and 4 or 8 points")
        self.d_model, self.n_levels, self.n_heads, self.n_points = d_model, n_levels, n_heads, n_points
        self.im2col_step = im2col_step
        self.sampling_offsets = nn.Linear(d_model, n_heads * n_levels * n_points * 3)
        self.attention_weights = nn.Linear(d_model, n_heads * n_levels * n_points)
        self.value_proj = nn.Linear(d_model, d_model)
        self.output_proj = nn.Linear(d_model, d_model)
        self._reset_parameters()

    def _reset_parameters(self):
        nn.init.constant_(self.sampling_offsets.weight, 0.0)
        # initial offsets: a ring of directions per head in the x-y plane tilted along z, growing with the point index
        theta = torch.arange(self.n_heads, dtype=torch.float32) * (2.0 * math.pi / self.n_heads)
        phi = torch.linspace(-0.5, 0.5, self.n_heads) * math.pi * 0.5
        grid = torch.stack([theta.cos() * phi.cos(), theta.sin() * phi.cos(), phi.sin()], -1)
        grid = grid / grid.abs().max(-1, keepdim=True)[0]
        grid = grid.view(self.n_heads, 1, 1, 3).repeat(1, self.n_levels, self.n_points, 1)
        for i in range(self.n_points):
            grid[:, :, i, :] *= i + 1
        with torch.no_grad():
            self.sampling_offsets.bias.copy_(grid.reshape(-1))
        nn.init.constant_(self.attention_weights.weight, 0.0)
        nn.init.constant_(self.attention_weights.bias, 0.0)
        nn.init.xavier_uniform_(self.value_proj.weight)
        nn.init.constant_(self.value_proj.bias, 0.0)
        nn.init.xavier_uniform_(self.output_proj.weight)
        nn.init.constant_(self.output_proj.bias, 0.0)

    def forward(self, query, reference_points, input_flatten, spatial_shapes, level_start_index, input_padding_mask=None):
        B, Q, _ = query.shape
        _, N, _ = input_flatten.shape
        G, L, K = self.n_heads, self.n_levels, self.n_points
        value = self.value_proj(input_flatten)
        if input_padding_mask is not None:
            value = value.masked_fill(input_padding_mask[..., None], 0.0)
        value = value.view(B, N, G, self.d_model // G).contiguous()
        offsets = self.sampling_offsets(query).view(B, Q, G, L, K, 3)
        logits = self.attention_weights(query).view(B, Q, G, L, K)
        packed = PackSamplingFunction.apply(offsets, reference_points, logits, spatial_shapes)
        out = FlashDeformAttnFunction.apply(value, spatial_shapes, level_start_index, packed, self.im2col_step, K, True)
        return self.output_proj(out)
