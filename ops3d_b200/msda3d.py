"""Multi-scale deformable 3D attention layer around the operator (the operator's usual caller).

The reference repository ships only the operator; its callers (MaskDINO-style encoder/decoder
layers) live elsewhere and build the packed input with separate divide / add / concatenate kernels.
``MSDeformAttn3D`` is that layer with the packing folded into the query-projection GEMM (``project_and_pack``: one
GEMM writes the fp32 packed tensor in its final form) or, with ``fused_projection=False``, done by one fused kernel
after the two projections:

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


class _MatmulF32Out(Function):
    """``a @ b`` for 16-bit (or fp32) CUDA matrices with an fp32 result: the GEMM accumulates in fp32 anyway, this
    keeps the accumulator's precision in the output instead of rounding it to 16 bits."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        if a.dtype == torch.float32:
            return torch.mm(a, b)
        return torch.mm(a, b, out_dtype=torch.float32)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        a, b = ctx.saved_tensors
        g = grad.to(a.dtype)
        return torch.mm(g, b.t()), torch.mm(a.t(), g)


def project_and_pack(query, reference_points, w_offsets, b_offsets, w_logits, b_logits, spatial_shapes, n_heads, n_points):
    """The two query projections of the layer, the division by the level extents, the reference-point addition and
    the planar packing as ONE GEMM whose fp32 output is the operator's ``sampling_loc_attn`` -- nothing is written
    twice and no packing pass follows.

    How: the rows of both weight matrices are re-ordered into the packed column order (per head: ``L*K*3`` coordinate
    columns, then ``L*K`` logit columns) with the coordinate rows pre-divided by ``(W_l, H_l, D_l)``; the input gets
    ``1 + 9*L`` extra columns -- a one (the bias row) and the reference points split into three 16-bit terms
    ``hi + mid + lo`` (24 mantissa bits, exact in an fp32 accumulator) that a one-hot block of the weights adds to the
    right coordinate columns.  ``packed = [query | 1 | ref_hi | ref_mid | ref_lo] @ W_aug^T``.

    query ``[B, Q, C]``; reference_points ``[B, Q, L, 3]``; w_offsets ``[G*L*K*3, C]`` (rows ordered g, l, k, axis),
    w_logits ``[G*L*K, C]``; returns ``[B, Q, G, L*K*4]`` fp32.  Differentiable w.r.t. all tensor arguments.
    """
    B, Q, C = query.shape
    G, K = n_heads, n_points
    L = spatial_shapes.shape[0]
    LK = L * K
    dt = query.dtype
    extent = spatial_shapes.flip(-1).to(torch.float32)                                  # [L, 3] = (W, H, D)
    col_extent = extent[:, None, :].expand(L, K, 3).reshape(1, LK * 3, 1)               # per coordinate column of a head
    w_pack = torch.cat([w_offsets.float().view(G, LK * 3, C) / col_extent, w_logits.float().view(G, LK, C)], 1)
    b_pack = torch.cat([b_offsets.float().view(G, LK * 3) / col_extent[..., 0], b_logits.float().view(G, LK)], 1)
    # coordinate column (l, k, axis) takes reference value (l, axis): a one-hot block; logit columns take none
    sel = torch.eye(L * 3, device=query.device).view(L, 1, 3, L * 3).expand(L, K, 3, L * 3).reshape(LK * 3, L * 3)
    sel = torch.cat([sel, sel.new_zeros(LK, L * 3)], 0)[None].expand(G, 4 * LK, L * 3)
    extra = 1 + 9 * L
    pad = (-(C + extra)) % 8
    w_aug = torch.cat([w_pack, b_pack[..., None], sel, sel, sel, w_pack.new_zeros(G, 4 * LK, pad)], -1)
    w_aug = w_aug.reshape(G * 4 * LK, C + extra + pad).to(dt)
    ref = reference_points.reshape(B * Q, L * 3).float()
    hi = ref.to(dt)
    mid = (ref - hi.float()).to(dt)
    lo = (ref - hi.float() - mid.float()).to(dt)
    q2 = query.reshape(B * Q, C)
    aug = torch.cat([q2, q2.new_ones(B * Q, 1), hi, mid, lo, q2.new_zeros(B * Q, pad)], -1)
    packed = _MatmulF32Out.apply(aug, w_aug.t())
    return packed.view(B, Q, G, 4 * LK)


class MSDeformAttn3D(nn.Module):
    def __init__(self, d_model: int = 256, n_levels: int = 3, n_heads: int = 8, n_points: int = 4, im2col_step: int = 64,
                 fused_projection: bool = True):
        super().__init__()
        if d_model % n_heads:
            raise ValueError("d_model must be divisible by n_heads")
        if n_points not in (4, 8) or not 1 <= n_levels <= 5:
            raise ValueError("the operator supports 1..5 levels and 4 or 8 points")
        self.d_model, self.n_levels, self.n_heads, self.n_points = d_model, n_levels, n_heads, n_points
        self.im2col_step = im2col_step
        self.fused_projection = fused_projection  # packing inside the projection GEMM (CUDA); else projections + pack kernel
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
        if self.fused_projection and query.is_cuda:
            packed = project_and_pack(query, reference_points, self.sampling_offsets.weight, self.sampling_offsets.bias,
                                      self.attention_weights.weight, self.attention_weights.bias, spatial_shapes, G, K)
        else:
            offsets = self.sampling_offsets(query).view(B, Q, G, L, K, 3)
            logits = self.attention_weights(query).view(B, Q, G, L, K)
            packed = PackSamplingFunction.apply(offsets, reference_points, logits, spatial_shapes)
        out = FlashDeformAttnFunction.apply(value, spatial_shapes, level_start_index, packed, self.im2col_step, K, True)
        return self.output_proj(out)
