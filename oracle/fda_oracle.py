"""CPU oracle for Flash Deformable 3D Attention.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch, what the reference package computes on
its own CPU path for this operator.  It exists to check the CUDA kernels; it is
never imported by the product package (``ops3d_b200``).  Only the test-suite,
the smoke check and the CPU-baseline / reference arm of ``bench.py`` use it.

Reference being restated (paths inside cell-observatory/ops3d):

* ``ops3d/flash_deform_attn.py:139-165`` ``ms_deform_attn_core_pytorch_3d`` --
  per level ``F.grid_sample(mode="bilinear", padding_mode="zeros",
  align_corners=False)`` on ``2*loc-1`` grids, weighted by *already soft-maxed*
  attention weights and summed over levels x points.
* ``tests/test_flash_deform_attn.py:31-40,106-132`` -- how the fused operator's
  packed input ``[coords (L*K*3) | logits (L*K)]`` maps onto the oracle's
  ``sampling_locations`` / ``attention_weights`` (softmax over the flattened
  ``L*K`` logits happens inside the fused op, outside the oracle).

The arithmetic itself lives in PyTorch (``F.grid_sample`` 5-D "bilinear" and
``F.softmax``; torch is unpinned by the reference's requirements, 2.11 here).

Parity pin: ``tests/golden/*.npz`` were produced by importing the reference
package itself (``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks
this module and the C restatement (``oracle/fda_oracle.c``) against them.
"""
from __future__ import annotations

import math
from typing import Sequence, Tuple

import torch
import torch.nn.functional as F

__all__ = [
    "ms_deform_attn_core_pytorch_3d",
    "pack_loc_attn",
    "unpack_loc_attn",
    "fused_forward",
    "fused_forward_backward",
    "level_start_index_of",
]


def level_start_index_of(spatial_shapes: torch.Tensor) -> torch.Tensor:
    """``cat(0, cumsum(prod(shapes))[:-1])`` as in reference ``tests/conftest.py:42-44``."""
    sizes = spatial_shapes.prod(1)
    return torch.cat((sizes.new_zeros(1), sizes.cumsum(0)[:-1]))


def _shape_list(spatial_shapes) -> list:
    if isinstance(spatial_shapes, torch.Tensor):
        return [tuple(int(v) for v in row) for row in spatial_shapes.tolist()]
    return [tuple(int(v) for v in row) for row in spatial_shapes]


def ms_deform_attn_core_pytorch_3d(value, value_spatial_shapes, sampling_locations, attention_weights):
    """Multi-scale trilinear sampling + weighted sum; same contract as the reference's
    debug function of this name (``ops3d/flash_deform_attn.py:139-165``).

    value               [B, N, G, D]   N = sum_l D_l*H_l*W_l, level-major, (z, y, x) row-major
    value_spatial_shapes[L, 3]         (D_l, H_l, W_l)
    sampling_locations  [B, Q, G, L, K, 3]  normalised (x, y, z) in [0, 1] (last dim as grid_sample)
    attention_weights   [B, Q, G, L, K]     already normalised over L*K
    returns             [B, Q, G*D]

    Written level by level with an accumulated output instead of one stacked
    tensor, so peak memory is one level's samples rather than all levels'.
    """
    B, N, G, D = value.shape
    _, Q, _, L, K, _ = sampling_locations.shape
    shapes = _shape_list(value_spatial_shapes)
    assert len(shapes) == L
    out = value.new_zeros(B * G, D, Q)
    start = 0
    for lvl, (dz, hy, wx) in enumerate(shapes):
        cells = dz * hy * wx
        # [B, cells, G, D] -> [B*G, D, dz, hy, wx]
        vol = value[:, start:start + cells].permute(0, 2, 3, 1).reshape(B * G, D, dz, hy, wx)
        start += cells
        # [B, Q, G, K, 3] -> [B*G, 1, Q, K, 3]; grid_sample takes coordinates in [-1, 1]
        grid = (2 * sampling_locations[:, :, :, lvl] - 1).permute(0, 2, 1, 3, 4).reshape(B * G, 1, Q, K, 3)
        sampled = F.grid_sample(vol, grid, mode="bilinear", padding_mode="zeros", align_corners=False)
        w = attention_weights[:, :, :, lvl].permute(0, 2, 1, 3).reshape(B * G, 1, Q, K)
        out = out + (sampled[:, :, 0] * w).sum(-1)
    # [B*G, D, Q] -> [B, Q, G*D]
    return out.view(B, G * D, Q).transpose(1, 2).contiguous()


def pack_loc_attn(sampling_locations: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
    """Planar packing used by the fused operator: ``[B,Q,G, L*K*3 coords | L*K logits]``
    (reference ``tests/test_flash_deform_attn.py:31-37``)."""
    B, Q, G, L, K, _ = sampling_locations.shape
    return torch.cat(
        [sampling_locations.reshape(B, Q, G, L * K * 3), logits.reshape(B, Q, G, L * K)], dim=-1
    )


def unpack_loc_attn(packed: torch.Tensor, L: int, K: int) -> Tuple[torch.Tensor, torch.Tensor]:
    B, Q, G, last = packed.shape
    assert last == L * K * 4
    loc = packed[..., : L * K * 3].reshape(B, Q, G, L, K, 3)
    logits = packed[..., L * K * 3:].reshape(B, Q, G, L, K)
    return loc, logits


def _softmax_lk(logits: torch.Tensor) -> torch.Tensor:
    B, Q, G, L, K = logits.shape
    return F.softmax(logits.flatten(-2, -1), dim=-1).unflatten(-1, (L, K))


def fused_forward(value, spatial_shapes, packed, K: int, chunk: int = 8192) -> torch.Tensor:
    """What the fused operator returns, computed with the oracle in fp32:
    softmax over the packed logits, then ``ms_deform_attn_core_pytorch_3d``.
    Queries are independent, so the oracle is evaluated ``chunk`` queries at a
    time to bound memory at large Q."""
    shapes = _shape_list(spatial_shapes)
    L = len(shapes)
    value = value.float()
    packed = packed.float()
    Q = packed.shape[1]
    outs = []
    with torch.no_grad():
        for q0 in range(0, Q, chunk):
            loc, logits = unpack_loc_attn(packed[:, q0:q0 + chunk], L, K)
            outs.append(ms_deform_attn_core_pytorch_3d(value, shapes, loc, _softmax_lk(logits)))
    return torch.cat(outs, dim=1) if len(outs) > 1 else outs[0]


def fused_forward_backward(value, spatial_shapes, packed, grad_out, K: int, chunk: int = 8192):
    """Forward plus autograd backward through softmax + oracle (as reference
    ``tests/test_flash_deform_attn.py:118-136`` does), in fp32, query-chunked.
    Returns ``(out, grad_value, grad_packed)``; ``grad_packed`` has the planar
    packed layout (coordinate gradients first, raw-logit gradients last)."""
    shapes = _shape_list(spatial_shapes)
    L = len(shapes)
    value32 = value.detach().float()
    packed32 = packed.detach().float()
    grad_out = grad_out.detach().float()
    Q = packed32.shape[1]
    grad_value = torch.zeros_like(value32)
    outs, gpacked = [], []
    for q0 in range(0, Q, chunk):
        with torch.enable_grad():  # also usable from inside another autograd backward
            v = value32.clone().requires_grad_(True)
            pk = packed32[:, q0:q0 + chunk].clone().requires_grad_(True)
            loc, logits = unpack_loc_attn(pk, L, K)
            out = ms_deform_attn_core_pytorch_3d(v, shapes, loc, _softmax_lk(logits))
            out.backward(grad_out[:, q0:q0 + chunk].reshape_as(out))
        grad_value += v.grad
        gpacked.append(pk.grad)
        outs.append(out.detach())
    return torch.cat(outs, dim=1), grad_value, torch.cat(gpacked, dim=1)


# --------------------------------------------------------------------------
# Seeded synthetic inputs with the shapes and value distributions of the
# benchmark configurations (value ~ N(0,1); coordinates uniform in
# [-0.05, 1.05]^3 or clustered around per-query centres; logits ~ N(0,1)).
# --------------------------------------------------------------------------

def make_inputs(
    shapes: Sequence[Sequence[int]],
    B: int,
    Q: int,
    G: int,
    D: int,
    K: int,
    seed: int = 0,
    coords: str = "uniform",
    lo: float = -0.05,
    hi: float = 1.05,
    sigma: float = 0.05,
):
    """Returns fp32 CPU tensors ``(value, shapes_t, level_start_index, packed, grad_out)``."""
    gen = torch.Generator().manual_seed(seed)
    shapes_t = torch.tensor([list(s) for s in shapes], dtype=torch.long)
    L = shapes_t.shape[0]
    N = int(shapes_t.prod(1).sum())
    value = torch.randn(B, N, G, D, generator=gen)
    if coords == "uniform":
        loc = torch.rand(B, Q, G, L, K, 3, generator=gen) * (hi - lo) + lo
    elif coords == "clustered":
        centre = torch.rand(B, Q, 1, 1, 1, 3, generator=gen)
        loc = (centre + sigma * torch.randn(B, Q, G, L, K, 3, generator=gen)).clamp_(lo, hi)
    else:
        raise ValueError(coords)
    logits = torch.randn(B, Q, G, L, K, generator=gen)
    packed = pack_loc_attn(loc, logits)
    gen1 = torch.Generator().manual_seed(seed + 1)
    grad_out = torch.randn(B, Q, G * D, generator=gen1)
    return value, shapes_t, level_start_index_of(shapes_t), packed, grad_out
