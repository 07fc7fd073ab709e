"""Query-sharded Flash Deformable 3D Attention over several GPUs (one process per GPU).

Every (batch, query) output row depends only on ``value[batch]`` and its own packed row, so the
queries of each batch element are split into contiguous, equal ranges, ``value`` is replicated,
and the forward needs no communication.  The backward has one exchange step: every rank scatters
into its own fp32 image of ``grad_value``; the images are summed with one all-reduce (NCCL over
NVLink on GPUs) and then cast once to the value dtype.  ``grad_sampling_loc_attn`` is row-local.

The reference has no multi-device path; this wrapper is the "queries sharded, value replicated,
grad_value all-reduced" arrangement of its single-device operator.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
from torch.autograd import Function
from torch.autograd.function import once_differentiable


def query_range(num_query: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous query range ``[begin, end)`` of ``rank``: the first ``num_query % world`` ranks get
    one extra query, so any query count works and ranges tile ``[0, num_query)`` exactly."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(num_query, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_queries(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Slice dimension 1 (queries) of ``[B, Q, ...]`` to this rank's range, contiguous."""
    b, e = query_range(t.shape[1], rank, world)
    return t[:, b:e].contiguous()


class CudaLocalOps:
    """Per-rank operator on raw device buffers through the C ABI (``libfda_b200.so``)."""

    def forward(self, value, shapes, lsi, packed, K, im2col_step):
        from . import capi
        return capi.forward(value, shapes, lsi, packed, K, im2col_step=im2col_step)

    def backward_accumulate(self, value, shapes, lsi, packed, grad_out, K, im2col_step):
        """Returns ``(accum_fp32 [B,N,G,D], grad_packed)``."""
        from . import capi
        accum = torch.empty(value.shape, dtype=torch.float32, device=value.device)
        grad_packed = capi.backward_accumulate(value, shapes, lsi, packed, grad_out, K, accum, im2col_step=im2col_step)
        return accum, grad_packed

    def cast(self, accum, dtype):
        from . import capi
        if dtype == torch.float32:
            return accum
        return capi.cast_grad_value(accum, torch.empty(accum.shape, dtype=dtype, device=accum.device))


class QueryShardedFlashDeformAttnFunction(Function):
    """``apply(value, shapes, level_start_index, packed_shard, im2col_step, K, group, local_ops)``

    ``packed_shard`` holds this rank's queries ``[B, Q_rank, G, L*K*4]``; returns ``[B, Q_rank, G*D]``.
    Backward returns the fully reduced ``grad_value`` (identical on every rank) and the local
    ``grad_packed_shard``.  ``local_ops`` is the per-rank operator (``CudaLocalOps()`` by default).
    """

    @staticmethod
    def forward(ctx, value, shapes, lsi, packed_shard, im2col_step, K, group=None, local_ops=None):
        ops = local_ops if local_ops is not None else CudaLocalOps()
        ctx.ops, ctx.group, ctx.K, ctx.im2col_step = ops, group, K, im2col_step
        L = shapes.shape[0]
        if packed_shard.shape[-1] != L * K * 4:
            raise ValueError(
                f"sampling_loc_attn last dimension ({packed_shard.shape[-1]}) does not match L={L}, K={K}")
        out = ops.forward(value, shapes, lsi, packed_shard, K, im2col_step)
        ctx.save_for_backward(value, shapes, lsi, packed_shard)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_out):
        value, shapes, lsi, packed_shard = ctx.saved_tensors
        accum, grad_packed = ctx.ops.backward_accumulate(
            value, shapes, lsi, packed_shard, grad_out.contiguous(), ctx.K, ctx.im2col_step)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(ctx.group) > 1:
            dist.all_reduce(accum, op=dist.ReduceOp.SUM, group=ctx.group)
        return ctx.ops.cast(accum, value.dtype), None, None, grad_packed, None, None, None, None


def sharded_flash_deform_attn(value, shapes, lsi, packed_shard, im2col_step, K, group=None,
                              local_ops: Optional[object] = None):
    return QueryShardedFlashDeformAttnFunction.apply(value, shapes, lsi, packed_shard, im2col_step, K, group, local_ops)
