"""Query-sharded Flash Deformable 3D Attention over several GPUs (one process per GPU).

Every (batch, query) output row depends only on ``value[batch]`` and its own packed row, so the
queries of each batch element are split into contiguous, equal ranges, ``value`` is replicated,
and the forward needs no communication.  The backward has one exchange step: every rank scatters
into its own fp32 image of ``grad_value``; the images are summed with one all-reduce (NCCL over
NVLink on GPUs) and then cast once to the value dtype.  ``grad_sampling_loc_attn`` is row-local.
On GPUs the default is ``PeerReducer``: the sum and the cast are one kernel over NVLink peer memory,
overlapped per batch element with the scatter kernel of the next one (``FDA_SHARDED_REDUCE=nccl``
selects the plain all-reduce + cast instead).

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


def slab_exchange_ranges(shapes_host, value_shape, plan, parts):
    """Element ranges (inside one batch element's ``[N, G, D]`` image) that become final, in order, when the
    largest level is scattered in ``parts`` slab groups and the other levels afterwards.

    ``plan = (level, slabs, planes_per_slab)`` as returned by ``capi.bin_plan``.  Returns
    ``(parts, part_ranges, rest_ranges)`` or ``None`` when a range would not be a multiple of 8 elements.
    After slab group g the planes ``[first_slab*depth, min(end_slab*depth, D))`` of the level are final: a
    slab's points touch planes z0 and z0+1, so the plane just above a group still receives the next slab."""
    level, slabs, depth = plan
    dims = [tuple(int(v) for v in row) for row in torch.as_tensor(shapes_host).tolist()]
    cells = [d * h * w for d, h, w in dims]
    if sum(cells) != value_shape[1]:
        return None
    gd = value_shape[2] * value_shape[3]
    per_batch = value_shape[1] * gd
    start = sum(cells[:level])
    Dz, H, W = dims[level]
    parts = max(1, min(parts, slabs))
    part_ranges = []
    for g in range(parts):
        z0 = (slabs * g // parts) * depth
        z1 = min((slabs * (g + 1) // parts) * depth, Dz)
        part_ranges.append(((start + z0 * H * W) * gd, (start + z1 * H * W) * gd))
    rest = [(0, start * gd), ((start + cells[level]) * gd, per_batch)]
    rest_ranges = [(a, b) for a, b in rest if b > a]
    if any((a % 8) or (b % 8) for a, b in part_ranges + rest_ranges):
        return None
    return parts, part_ranges, rest_ranges


class PeerReducer:
    """Backward of one rank with the cross-GPU reduction fused into the cast and overlapped with compute.

    Holds two symmetric-memory buffers (every rank can address every rank's copy over NVLink): the
    fp32 image of ``grad_value`` and the reduced ``grad_value`` itself.  Per batch element the scatter
    kernel runs on the caller's stream; as soon as it is done a high-priority side stream runs
    barrier -> reduce+cast kernel (``fda_multimem_reduce_cast``: my slice summed inside NVSwitch and
    multicast back, when the buffers have a multicast binding; else ``fda_peer_reduce_cast``: pull my
    slice from all ranks, sum, cast, push to all ranks) -> barrier, while the caller's stream already scatters the next batch element.  Only the last
    batch element's exchange is exposed.  When ``spatial_shapes`` is given, each batch element is
    further split: the largest pyramid level first, the others second, so that the largest level's
    share of the image (most of the bytes) travels while the rest computes; and when that level is
    handled by the slab-binned kernels, it is launched in slab groups whose finished z-ranges are
    exchanged one by one (``FDA_SLAB_PARTS``; 4 groups from 4 ranks up, else 1).

    ``backward`` returns a ``grad_value`` that aliases the symmetric buffer: it is valid until the
    next ``backward`` call on this object (clone it to keep it longer).
    """

    def __init__(self, value_shape, dtype, device, group=None, spatial_shapes=None):
        import os

        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.shape, self.dtype, self.device = tuple(value_shape), dtype, device
        self.image = symm_mem.empty(*self.shape, dtype=torch.float32, device=device)
        self.out = symm_mem.empty(*self.shape, dtype=dtype, device=device)
        self.h_image = symm_mem.rendezvous(self.image, self.group)
        self.h_out = symm_mem.rendezvous(self.out, self.group)
        self.image_ptrs = [int(p) for p in self.h_image.buffer_ptrs]
        self.out_ptrs = [int(p) for p in self.h_out.buffer_ptrs]
        self.mc_image = int(getattr(self.h_image, "multicast_ptr", 0) or 0)
        self.mc_out = int(getattr(self.h_out, "multicast_ptr", 0) or 0)
        mode = os.environ.get("FDA_PEER_REDUCE_MODE", "auto")  # auto | multimem | p2p (pull) | push
        # Measured on 8 x B200: standing alone the in-switch reduction is the faster exchange (3.7 vs 4.4 ms
        # for a 1.22 GB image), but overlapped with the slab-binned backward it is the slower one (step
        # 10.0 vs 8.4 ms): plain peer loads disturb the L2-resident slabs less.  So peer loads by default.
        want_mc = mode == "multimem"
        self.use_multimem = want_mc and self.mc_image != 0 and self.mc_out != 0 and self.world > 1
        if mode == "multimem" and not self.use_multimem:
            raise RuntimeError("FDA_PEER_REDUCE_MODE=multimem but the buffers have no multicast binding")
        self.side = torch.cuda.Stream(device=device, priority=-1)
        self.per_batch = int(self.image[0].numel())
        self.use_push = mode == "push" and self.world > 1
        if self.use_push:
            # staging: one slot per source rank, each as long as the longest slice of the largest exchange
            self.slot = ((self.per_batch // 8 + self.world - 1) // self.world) * 8
            self.staging = symm_mem.empty(self.world * self.slot, dtype=torch.float32, device=device)
            self.h_staging = symm_mem.rendezvous(self.staging, self.group)
            self.staging_ptrs = [int(p) for p in self.h_staging.buffer_ptrs]
        self.scratch = None  # slab-binning scratch per batch element, allocated on first use
        # The image is handed back zero-filled after every backward (on the side stream, off the critical
        # path: it overlaps whatever the caller runs next), so the scatter kernels need not clear it first.
        self.image.zero_()
        self._image_clean = True
        if self.per_batch % 8:
            raise ValueError("elements per batch element must be a multiple of 8")
        # Level schedule: the largest level first (when it sits at either end of the pyramid), so that
        # its share of the image -- most of the bytes -- is exchanged while the other levels compute.
        self.passes = None
        self.shapes_host = None if spatial_shapes is None else torch.as_tensor(spatial_shapes).cpu().long().contiguous()
        self.slab_plan = None     # decided at the first backward (needs the query and point counts)
        self.slab_plan_key = None
        if spatial_shapes is not None and os.environ.get("FDA_LEVEL_SPLIT", "1") != "0":
            cells = [int(c) for c in torch.as_tensor(spatial_shapes).cpu().prod(1).tolist()]
            L = len(cells)
            gd = self.shape[2] * self.shape[3]
            if L > 1 and sum(cells) == self.shape[1]:
                big = max(range(L), key=lambda l: cells[l])
                if big == 0:
                    self.passes = [(0, 1), (1, L)]
                elif big == L - 1:
                    self.passes = [(L - 1, L), (0, L - 1)]
                if self.passes:
                    starts = [sum(cells[:l]) for l in range(L + 1)]
                    self.ranges = [(starts[a] * gd, starts[b] * gd) for a, b in self.passes]  # element ranges
                    if any((e0 % 8) or (e1 % 8) for e0, e1 in self.ranges):
                        self.passes = None

    def _check_level_order(self, lsi):
        """The level-wise and slab-wise exchange ranges assume levels stored back to back in index order
        (level_start_index = exclusive cumsum of the level sizes).  Checked once per level_start_index
        tensor; any other arrangement falls back to one exchange per batch element."""
        key = (lsi.data_ptr(), lsi._version)
        if getattr(self, "_lsi_checked", None) == key:
            return
        self._lsi_checked = key
        if self.shapes_host is None:
            return
        cells = self.shapes_host.prod(1)
        standard = torch.cat((cells.new_zeros(1), cells.cumsum(0)[:-1]))
        if not torch.equal(lsi.detach().cpu().long(), standard):
            self.shapes_host = None   # disables both split pipelines
            self.passes = None
            self.slab_plan, self.slab_plan_key = None, None

    def _plan_slabs(self, value, packed, K, scratch):
        """Host copy of the kernels' slab plan (same function, fda_backward_bin_plan) -> exchange ranges."""
        import os

        from . import capi

        key = (packed.shape[1], K)
        if self.slab_plan_key == key:
            return
        self.slab_plan_key, self.slab_plan = key, None
        if self.shapes_host is None or scratch is None or os.environ.get("FDA_LEVEL_SPLIT", "1") == "0":
            return
        plan = capi.bin_plan(self.shapes_host, (1,) + tuple(value.shape[1:]), packed.shape[1], K)
        if plan is None:
            return
        # Slab groups per level: more groups start the exchange earlier but add launches and barriers.  Measured:
        # on 2 GPUs (exchange short against compute) 1 / 2 / 4 groups give 27.7 / 27.9 / 28.1 ms per step, on
        # 8 GPUs 4 groups gave the shortest backward relative to the box's forward time.
        default_parts = 4 if self.world >= 4 else 1
        parts = max(1, int(os.environ.get("FDA_SLAB_PARTS", str(default_parts))))
        self.slab_plan = slab_exchange_ranges(self.shapes_host, self.shape, plan, parts)

    def _exchange(self, elem_begin, elem_count, out_elem):
        """barrier -> reduce+cast of image[elem_begin : elem_begin+elem_count) -> barrier, on the current stream."""
        from . import capi

        offs = (elem_begin * 4, elem_begin * out_elem)
        if self.use_push:
            img = self.image_ptrs[self.rank] + offs[0]
            capi.peer_push_partials(img, self.staging_ptrs, self.slot, self.rank, elem_count, self.device)
            self.h_image.barrier(channel=0)   # every rank's partials have landed in the owners' staging areas
            capi.peer_reduce_staged_cast(img, self.staging_ptrs[self.rank], self.slot,
                                         [p + offs[1] for p in self.out_ptrs], self.rank, elem_count, self.dtype, self.device)
            self.h_out.barrier(channel=0)     # every rank's results have landed; staging areas are free again
            return
        self.h_image.barrier(channel=0)   # every rank's part of the image is complete
        if self.use_multimem:             # in-switch sum (NVLS): 1/R of the bytes per GPU
            capi.multimem_reduce_cast(self.mc_image, self.mc_out, self.world, self.rank, elem_count, self.dtype,
                                      self.device, byte_offsets=offs)
        else:                             # plain peer loads / stores
            capi.peer_reduce_cast(self.image_ptrs, self.out_ptrs, self.rank, elem_count, self.dtype, self.device,
                                  byte_offsets=offs)
        self.h_out.barrier(channel=0)     # every rank's pushes have landed

    def backward(self, value, shapes, lsi, packed, grad_out, K, im2col_step=64, grad_packed=None):
        from . import capi

        if tuple(value.shape) != self.shape or value.dtype != self.dtype:
            raise ValueError("PeerReducer was built for another value shape / dtype")
        B = value.shape[0]
        if grad_packed is None:
            grad_packed = torch.empty_like(packed)
        main = torch.cuda.current_stream(self.device)
        self.side.wait_stream(main)  # earlier readers of self.out / self.image are done
        main.wait_stream(self.side)  # the zero-fill issued after the previous backward is done
        zero = 0 if self._image_clean else capi.BWD_ZERO_IMAGE
        self._image_clean = False
        out_elem = self.out.element_size()

        def hand_over(elem_begin, elem_count):
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(self.side):
                self.side.wait_event(done)
                self._exchange(elem_begin, elem_count, out_elem)

        from . import capi as _capi
        if self.scratch is None:
            # one scratch per batch element: in pass-major order the slab lists of every element stay alive
            nbytes = _capi.scratch_bytes(value[:1], packed[:1], K)
            self.scratch = [torch.empty(nbytes, dtype=torch.uint8, device=self.device) for _ in range(B)] if nbytes else False
        scratch_of = (lambda b: self.scratch[b]) if self.scratch is not False else (lambda b: None)
        scratch = scratch_of(0)
        self._check_level_order(lsi)
        self._plan_slabs(value, packed, K, scratch)

        def args_of(b):
            return (value[b:b + 1], shapes, lsi, packed[b:b + 1], grad_out[b:b + 1], K, self.image[b:b + 1],
                    grad_packed[b:b + 1])

        if self.slab_plan is not None:
            # Slab pipeline: the largest level is scattered slab group by slab group; the z-range a group has
            # finished is handed to the exchange while the next group (and later the other levels) compute.
            parts, part_ranges, rest_ranges = self.slab_plan
            for g in range(parts):
                for b in range(B):
                    capi.backward_binned_part(*args_of(b), g, parts, zero, scratch_of(b), im2col_step=im2col_step)
                    e0, e1 = part_ranges[g]
                    hand_over(b * self.per_batch + e0, e1 - e0)
            for b in range(B):
                capi.backward_accumulate_levels(*args_of(b), 0, shapes.shape[0],
                                                capi.BWD_RESUME | capi.BWD_FINALIZE | capi.BWD_BINNED_DONE,
                                                im2col_step=im2col_step, scratch=scratch_of(b))
                for e0, e1 in rest_ranges:
                    hand_over(b * self.per_batch + e0, e1 - e0)
        elif self.passes is None:
            for b in range(B):
                capi.backward_accumulate_levels(*args_of(b), 0, shapes.shape[0], zero | capi.BWD_FINALIZE,
                                                im2col_step=im2col_step, scratch=scratch_of(b))
                hand_over(b * self.per_batch, self.per_batch)
        else:
            # pass-major order: the big level of every batch element first, so that all of its exchanges
            # hide behind later launches and only the small remainder of the last element is exposed
            for n, ((lb, le), (e0, e1)) in enumerate(zip(self.passes, self.ranges)):
                last = n == len(self.passes) - 1
                flags = (zero if n == 0 else capi.BWD_RESUME) | (capi.BWD_FINALIZE if last else 0)
                for b in range(B):
                    capi.backward_accumulate_levels(*args_of(b), lb, le, flags, im2col_step=im2col_step, scratch=scratch_of(b))
                    hand_over(b * self.per_batch + e0, e1 - e0)
        finished = torch.cuda.Event()
        finished.record(self.side)
        main.wait_event(finished)       # all exchanges done: self.out is complete on every rank
        with torch.cuda.stream(self.side):
            self.image.zero_()          # every rank has finished reading this image (last barrier above)
        self._image_clean = True
        return self.out, grad_packed


class CudaLocalOps:
    """Per-rank operator on raw device buffers through the C ABI (``libfda_b200.so``)."""

    def __init__(self):
        self._reducers = {}

    def backward_reduced(self, value, shapes, lsi, packed, grad_out, K, im2col_step, group):
        """Backward with the cross-rank sum done by ``PeerReducer`` (NVLink peer memory).  Returns
        ``None`` when ``FDA_SHARDED_REDUCE=nccl`` asks for the plain all-reduce path instead."""
        import os

        if os.environ.get("FDA_SHARDED_REDUCE", "peer") != "peer":
            return None
        key = (tuple(value.shape), value.dtype, value.device, id(group))
        if key not in self._reducers:
            self._reducers[key] = PeerReducer(value.shape, value.dtype, value.device, group, spatial_shapes=shapes)
        gv, gp = self._reducers[key].backward(value, shapes, lsi, packed, grad_out, K, im2col_step)
        return gv.clone(), gp

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


_DEFAULT_OPS = None


def _default_cuda_ops():
    global _DEFAULT_OPS
    if _DEFAULT_OPS is None:
        _DEFAULT_OPS = CudaLocalOps()
    return _DEFAULT_OPS


class QueryShardedFlashDeformAttnFunction(Function):
    """``apply(value, shapes, level_start_index, packed_shard, im2col_step, K, group, local_ops)``

    ``packed_shard`` holds this rank's queries ``[B, Q_rank, G, L*K*4]``; returns ``[B, Q_rank, G*D]``.
    Backward returns the fully reduced ``grad_value`` (identical on every rank) and the local
    ``grad_packed_shard``.  ``local_ops`` is the per-rank operator (``CudaLocalOps()`` by default).
    """

    @staticmethod
    def forward(ctx, value, shapes, lsi, packed_shard, im2col_step, K, group=None, local_ops=None):
        ops = local_ops if local_ops is not None else _default_cuda_ops()
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
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(ctx.group) > 1
        if multi and hasattr(ctx.ops, "backward_reduced"):
            fused = ctx.ops.backward_reduced(value, shapes, lsi, packed_shard, grad_out.contiguous(), ctx.K,
                                             ctx.im2col_step, ctx.group)
            if fused is not None:
                return fused[0], None, None, fused[1], None, None, None, None
        accum, grad_packed = ctx.ops.backward_accumulate(
            value, shapes, lsi, packed_shard, grad_out.contiguous(), ctx.K, ctx.im2col_step)
        if multi:
            dist.all_reduce(accum, op=dist.ReduceOp.SUM, group=ctx.group)
        return ctx.ops.cast(accum, value.dtype), None, None, grad_packed, None, None, None, None


def sharded_flash_deform_attn(value, shapes, lsi, packed_shard, im2col_step, K, group=None,
                              local_ops: Optional[object] = None):
    return QueryShardedFlashDeformAttnFunction.apply(value, shapes, lsi, packed_shard, im2col_step, K, group, local_ops)
