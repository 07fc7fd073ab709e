"""Flash Deformable 3D Attention sharded over several GPUs (one process per GPU).

Every (batch, query) output row depends only on ``value[batch]`` and its own packed row, so the rows
are split over the ranks, ``value`` is replicated, and the forward needs no communication.  The
backward has one exchange step: ranks that worked on the same batch element each hold a partial fp32
image of ``grad_value[batch]``; the partial images are summed (over NVLink on GPUs) and cast once to
the value dtype, and every rank receives the whole ``grad_value``.  ``grad_sampling_loc_attn`` is row-local.

Partition (``partition``): the flattened ``(batch, query)`` rows are cut into ``world`` contiguous
ranges that stay batch-aligned whenever the counts allow it, so that a rank reads, zero-fills,
scatters into and exchanges the image of ONE batch element (or of whole batch elements):

* ``world`` divides ``B``: every rank owns ``B / world`` whole batch elements -- no sum at all, the
  exchange is a cast + broadcast of finished images;
* ``B`` divides ``world`` and ``world / B`` divides the number of heads: the ranks of a group split the HEADS of
  one batch element ("batch-heads").  A head's rows read and write only that head's channels of ``value`` /
  ``grad_value``, so the group needs no sum either -- every rank converts its finished slice of the image and
  stores it into every rank's ``grad_value`` -- and a rank sees every query, so the density of sampling points
  per cell that the cell-sorted backward lives on does not drop with the number of ranks;
* ``B`` divides ``world`` otherwise: the ``world / B`` ranks of a group split the queries of one batch element
  and sum only among themselves ("batch-groups"; ``FDA_PARTITION=rows`` prefers this over the head split);
* otherwise the queries of every batch element are split over all ranks (every rank touches every
  image; ``FDA_PARTITION=queries`` forces this arrangement).

On GPUs the default exchange is ``PeerReducer``: sum and cast are one kernel over NVLink peer memory,
pipelined with the scatter kernels (``FDA_SHARDED_REDUCE=nccl`` selects a plain all-reduce + cast).

The reference has no multi-device path; this wrapper is the "queries/batch sharded, value replicated,
grad_value all-reduced" arrangement of its single-device operator.
"""
from __future__ import annotations

import os
from typing import NamedTuple, Optional, Tuple

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


class Partition(NamedTuple):
    """This rank's share of the ``[B, Q]`` rows: batch elements ``[b_begin, b_end)``, queries
    ``[q_begin, q_end)`` of each of them, heads ``[h_begin, h_end)`` (``0, 0``: all heads), and the ranks that share
    those batch elements (``group``, in rank order; this rank is ``group[group_rank]``)."""
    b_begin: int
    b_end: int
    q_begin: int
    q_end: int
    group: Tuple[int, ...]
    group_rank: int
    kind: str  # "batch" (whole batch elements), "batch-heads" / "batch-groups" (one element per group), "queries"
    h_begin: int = 0
    h_end: int = 0

    @property
    def splits_heads(self) -> bool:
        return self.h_end > self.h_begin


def partition(num_batch: int, num_query: int, rank: int, world: int, mode: Optional[str] = None,
              num_heads: Optional[int] = None) -> Partition:
    """``mode`` (default: ``FDA_PARTITION``, else "auto"): "auto", "rows" (auto, but never split heads) or "queries".
    ``num_heads`` makes the head split available to "auto"."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    mode = mode or os.environ.get("FDA_PARTITION", "auto")
    if mode not in ("auto", "rows", "queries"):
        raise ValueError(f"FDA_PARTITION must be 'auto', 'rows' or 'queries', got {mode!r}")
    if mode != "queries" and world > 1 and num_batch % world == 0:
        per = num_batch // world
        return Partition(rank * per, (rank + 1) * per, 0, num_query, (rank,), 0, "batch")
    if mode != "queries" and world > 1 and world % num_batch == 0:
        size = world // num_batch
        b, sub = divmod(rank, size)
        group = tuple(range(b * size, (b + 1) * size))
        if mode == "auto" and num_heads and num_heads % size == 0:
            per = num_heads // size
            return Partition(b, b + 1, 0, num_query, group, sub, "batch-heads", sub * per, (sub + 1) * per)
        qb, qe = query_range(num_query, sub, size)
        return Partition(b, b + 1, qb, qe, group, sub, "batch-groups")
    qb, qe = query_range(num_query, rank, world)
    return Partition(0, num_batch, qb, qe, tuple(range(world)), rank, "queries")


def shard_rows(t: torch.Tensor, part: Partition, num_heads: Optional[int] = None) -> torch.Tensor:
    """This rank's rows of a full ``[B, Q, ...]`` tensor, contiguous: ``[b_end-b_begin, q_end-q_begin, ...]``.
    With a head split, dimension 2 of a 4-D tensor ``[B, Q, G, ...]`` is cut to the rank's heads, and a 3-D tensor
    ``[B, Q, G*D]`` is cut as ``[B, Q, G, D]`` (``num_heads`` = G required)."""
    rows = t[part.b_begin:part.b_end, part.q_begin:part.q_end]
    if part.splits_heads:
        if rows.dim() == 4:
            rows = rows[:, :, part.h_begin:part.h_end]
        elif rows.dim() == 3:
            if not num_heads or rows.shape[2] % num_heads:
                raise ValueError("shard_rows: a [B, Q, G*D] tensor under a head split needs num_heads")
            rows = rows.reshape(rows.shape[0], rows.shape[1], num_heads, -1)[:, :, part.h_begin:part.h_end]
            rows = rows.reshape(rows.shape[0], rows.shape[1], -1)
        else:
            raise ValueError("shard_rows: expected [B, Q, G, ...] or [B, Q, G*D] under a head split")
    return rows.contiguous()


def shard_value(value: torch.Tensor, part: Partition) -> torch.Tensor:
    """The part of ``value [B, N, G, D]`` this rank's rows read: its batch elements, and under a head split its heads
    (a compact copy)."""
    v = value[part.b_begin:part.b_end]
    return v[:, :, part.h_begin:part.h_end].contiguous() if part.splits_heads else v


def shard_queries(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Slice dimension 1 (queries) of ``[B, Q, ...]`` to the query range of ``rank`` (the "queries"
    partition), contiguous."""
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
    fp32 image of this rank's batch elements and the reduced ``grad_value`` ``[B, N, G, D]``.  As soon
    as a piece of an image is final on the caller's stream, a high-priority side stream runs
    barrier -> reduce+cast kernel -> barrier for that piece, while the caller's stream already computes
    the next one.  The kernel (``fda_group_reduce_cast``) pulls this rank's slice of the piece from
    the ranks of its group (those that hold partial sums of the same batch element), sums in fp32,
    converts once and stores the result into every rank's ``grad_value``; with the "queries" partition
    ``FDA_PEER_REDUCE_MODE=multimem|push`` select the NVSwitch-multicast and the posted-store variants.
    Pieces, when ``spatial_shapes`` is given: the largest pyramid level first (most of the bytes), the
    other levels second; and when that level is handled by the slab-binned kernels it is launched in
    slab groups whose finished z-ranges are exchanged one by one (``FDA_SLAB_PARTS``, default one group:
    the level as a whole).  Only the small remainder of the last batch element is exposed.

    All ranks must call ``backward`` with the same shapes: every rank issues the same sequence of
    barriers.  The schedule (slab plan, level passes) is agreed on across ranks with one small
    all-reduce whenever the problem changes; if ranks disagree, all fall back to one exchange per
    batch element.

    ``backward`` returns a ``grad_value`` that aliases the symmetric buffer: it is valid until the
    next ``backward`` call on this object (copy it to keep it longer).
    """

    def __init__(self, value_shape, dtype, device, group=None, spatial_shapes=None, part: Optional[Partition] = None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.shape, self.dtype, self.device = tuple(value_shape), dtype, device
        B = self.shape[0]
        self.part = part if part is not None else partition(B, 0, self.rank, self.world)
        self.nb = self.part.b_end - self.part.b_begin   # batch elements this rank works on (same on every rank)
        self.heads = self.part.splits_heads              # this rank's image is a finished slice: no sum, only a broadcast
        self.gr = (self.part.h_end - self.part.h_begin) if self.heads else self.shape[2]   # heads of this rank's image
        self.image = symm_mem.empty(self.nb, self.shape[1], self.gr, self.shape[3], dtype=torch.float32, device=device)
        self.out = symm_mem.empty(*self.shape, dtype=dtype, device=device)
        self.h_image = symm_mem.rendezvous(self.image, self.group)
        self.h_out = symm_mem.rendezvous(self.out, self.group)
        self.image_ptrs = [int(p) for p in self.h_image.buffer_ptrs]
        self.out_ptrs = [int(p) for p in self.h_out.buffer_ptrs]
        self.group_image_ptrs = [self.image_ptrs[r] for r in self.part.group]
        self.mc_image = int(getattr(self.h_image, "multicast_ptr", 0) or 0)
        self.mc_out = int(getattr(self.h_out, "multicast_ptr", 0) or 0)
        mode = os.environ.get("FDA_PEER_REDUCE_MODE", "auto")  # auto | multimem | p2p (pull) | push
        whole_job = len(self.part.group) == self.world and self.nb == B
        if mode in ("multimem", "push") and (not whole_job or self.heads):
            raise RuntimeError(f"FDA_PEER_REDUCE_MODE={mode} needs the 'queries' partition (FDA_PARTITION=queries)")
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
        # The image is handed back zero-filled after every backward (on the side stream, off the critical
        # path: it overlaps whatever the caller runs next), so the scatter kernels need not clear it first.
        self.image.zero_()
        self._image_clean = True
        if self.per_batch % 8:
            raise ValueError("elements per batch element must be a multiple of 8")
        self.shapes_host = None if spatial_shapes is None else torch.as_tensor(spatial_shapes).cpu().long().contiguous()
        self._schedule_key = None
        self._schedule = None
        self._scratch = None

    # ---- schedule --------------------------------------------------------------------------------------------
    def _level_passes(self, lsi):
        """Largest level first (when it sits at either end of the pyramid and the levels are stored back to
        back in index order): ``[(level_begin, level_end, elem_begin, elem_end), ...]`` or ``None``."""
        if self.shapes_host is None or os.environ.get("FDA_LEVEL_SPLIT", "1") == "0":
            return None
        cells_t = self.shapes_host.prod(1)
        standard = torch.cat((cells_t.new_zeros(1), cells_t.cumsum(0)[:-1]))
        if not torch.equal(lsi.detach().cpu().long(), standard):
            return None
        cells = [int(c) for c in cells_t.tolist()]
        L = len(cells)
        gd = self.gr * self.shape[3]
        if L < 2 or sum(cells) != self.shape[1]:
            return None
        big = max(range(L), key=lambda l: cells[l])
        if big == 0:
            levels = [(0, 1), (1, L)]
        elif big == L - 1:
            levels = [(L - 1, L), (0, L - 1)]
        else:
            return None
        starts = [sum(cells[:l]) for l in range(L + 1)]
        passes = [(a, b, starts[a] * gd, starts[b] * gd) for a, b in levels]
        if any((e0 % 8) or (e1 % 8) for _, _, e0, e1 in passes):
            return None
        return passes

    def _plan(self, value, lsi, packed, K):
        """Decides, once per problem, how the backward is cut into pieces -- and makes sure every rank decided
        the same (they all issue one barrier pair per piece)."""
        from . import capi

        key = (tuple(packed.shape), packed.dtype, K, lsi.data_ptr(), lsi._version)
        if key == self._schedule_key:
            return
        one = (1,) + tuple(value.shape[1:])   # `value` is this rank's part (shard_value): compact under a head split
        nbytes = capi.scratch_bytes(value[:1], packed[:1], K)
        passes = self._level_passes(lsi)
        slab = None
        # the cell-sorted backward (when the library chooses it for this rank's rows) works level range by level range,
        # not slab group by slab group
        sorted_path = capi.backward_path(value[:1], packed[:1], K) == 2
        if passes is not None and nbytes and not sorted_path:
            plan = capi.bin_plan(self.shapes_host, one, packed.shape[1], K)
            if plan is not None:
                # Slab groups per level: more groups start the exchange earlier but add launches and barriers.
                # Measured with the batch-aligned partition on 8 GPUs (4 ranks per batch element): 1 / 2 / 4 / 8
                # groups give 7.69 / 7.80 / 8.07 / 8.58 ms per step; on 2 GPUs 1 / 2 / 4 groups 27.7 / 27.9 / 28.1 ms.
                parts = max(1, int(os.environ.get("FDA_SLAB_PARTS", "1")))
                slab = slab_exchange_ranges(self.shapes_host, one, plan, parts)
        if slab is not None:
            schedule = ("slabs", slab)
        elif passes is not None:
            schedule = ("levels", passes)
        else:
            schedule = ("whole", None)
        # every rank must have arrived at the same pieces: compare a fingerprint across the group
        flat = [len(schedule[0]), packed.shape[0], K, int(nbytes > 0), int(sorted_path)]  # query counts may differ by one between ranks
        if schedule[0] == "slabs":
            flat += [slab[0]] + [v for r in slab[1] + slab[2] for v in r]
        elif schedule[0] == "levels":
            flat += [v for p in passes for v in p]
        flat = flat + [0] * (96 - len(flat)) if len(flat) <= 96 else flat[:95] + [hash(tuple(flat)) % (1 << 40)]
        t = torch.tensor(flat + [-v for v in flat], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        t = t.tolist()
        if any(a != -b for a, b in zip(t[:96], t[96:])):
            schedule = ("whole", None)  # ranks disagree: the one arrangement that needs no shared plan
            if t[1] != -t[97]:
                raise RuntimeError("PeerReducer.backward: ranks hold different numbers of batch elements; "
                                   "shard the inputs with partition() / shard_rows()")
        self._scratch = ([torch.empty(nbytes, dtype=torch.uint8, device=self.device) for _ in range(self.nb)]
                         if nbytes else None)
        self._schedule, self._schedule_key = schedule, key

    # ---- exchange --------------------------------------------------------------------------------------------
    def _exchange(self, local_b, elem_begin, elem_count):
        """barrier -> reduce+cast of image[local_b][elem_begin : elem_begin+elem_count) -> barrier, on the
        current stream."""
        from . import capi

        out_elem = self.out.element_size()
        if self.heads:
            # this rank's slice of the image is final: convert it and store it into every rank's grad_value
            slice_elems, full_elems = self.gr * self.shape[3], self.shape[2] * self.shape[3]
            if elem_begin % slice_elems or elem_count % slice_elems:
                raise RuntimeError("head-sharded exchange: a piece must consist of whole cells")
            batch_off = (self.part.b_begin + local_b) * self.shape[1] * full_elems * out_elem
            self.h_image.barrier(channel=0)   # nobody still reads the grad_value of the previous backward
            capi.head_slice_cast_push(self.image_ptrs[self.rank] + local_b * self.per_batch * 4,
                                      [p + batch_off for p in self.out_ptrs], self.rank, elem_begin // slice_elems,
                                      elem_count // slice_elems, slice_elems, full_elems, self.part.h_begin * self.shape[3],
                                      self.dtype, self.device)
            self.h_out.barrier(channel=0)     # every rank's slices have landed
            return
        img_off = (local_b * self.per_batch + elem_begin) * 4
        out_off = ((self.part.b_begin + local_b) * self.per_batch + elem_begin) * out_elem
        if self.use_push:
            img = self.image_ptrs[self.rank] + img_off
            capi.peer_push_partials(img, self.staging_ptrs, self.slot, self.rank, elem_count, self.device)
            self.h_image.barrier(channel=0)   # every rank's partials have landed in the owners' staging areas
            capi.peer_reduce_staged_cast(img, self.staging_ptrs[self.rank], self.slot,
                                         [p + out_off for p in self.out_ptrs], self.rank, elem_count, self.dtype, self.device)
            self.h_out.barrier(channel=0)     # every rank's results have landed; staging areas are free again
            return
        self.h_image.barrier(channel=0)   # every rank's part of the image is complete
        if self.use_multimem:             # in-switch sum (NVLS): 1/R of the bytes per GPU
            capi.multimem_reduce_cast(self.mc_image, self.mc_out, self.world, self.rank, elem_count, self.dtype,
                                      self.device, byte_offsets=(img_off, out_off))
        else:                             # plain peer loads from the group / stores to everyone
            capi.group_reduce_cast(self.group_image_ptrs, self.part.group_rank, self.out_ptrs, self.rank, elem_count,
                                   self.dtype, self.device, byte_offsets=(img_off, out_off))
        self.h_out.barrier(channel=0)     # every rank's pushes have landed

    def backward(self, value, shapes, lsi, packed, grad_out, K, im2col_step=64, grad_packed=None):
        """``value`` is the full replicated ``[B, N, G, D]``; ``packed`` / ``grad_out`` are this rank's rows
        ``[nb, Q_rank, ...]`` (``shard_rows``).  Returns ``(grad_value [B, N, G, D], grad_packed)``."""
        from . import capi

        if tuple(value.shape) != self.shape or value.dtype != self.dtype:
            raise ValueError("PeerReducer was built for another value shape / dtype")
        value = shard_value(value, self.part)   # [nb, N, heads of this rank, D]
        if packed.shape[0] != self.nb or grad_out.shape[0] != self.nb:
            raise ValueError(f"this rank works on {self.nb} batch element(s), got rows for {packed.shape[0]}")
        L = shapes.shape[0]
        if grad_packed is None:
            grad_packed = torch.empty_like(packed)
        # everything that can raise happens before the first barrier is queued
        self._plan(value, lsi, packed, K)
        main = torch.cuda.current_stream(self.device)
        self.side.wait_stream(main)  # earlier readers of self.out / self.image are done
        main.wait_stream(self.side)  # the zero-fill issued after the previous backward is done
        zero = 0 if self._image_clean else capi.BWD_ZERO_IMAGE
        self._image_clean = False
        scratch_of = (lambda lb: self._scratch[lb]) if self._scratch is not None else (lambda lb: None)

        def hand_over(lb, elem_begin, elem_count):
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(self.side):
                self.side.wait_event(done)
                self._exchange(lb, elem_begin, elem_count)

        def args_of(lb):
            return (value[lb:lb + 1], shapes, lsi, packed[lb:lb + 1], grad_out[lb:lb + 1], K,
                    self.image[lb:lb + 1], grad_packed[lb:lb + 1])

        kind, plan = self._schedule
        if kind == "slabs":
            # Slab pipeline: the largest level is scattered slab group by slab group; the z-range a group has
            # finished is handed to the exchange while the next group (and later the other levels) compute.
            parts, part_ranges, rest_ranges = plan
            for g in range(parts):
                for lb in range(self.nb):
                    capi.backward_binned_part(*args_of(lb), g, parts, zero, scratch_of(lb), im2col_step=im2col_step)
                    e0, e1 = part_ranges[g]
                    hand_over(lb, e0, e1 - e0)
            for lb in range(self.nb):
                capi.backward_accumulate_levels(*args_of(lb), 0, L,
                                                capi.BWD_RESUME | capi.BWD_FINALIZE | capi.BWD_BINNED_DONE,
                                                im2col_step=im2col_step, scratch=scratch_of(lb))
                for e0, e1 in rest_ranges:
                    hand_over(lb, e0, e1 - e0)
        elif kind == "levels":
            # pass-major order: the big level of every batch element first, so that all of its exchanges
            # hide behind later launches and only the small remainder of the last element is exposed
            for n, (la, le, e0, e1) in enumerate(plan):
                last = n == len(plan) - 1
                flags = (zero if n == 0 else capi.BWD_RESUME) | (capi.BWD_FINALIZE if last else 0)
                for lb in range(self.nb):
                    capi.backward_accumulate_levels(*args_of(lb), la, le, flags, im2col_step=im2col_step,
                                                    scratch=scratch_of(lb))
                    hand_over(lb, e0, e1 - e0)
        else:
            for lb in range(self.nb):
                capi.backward_accumulate_levels(*args_of(lb), 0, L, zero | capi.BWD_FINALIZE,
                                                im2col_step=im2col_step, scratch=scratch_of(lb))
                hand_over(lb, 0, self.per_batch)
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

    def backward_reduced(self, value, shapes, lsi, packed, grad_out, K, im2col_step, group, part):
        """Backward with the cross-rank sum done by ``PeerReducer`` (NVLink peer memory).  Returns
        ``None`` when ``FDA_SHARDED_REDUCE=nccl`` asks for the plain all-reduce path instead."""
        if os.environ.get("FDA_SHARDED_REDUCE", "peer") != "peer":
            return None
        key = (tuple(value.shape), value.dtype, value.device, id(group), part)
        if key not in self._reducers:
            self._reducers[key] = PeerReducer(value.shape, value.dtype, value.device, group, spatial_shapes=shapes, part=part)
        gv, gp = self._reducers[key].backward(value, shapes, lsi, packed, grad_out, K, im2col_step)
        # autograd may keep the returned tensor as ``value.grad``; it must not alias a buffer the next backward rewrites
        return gv.clone(), gp

    def forward(self, value, shapes, lsi, packed, K, im2col_step):
        from . import capi
        return capi.forward(value, shapes, lsi, packed, K, im2col_step=im2col_step)

    def backward_accumulate(self, value, shapes, lsi, packed, grad_out, K, im2col_step):
        """Returns ``(accum_fp32 like value, grad_packed)``."""
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


class ShardedFlashDeformAttnFunction(Function):
    """``apply(value, shapes, level_start_index, packed_rows, im2col_step, K, group, local_ops, part)``

    ``value`` is the full ``[B, N, G, D]`` on every rank; ``packed_rows`` holds this rank's rows
    ``[b_end-b_begin, q_end-q_begin, G, L*K*4]`` of partition ``part`` (``shard_rows``; only the rank's heads under a
    head split); returns the matching ``[.., .., G*D]`` rows of the output.  Backward returns the fully reduced ``grad_value`` (identical on
    every rank) and the local ``grad_packed_rows``.  ``local_ops`` is the per-rank operator
    (``CudaLocalOps()`` by default).
    """

    @staticmethod
    def forward(ctx, value, shapes, lsi, packed_rows, im2col_step, K, group=None, local_ops=None, part=None):
        ops = local_ops if local_ops is not None else _default_cuda_ops()
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        if part is None:
            if multi:
                # without the total query count only the batch split is known; the query range is the caller's
                p = partition(value.shape[0], 0, dist.get_rank(group), dist.get_world_size(group))
                part = p._replace(q_end=packed_rows.shape[1])
            else:
                part = Partition(0, value.shape[0], 0, packed_rows.shape[1], (0,), 0, "queries")
        ctx.ops, ctx.group, ctx.K, ctx.im2col_step, ctx.part, ctx.multi = ops, group, K, im2col_step, part, multi
        L = shapes.shape[0]
        if packed_rows.shape[-1] != L * K * 4:
            raise ValueError(
                f"sampling_loc_attn last dimension ({packed_rows.shape[-1]}) does not match L={L}, K={K}")
        if packed_rows.shape[0] != part.b_end - part.b_begin:
            raise ValueError(f"packed_rows holds {packed_rows.shape[0]} batch element(s), the partition "
                             f"{part.b_end - part.b_begin}: slice the inputs with shard_rows()")
        out = ops.forward(shard_value(value, part), shapes, lsi, packed_rows, K, im2col_step)
        ctx.save_for_backward(value, shapes, lsi, packed_rows)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_out):
        value, shapes, lsi, packed_rows = ctx.saved_tensors
        part = ctx.part
        none = (None,) * 5
        if ctx.multi and hasattr(ctx.ops, "backward_reduced"):
            fused = ctx.ops.backward_reduced(value, shapes, lsi, packed_rows, grad_out.contiguous(), ctx.K,
                                             ctx.im2col_step, ctx.group, part)
            if fused is not None:
                return (fused[0], None, None, fused[1]) + none
        local_value = shard_value(value, part)
        accum, grad_packed = ctx.ops.backward_accumulate(
            local_value, shapes, lsi, packed_rows, grad_out.contiguous(), ctx.K, ctx.im2col_step)
        if ctx.multi:
            if accum.shape != value.shape:  # batch-aligned partition: place the local images, sum the rest as zeros
                full = torch.zeros(value.shape, dtype=accum.dtype, device=accum.device)
                if part.splits_heads:
                    full[part.b_begin:part.b_end, :, part.h_begin:part.h_end] = accum
                else:
                    full[part.b_begin:part.b_end] = accum
                accum = full
            dist.all_reduce(accum, op=dist.ReduceOp.SUM, group=ctx.group)
        return (ctx.ops.cast(accum, value.dtype), None, None, grad_packed) + none


QueryShardedFlashDeformAttnFunction = ShardedFlashDeformAttnFunction  # earlier name


def sharded_flash_deform_attn(value, shapes, lsi, packed_rows, im2col_step, K, group=None,
                              local_ops: Optional[object] = None, part: Optional[Partition] = None):
    return ShardedFlashDeformAttnFunction.apply(value, shapes, lsi, packed_rows, im2col_step, K, group, local_ops, part)
