"""Forward + backward of the operator for callers whose tensors live in HOST memory.

The straightforward way -- copy everything in, run forward and backward, copy everything out -- leaves
the GPU idle during 4.9 GB of PCIe traffic each way at the benchmark's largest configuration, and PCIe
idle during the kernels.  Rows (queries) are independent and ``grad_value`` accumulates, so the step is
cut into query chunks that flow through three streams:

    upload    value[b] once, then per chunk its packed rows and grad_output rows   (host -> device)
    compute   forward(chunk) -> out rows; backward(chunk) accumulates into the fp32 image of grad_value[b]
              (zero-filled by the first chunk of b) and writes the chunk's grad_packed rows;
              after the last chunk of b the image is cast (or, on several GPUs, exchanged) once
    download  per chunk out rows and grad_packed rows, then grad_value[b]          (device -> host)

with three device slots per direction, so chunk i+1 uploads and chunk i-1 downloads while chunk i
computes (PCIe is full duplex).  Results equal the one-shot operator's up to the order of the fp32
atomics in ``grad_value``; ``out`` and ``grad_packed`` rows are bit-identical.

Same call surface as ``FlashDeformAttnFunction`` forward + backward (reference
``ops3d/flash_deform_attn.py:68-136``) with host tensors; ``grad_output`` is an input because the
step is not split at a loss computed on the host.  Host tensors should be pinned; pageable memory
works but the copies then do not overlap.

Several GPUs: pass the rank's ``PeerReducer``; the tensors are this rank's rows (``sharded.shard_rows``),
``value_h`` is the full value (the ranks that share a batch element each upload an equal slice of it and
all-gather the slices over NVLink), the images are summed over NVLink after the last chunk of a batch
element, and each rank downloads ``1/world`` of the reduced ``grad_value`` (``grad_value_h`` is the
full-size host buffer; the slice this rank fills is returned).
"""
from __future__ import annotations

import os

import torch

from . import capi


class HostStreamedStep:
    SLOTS = 3

    def __init__(self, value_shape, value_dtype, rows_shape, packed_dtype, K, shapes, level_start_index, device,
                 chunk_queries=None, reducer=None):
        """``value_shape`` = full ``[B, N, G, D]``; ``rows_shape`` = ``[nb, Q_rows, G, L*K*4]`` of the packed rows
        this process handles (``nb = B`` on one GPU); ``shapes`` / ``level_start_index`` on the device."""
        B, N, G, D = value_shape
        nb, Q, G2, last = rows_shape
        if G2 != G or last % (4 * K):
            raise ValueError("rows_shape must be [nb, Q, G, L*K*4]")
        self.value_shape, self.vdt, self.pdt, self.K, self.L = tuple(value_shape), value_dtype, packed_dtype, K, last // (4 * K)
        self.nb, self.Q, self.device = nb, Q, device
        self.shapes, self.lsi = shapes, level_start_index
        self.reducer = reducer
        if reducer is not None and reducer.part.splits_heads:
            raise ValueError("HostStreamedStep streams query chunks: build the reducer on a partition that splits "
                             "queries, not heads (partition(..., mode='rows'))")
        self.b_begin = reducer.part.b_begin if reducer is not None else 0
        if reducer is None and nb != B:
            raise ValueError("without a reducer the rows must cover every batch element")
        if chunk_queries is None:
            per_b = int(os.environ.get("FDA_HOST_CHUNKS", "16"))  # 4 / 8 / 16 chunks per batch element: 117.9 / 111.7 / 109.4 ms per step at the largest configuration
            chunk_queries = -(-Q // max(1, per_b))
        self.chunk = max(1, min(int(chunk_queries), Q))
        self.chunks = [(q0, min(q0 + self.chunk, Q)) for q0 in range(0, Q, self.chunk)]
        dev = device
        self.value_d = torch.empty(nb, N, G, D, dtype=value_dtype, device=dev)
        if reducer is None:
            self.grad_value_d = torch.empty(nb, N, G, D, dtype=value_dtype, device=dev)
            self.image = (torch.empty(nb, N, G, D, dtype=torch.float32, device=dev)
                          if value_dtype != torch.float32 else self.grad_value_d)
        else:
            self.grad_value_d, self.image = reducer.out, reducer.image
        S = self.SLOTS
        self.packed_c = [torch.empty(1, self.chunk, G, last, dtype=packed_dtype, device=dev) for _ in range(S)]
        self.go_c = [torch.empty(1, self.chunk, G * D, dtype=value_dtype, device=dev) for _ in range(S)]
        self.out_c = [torch.empty(1, self.chunk, G * D, dtype=value_dtype, device=dev) for _ in range(S)]
        self.gp_c = [torch.empty(1, self.chunk, G, last, dtype=packed_dtype, device=dev) for _ in range(S)]
        nscr = capi.scratch_bytes(self.value_d[:1], self.packed_c[0], K)
        self.scratch = [torch.empty(nscr, dtype=torch.uint8, device=dev) if nscr else None for _ in range(S)]
        self.up = torch.cuda.Stream(device=dev)
        self.comp = torch.cuda.Stream(device=dev)
        self.down = torch.cuda.Stream(device=dev)
        ev = lambda: torch.cuda.Event()  # noqa: E731
        self.ev_in_ready = [ev() for _ in range(S)]
        self.ev_in_free = [ev() for _ in range(S)]
        self.ev_done = [ev() for _ in range(S)]
        self.ev_out_free = [ev() for _ in range(S)]
        self.ev_value = [ev() for _ in range(nb)]
        self.ev_gv = [ev() for _ in range(nb)]
        self.h2d_bytes = self.d2h_bytes = 0
        # Several ranks working on the same batch element: each uploads an equal slice of value[b] over PCIe and
        # the slices are all-gathered over NVLink, instead of every rank uploading all of it.
        self.gather_group, self.gather_size, self.gather_rank = None, 1, 0
        if reducer is not None and len(reducer.part.group) > 1 and (N * G * D) % (8 * len(reducer.part.group)) == 0:
            import torch.distributed as dist

            size = len(reducer.part.group)
            if size == reducer.world:
                mine = reducer.group
            else:  # every rank creates every group, in the same order
                mine = None
                for first in range(0, reducer.world, size):
                    ranks = list(range(first, first + size))
                    g = dist.new_group(ranks)
                    if reducer.rank in ranks:
                        mine = g
            self.gather_group, self.gather_size, self.gather_rank = mine, size, reducer.part.group_rank

    def run(self, value_h, packed_h, grad_out_h, out_h, grad_value_h, grad_packed_h):
        """Queues the whole step on the internal streams and makes the current stream wait for it (the call
        itself returns before the GPU is done; synchronise before reading the host outputs).  Returns the
        ``(flat_begin, flat_end)`` element range of ``grad_value_h`` this call filled."""
        K, L, S, nb = self.K, self.L, self.SLOTS, self.nb
        cur = torch.cuda.current_stream(self.device)
        for s in (self.up, self.comp, self.down):
            s.wait_stream(cur)
        red = self.reducer
        zero_first = capi.BWD_ZERO_IMAGE
        if red is not None:
            red.side.wait_stream(cur)
            self.comp.wait_stream(red.side)     # the zero-fill queued after the previous backward is done
            zero_first = 0 if red._image_clean else capi.BWD_ZERO_IMAGE
            red._image_clean = False
        h2d = d2h = 0
        n = 0
        for lb in range(nb):
            gb = self.b_begin + lb
            with torch.cuda.stream(self.up):
                if self.gather_group is None:
                    self.value_d[lb].copy_(value_h[gb], non_blocking=True)
                    h2d += self.value_d[lb].numel() * self.value_d.element_size()
                else:
                    import torch.distributed as dist

                    flat_d, flat_h = self.value_d[lb].view(-1), value_h[gb].view(-1)
                    per = flat_d.numel() // self.gather_size
                    piece = flat_d[self.gather_rank * per:(self.gather_rank + 1) * per]
                    piece.copy_(flat_h[self.gather_rank * per:(self.gather_rank + 1) * per], non_blocking=True)
                    dist.all_gather_into_tensor(flat_d, piece, group=self.gather_group)  # in place: piece sits at its slot
                    h2d += per * self.value_d.element_size()
                self.ev_value[lb].record(self.up)
            for c, (q0, q1) in enumerate(self.chunks):
                slot, m = n % S, q1 - q0
                pk, go = self.packed_c[slot][:, :m], self.go_c[slot][:, :m]
                out, gp = self.out_c[slot][:, :m], self.gp_c[slot][:, :m]
                with torch.cuda.stream(self.up):
                    if n >= S:
                        self.up.wait_event(self.ev_in_free[slot])    # the chunk that used this slot has been computed
                    pk.copy_(packed_h[lb:lb + 1, q0:q1], non_blocking=True)
                    go.copy_(grad_out_h[lb:lb + 1, q0:q1], non_blocking=True)
                    self.ev_in_ready[slot].record(self.up)
                h2d += pk.numel() * pk.element_size() + go.numel() * go.element_size()
                with torch.cuda.stream(self.comp):
                    self.comp.wait_event(self.ev_in_ready[slot])
                    if c == 0:
                        self.comp.wait_event(self.ev_value[lb])
                    if n >= S:
                        self.comp.wait_event(self.ev_out_free[slot])  # its results have left the slot
                    v = self.value_d[lb:lb + 1]
                    capi.forward(v, self.shapes, self.lsi, pk, K, out=out)
                    capi.backward_accumulate_levels(v, self.shapes, self.lsi, pk, go, K, self.image[lb:lb + 1], gp, 0, L,
                                                    (zero_first if c == 0 else 0) | capi.BWD_FINALIZE,
                                                    scratch=self.scratch[slot])
                    self.ev_in_free[slot].record(self.comp)
                    self.ev_done[slot].record(self.comp)
                with torch.cuda.stream(self.down):
                    self.down.wait_event(self.ev_done[slot])
                    out_h[lb:lb + 1, q0:q1].copy_(out, non_blocking=True)
                    grad_packed_h[lb:lb + 1, q0:q1].copy_(gp, non_blocking=True)
                    self.ev_out_free[slot].record(self.down)
                d2h += out.numel() * out.element_size() + gp.numel() * gp.element_size()
                n += 1
            # this batch element's image is complete
            if red is None:
                with torch.cuda.stream(self.comp):
                    if self.vdt != torch.float32:
                        capi.cast_grad_value(self.image[lb], self.grad_value_d[lb])
                    self.ev_gv[lb].record(self.comp)
                with torch.cuda.stream(self.down):
                    self.down.wait_event(self.ev_gv[lb])
                    grad_value_h[lb].copy_(self.grad_value_d[lb], non_blocking=True)
                d2h += self.grad_value_d[lb].numel() * self.grad_value_d.element_size()
            else:
                done = torch.cuda.Event()
                done.record(self.comp)
                with torch.cuda.stream(red.side):
                    red.side.wait_event(done)
                    red._exchange(lb, 0, red.per_batch)   # sum over the group + cast, result on every rank
        filled = (0, grad_value_h.numel())
        if red is not None:
            total = self.grad_value_d.numel()
            f0, f1 = (total // 8) * red.rank // red.world * 8, (total // 8) * (red.rank + 1) // red.world * 8
            if red.rank == red.world - 1:
                f1 = total
            with torch.cuda.stream(self.down):
                self.down.wait_stream(red.side)            # all exchanges done: grad_value complete on every rank
                grad_value_h.view(-1)[f0:f1].copy_(self.grad_value_d.view(-1)[f0:f1], non_blocking=True)
            with torch.cuda.stream(red.side):
                red.side.wait_stream(self.down)
                red.image.zero_()
            red._image_clean = True
            d2h += (f1 - f0) * self.grad_value_d.element_size()
            filled = (f0, f1)
        for s in (self.up, self.comp, self.down):
            cur.wait_stream(s)
        if red is not None:
            cur.wait_stream(red.side)
        self.h2d_bytes, self.d2h_bytes = h2d, d2h
        return filled


def flash_deform_attn_host(value_h, spatial_shapes, level_start_index, sampling_loc_attn_h, grad_output_h, K=8,
                           device=None, chunk_queries=None, pin=True):
    """One-shot convenience wrapper: forward + backward with host tensors, returns host tensors
    ``(output, grad_value, grad_sampling_loc_attn)``.  Builds the device slots on every call; keep a
    ``HostStreamedStep`` around when calling repeatedly with the same shapes."""
    device = torch.device(device if device is not None else "cuda")
    shapes = spatial_shapes.to(device)
    lsi = level_start_index.to(device)
    step = HostStreamedStep(value_h.shape, value_h.dtype, sampling_loc_attn_h.shape, sampling_loc_attn_h.dtype, K, shapes,
                            lsi, device, chunk_queries=chunk_queries)

    def host_like(shape, dtype):
        t = torch.empty(shape, dtype=dtype)
        return t.pin_memory() if pin else t

    B, Q, G, _ = sampling_loc_attn_h.shape
    out_h = host_like((B, Q, G * value_h.shape[3]), value_h.dtype)
    gv_h = host_like(value_h.shape, value_h.dtype)
    gp_h = host_like(sampling_loc_attn_h.shape, sampling_loc_attn_h.dtype)
    with torch.cuda.device(device):
        step.run(value_h, sampling_loc_attn_h, grad_output_h, out_h, gv_h, gp_h)
        torch.cuda.synchronize(device)
    return out_h, gv_h, gp_h
