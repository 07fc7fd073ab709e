"""ctypes view of the C ABI in ``include/fda_b200.h`` (``libfda_b200.so``), for callers that hold raw
device buffers: the parity tests, the benchmark and the multi-GPU wrapper.  Tensors are only used
here as owners of device memory; the library sees pointers, sizes and a stream.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FDA_B200_LIBRARY") or os.path.join(_HERE, "libfda_b200.so")  # override: another build of the same ABI

DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

EXPORTS = (
    "fda_status_string", "fda_last_cuda_error", "fda_version", "fda_forward",
    "fda_backward_workspace_bytes", "fda_backward_scratch_bytes", "fda_backward_sorted_scratch_bytes", "fda_backward_path", "fda_forward_head_group", "fda_backward", "fda_backward_accumulate", "fda_cast_grad_value",
    "fda_backward_noalloc", "fda_peer_reduce_cast", "fda_multimem_reduce_cast", "fda_backward_accumulate_levels",
    "fda_peer_push_partials", "fda_peer_reduce_staged_cast", "fda_backward_bin_plan", "fda_backward_binned_part",
    "fda_pack_sampling", "fda_pack_sampling_backward", "fda_dcnv4_forward", "fda_dcnv4_backward",
    "fda_dcnv4_backward_workspace_bytes", "fda_dcnv4_output_size", "fda_roi_align3d_forward", "fda_roi_align3d_backward",
    "fda_nms3d", "fda_nms3d_workspace_bytes", "fda_reload_config", "fda_group_reduce_cast", "fda_head_slice_cast_push",
    "fda_backward_touched_rows", "fda_cast_grad_value_touched",
)
BWD_ZERO_IMAGE, BWD_RESUME, BWD_FINALIZE, BWD_BINNED_DONE, BWD_ZERO_TOUCHED = 1, 2, 4, 8, 16
NOALLOC_MAX_ELEMENTS = 16 * 1024 * 1024

_lib = None

# Kernels launched through this module since import (this library's own kernels only; zero-fills are
# cudaMemsetAsync calls and are not counted).  Benchmarks read the difference around a timed region.
KERNEL_LAUNCHES = 0


def _count(n: int):
    global KERNEL_LAUNCHES
    KERNEL_LAUNCHES += n


class FdaError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"fda status {status}: {message}")
        self.status = status


def load() -> ctypes.CDLL:
    """Loads the library; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} not built; run `python -m ops3d_b200.build`")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.fda_status_string.argtypes = [i]
    lib.fda_status_string.restype = ctypes.c_char_p
    lib.fda_last_cuda_error.restype = i
    lib.fda_version.restype = i
    lib.fda_forward.argtypes = [vp] * 5 + [i] * 13 + [vp]
    lib.fda_forward.restype = i
    lib.fda_backward_workspace_bytes.argtypes = [i] * 9
    lib.fda_backward_scratch_bytes.argtypes = [i] * 8
    lib.fda_backward_path.argtypes = [i] * 8
    lib.fda_backward_path.restype = i
    lib.fda_forward_head_group.argtypes = [i] * 7
    lib.fda_forward_head_group.restype = i
    lib.fda_backward_sorted_scratch_bytes.argtypes = [i] * 8
    lib.fda_backward_sorted_scratch_bytes.restype = sz
    lib.fda_reload_config.restype = None
    lib.fda_backward_touched_rows.argtypes = [i] * 8
    lib.fda_backward_touched_rows.restype = i
    lib.fda_cast_grad_value_touched.argtypes = [vp] * 5 + [i] * 9 + [vp]
    lib.fda_cast_grad_value_touched.restype = i
    lib.fda_group_reduce_cast.argtypes = [vp, i, i, vp, i, i, sz, i, vp]
    lib.fda_group_reduce_cast.restype = i
    lib.fda_head_slice_cast_push.argtypes = [vp, vp, i, i, sz, sz, i, i, i, i, vp]
    lib.fda_head_slice_cast_push.restype = i
    lib.fda_backward_scratch_bytes.restype = sz
    lib.fda_backward_workspace_bytes.restype = sz
    lib.fda_backward.argtypes = [vp] * 8 + [sz] + [i] * 12 + [vp]
    lib.fda_backward.restype = i
    lib.fda_backward_accumulate.argtypes = [vp] * 7 + [i] * 10 + [vp]
    lib.fda_backward_accumulate.restype = i
    lib.fda_backward_accumulate_levels.argtypes = [vp] * 7 + [i] * 13 + [vp, sz, vp]
    lib.fda_backward_accumulate_levels.restype = i
    lib.fda_backward_bin_plan.argtypes = [vp] + [i] * 7 + [vp, vp, vp]
    lib.fda_backward_bin_plan.restype = i
    lib.fda_backward_binned_part.argtypes = [vp] * 7 + [i] * 13 + [vp, sz, vp]
    lib.fda_backward_binned_part.restype = i
    lib.fda_pack_sampling.argtypes = [vp] * 5 + [i] * 6 + [vp]
    lib.fda_pack_sampling.restype = i
    lib.fda_pack_sampling_backward.argtypes = [vp] * 5 + [i] * 6 + [vp]
    lib.fda_pack_sampling_backward.restype = i
    f = ctypes.c_float
    lib.fda_dcnv4_output_size.argtypes = [i, i, i] + [vp] * 7
    lib.fda_dcnv4_output_size.restype = i
    lib.fda_dcnv4_forward.argtypes = [vp] * 3 + [i] * 6 + [vp] * 4 + [f] + [i] * 5 + [vp]
    lib.fda_dcnv4_forward.restype = i
    lib.fda_dcnv4_backward_workspace_bytes.argtypes = [i] * 7
    lib.fda_dcnv4_backward_workspace_bytes.restype = sz
    lib.fda_dcnv4_backward.argtypes = [vp] * 6 + [sz] + [i] * 6 + [vp] * 4 + [f] + [i] * 5 + [vp]
    lib.fda_dcnv4_backward.restype = i
    lib.fda_roi_align3d_forward.argtypes = [vp] * 3 + [i] * 8 + [f] + [i] * 3 + [vp]
    lib.fda_roi_align3d_forward.restype = i
    lib.fda_roi_align3d_backward.argtypes = [vp] * 3 + [i] * 8 + [f] + [i] * 3 + [vp]
    lib.fda_roi_align3d_backward.restype = i
    lib.fda_nms3d_workspace_bytes.argtypes = [i]
    lib.fda_nms3d_workspace_bytes.restype = sz
    lib.fda_nms3d.argtypes = [vp, i, f, vp, sz, vp, vp, vp]
    lib.fda_nms3d.restype = i
    lib.fda_cast_grad_value.argtypes = [vp, vp, sz, i, vp]
    lib.fda_cast_grad_value.restype = i
    lib.fda_backward_noalloc.argtypes = [vp] * 7 + [i] * 10 + [vp]
    lib.fda_backward_noalloc.restype = i
    lib.fda_peer_reduce_cast.argtypes = [vp, vp, i, i, sz, i, vp]
    lib.fda_peer_reduce_cast.restype = i
    lib.fda_peer_push_partials.argtypes = [vp, vp, sz, i, i, sz, vp]
    lib.fda_peer_push_partials.restype = i
    lib.fda_peer_reduce_staged_cast.argtypes = [vp, vp, sz, vp, i, i, sz, i, vp]
    lib.fda_peer_reduce_staged_cast.restype = i
    lib.fda_multimem_reduce_cast.argtypes = [vp, vp, i, i, sz, i, vp]
    lib.fda_multimem_reduce_cast.restype = i
    _lib = lib
    return lib


def check(status: int):
    if status != 0:
        msg = load().fda_status_string(status).decode()
        if status == 10:
            msg += f" (cudaError {load().fda_last_cuda_error()})"
        raise FdaError(status, msg)


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _dims(value, shapes, packed):
    B, N, G, D = value.shape
    return B, N, G, D, shapes.shape[0], packed.shape[1]


def forward(value, shapes, lsi, packed, K, im2col_step=64, use_reg=True, out=None):
    """``fda_forward`` on CUDA tensors; returns ``[B, Q, G*D]`` in ``value.dtype``."""
    B, N, G, D, L, Q = _dims(value, shapes, packed)
    if out is None:
        out = torch.empty(B, Q, G * D, dtype=value.dtype, device=value.device)
    with torch.cuda.device(value.device):
        check(load().fda_forward(
            value.data_ptr(), shapes.data_ptr(), lsi.data_ptr(), packed.data_ptr(), out.data_ptr(),
            B, N, G, D, L, Q, K, DTYPE_CODE[value.dtype], DTYPE_CODE[packed.dtype],
            im2col_step, 8, 0, int(bool(use_reg)), _stream(value)))
    _count(1)
    return out


def reload_config():
    """Makes the library re-read its FDA_* environment knobs (it reads them once, when loaded)."""
    load().fda_reload_config()


def _levels(packed, K) -> int:
    return packed.shape[-1] // (4 * K)


def workspace_bytes(value, packed, K) -> int:
    B, N, G, D = value.shape
    return int(load().fda_backward_workspace_bytes(B, N, G, D, _levels(packed, K), packed.shape[1], K,
                                                   DTYPE_CODE[value.dtype], DTYPE_CODE[packed.dtype]))


def scratch_bytes(value, packed, K) -> int:
    """Bytes of scratch for launches that hand work to one another (slab lists; fp32 logit-gradient plane for
    16-bit offsets)."""
    B, N, G, D = value.shape
    args = (B, N, G, D, _levels(packed, K), packed.shape[1], K)
    return max(int(load().fda_backward_scratch_bytes(*args, DTYPE_CODE[packed.dtype])),
               int(load().fda_backward_sorted_scratch_bytes(*args, DTYPE_CODE[value.dtype])))


def binning_applies(value, packed, K) -> bool:
    """True when the slab-binned path handles the largest level of this problem (given scratch)."""
    B, N, G, D = value.shape
    return int(load().fda_backward_scratch_bytes(B, N, G, D, _levels(packed, K), packed.shape[1], K, 0)) > 0


def forward_head_group(value, packed, K) -> int:
    """Heads per group of the forward's row order (``G``: plain row order)."""
    B, N, G, D = value.shape
    return int(load().fda_forward_head_group(N, G, D, _levels(packed, K), packed.shape[1], K, DTYPE_CODE[value.dtype]))


def backward_path(value, packed, K) -> int:
    """0 plain scatter kernel, 1 slab-binned largest level, 2 cell-sorted (what a call with scratch takes)."""
    B, N, G, D = value.shape
    return int(load().fda_backward_path(B, N, G, D, _levels(packed, K), packed.shape[1], K, DTYPE_CODE[value.dtype]))


def backward_touched_rows(value, packed, K) -> bool:
    """True when ``fda_backward`` zero-fills and converts only the image rows that sampling points touch."""
    B, N, G, D = value.shape
    return bool(load().fda_backward_touched_rows(B, N, G, D, _levels(packed, K), packed.shape[1], K, DTYPE_CODE[value.dtype]))


def _scatter_launches(value, packed, K, first=True, last=True) -> int:
    """Kernels of one scatter call that was given scratch: sorted = (count, 3 x scan, fill on the first launch of a
    sequence) + walk (+ finalize on the last); binned = count, scan, fill, binned + plain; else the plain kernel."""
    path = backward_path(value, packed, K)
    if path == 2:
        return (5 if first else 0) + 1 + (1 if last else 0)
    return 5 if path == 1 else 1


def backward(value, shapes, lsi, packed, grad_out, K, im2col_step=64, grad_value=None, grad_packed=None,
             workspace=None):
    """``fda_backward`` on CUDA tensors; returns ``(grad_value, grad_packed)``."""
    B, N, G, D, L, Q = _dims(value, shapes, packed)
    if grad_value is None:
        grad_value = torch.empty_like(value)
    if grad_packed is None:
        grad_packed = torch.empty_like(packed)
    need = workspace_bytes(value, packed, K)
    if need and workspace is None:
        workspace = torch.empty((need + 3) // 4, dtype=torch.float32, device=value.device)
    with torch.cuda.device(value.device):
        check(load().fda_backward(
            value.data_ptr(), shapes.data_ptr(), lsi.data_ptr(), packed.data_ptr(), grad_out.data_ptr(),
            grad_value.data_ptr(), grad_packed.data_ptr(),
            workspace.data_ptr() if workspace is not None else None,
            workspace.numel() * workspace.element_size() if workspace is not None else 0,
            B, N, G, D, L, Q, K, DTYPE_CODE[value.dtype], DTYPE_CODE[packed.dtype],
            im2col_step, 1, 0, _stream(value)))
    # scatter kernels (the workspace includes the scratch of the binned / sorted path when one applies) + cast;
    # the sparse image handling adds the pass that zeroes the touched rows
    _count(_scatter_launches(value, packed, K) + (1 if value.dtype != torch.float32 else 0)
           + (1 if backward_touched_rows(value, packed, K) else 0))
    return grad_value, grad_packed


def backward_accumulate(value, shapes, lsi, packed, grad_out, K, accum, grad_packed=None, im2col_step=64):
    """``fda_backward_accumulate``: zero-fills and fills the fp32 image ``accum``; returns ``grad_packed``."""
    B, N, G, D, L, Q = _dims(value, shapes, packed)
    if grad_packed is None:
        grad_packed = torch.empty_like(packed)
    with torch.cuda.device(value.device):
        check(load().fda_backward_accumulate(
            value.data_ptr(), shapes.data_ptr(), lsi.data_ptr(), packed.data_ptr(), grad_out.data_ptr(),
            accum.data_ptr(), grad_packed.data_ptr(),
            B, N, G, D, L, Q, K, DTYPE_CODE[value.dtype], DTYPE_CODE[packed.dtype], im2col_step, _stream(value)))
    _count(1)
    return grad_packed


def backward_accumulate_levels(value, shapes, lsi, packed, grad_out, K, accum, grad_packed, level_begin, level_end,
                               flags, im2col_step=64, scratch=None):
    """``fda_backward_accumulate_levels``: one launch over the levels ``[level_begin, level_end)``.
    ``scratch`` (a tensor of at least ``scratch_bytes()`` bytes) enables the slab-binned path."""
    B, N, G, D, L, Q = _dims(value, shapes, packed)
    with torch.cuda.device(value.device):
        check(load().fda_backward_accumulate_levels(
            value.data_ptr(), shapes.data_ptr(), lsi.data_ptr(), packed.data_ptr(), grad_out.data_ptr(),
            accum.data_ptr(), grad_packed.data_ptr(),
            B, N, G, D, L, Q, K, DTYPE_CODE[value.dtype], DTYPE_CODE[packed.dtype], im2col_step,
            level_begin, level_end, flags,
            scratch.data_ptr() if scratch is not None else None,
            scratch.numel() * scratch.element_size() if scratch is not None else 0, _stream(value)))
    if (flags & BWD_ZERO_TOUCHED) and not (flags & BWD_ZERO_IMAGE) and value.dtype != torch.float32:
        _count(1)
    if scratch is None or (flags & BWD_BINNED_DONE):
        _count(1)
    else:
        _count(_scatter_launches(value, packed, K, first=not (flags & BWD_RESUME), last=bool(flags & BWD_FINALIZE)))
    return grad_packed


def bin_plan(shapes_host, value_shape, num_query, K):
    """``fda_backward_bin_plan`` on a host copy of the shapes: ``None`` when binning does not apply, else
    ``(level, slabs, planes_per_slab)``."""
    sh = torch.as_tensor(shapes_host).cpu().long().contiguous()
    B, N, G, D = value_shape
    lvl, slabs, depth = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
    ok = load().fda_backward_bin_plan(sh.data_ptr(), sh.shape[0], B, N, G, D, num_query, K,
                                      ctypes.addressof(lvl), ctypes.addressof(slabs), ctypes.addressof(depth))
    return (lvl.value, slabs.value, depth.value) if ok else None


def backward_binned_part(value, shapes, lsi, packed, grad_out, K, accum, grad_packed, part, parts, flags, scratch,
                         im2col_step=64):
    """``fda_backward_binned_part``: slab group ``part`` of ``parts`` of the largest level."""
    B, N, G, D, L, Q = _dims(value, shapes, packed)
    with torch.cuda.device(value.device):
        check(load().fda_backward_binned_part(
            value.data_ptr(), shapes.data_ptr(), lsi.data_ptr(), packed.data_ptr(), grad_out.data_ptr(),
            accum.data_ptr(), grad_packed.data_ptr(),
            B, N, G, D, L, Q, K, DTYPE_CODE[value.dtype], DTYPE_CODE[packed.dtype], im2col_step,
            part, parts, flags, scratch.data_ptr(), scratch.numel() * scratch.element_size(), _stream(value)))
    _count(1 + (3 if part == 0 else 0))
    return grad_packed


def cast_grad_value(accum, grad_value):
    with torch.cuda.device(accum.device):
        check(load().fda_cast_grad_value(accum.data_ptr(), grad_value.data_ptr(), accum.numel(),
                                         DTYPE_CODE[grad_value.dtype], _stream(accum)))
    _count(1 if grad_value.dtype != torch.float32 else 0)
    return grad_value


def cast_grad_value_touched(accum, grad_value, shapes, lsi, packed, K):
    """``fda_cast_grad_value_touched``: zero-fills ``grad_value`` and converts the image rows that the sampling points
    of ``packed`` touch (the counterpart of ``BWD_ZERO_TOUCHED``)."""
    B, N, G, D = grad_value.shape
    with torch.cuda.device(accum.device):
        check(load().fda_cast_grad_value_touched(
            accum.data_ptr(), grad_value.data_ptr(), shapes.data_ptr(), lsi.data_ptr(), packed.data_ptr(),
            B, N, G, D, shapes.shape[0], packed.shape[1], K, DTYPE_CODE[grad_value.dtype], DTYPE_CODE[packed.dtype],
            _stream(accum)))
    _count(1)
    return grad_value


def backward_noalloc(value, shapes, lsi, packed, grad_out, K, grad_value, grad_packed, im2col_step=64):
    """``fda_backward_noalloc``: the caller passes inputs and BOTH outputs; nothing is allocated here or
    in the library (the fp32 accumulation image is a fixed array inside ``libfda_b200.so``).  Raises
    ``FdaError`` (status 11) when ``value`` is 16-bit and has more than ``NOALLOC_MAX_ELEMENTS`` elements."""
    B, N, G, D, L, Q = _dims(value, shapes, packed)
    with torch.cuda.device(value.device):
        check(load().fda_backward_noalloc(
            value.data_ptr(), shapes.data_ptr(), lsi.data_ptr(), packed.data_ptr(), grad_out.data_ptr(),
            grad_value.data_ptr(), grad_packed.data_ptr(),
            B, N, G, D, L, Q, K, DTYPE_CODE[value.dtype], DTYPE_CODE[packed.dtype], im2col_step, _stream(value)))
    _count(1 + (1 if value.dtype != torch.float32 else 0))
    return grad_value, grad_packed


def peer_reduce_cast(image_ptrs, output_ptrs, rank, num_elements, dtype, device, byte_offsets=(0, 0)):
    """``fda_peer_reduce_cast`` on lists of per-rank device addresses (ints), e.g. the ``buffer_ptrs``
    of two symmetric-memory allocations.  ``byte_offsets`` = (image, output) offsets added to every
    address (to address one batch element of a larger buffer).  Runs on the current stream of
    ``device``; the caller provides the barriers before and after."""
    world = len(image_ptrs)
    imgs = (ctypes.c_void_p * world)(*[p + byte_offsets[0] for p in image_ptrs])
    outs = (ctypes.c_void_p * world)(*[p + byte_offsets[1] for p in output_ptrs])
    with torch.cuda.device(device):
        check(load().fda_peer_reduce_cast(imgs, outs, world, rank, num_elements, DTYPE_CODE[dtype],
                                          torch.cuda.current_stream(device).cuda_stream))
    _count(1)


def group_reduce_cast(group_image_ptrs, group_rank, output_ptrs, rank, num_elements, dtype, device, byte_offsets=(0, 0)):
    """``fda_group_reduce_cast``: like ``peer_reduce_cast`` but only the ranks of one group hold partial images
    (``group_image_ptrs``, indexed by rank within the group); the result goes to every rank's output."""
    gsize, world = len(group_image_ptrs), len(output_ptrs)
    imgs = (ctypes.c_void_p * gsize)(*[p + byte_offsets[0] for p in group_image_ptrs])
    outs = (ctypes.c_void_p * world)(*[p + byte_offsets[1] for p in output_ptrs])
    with torch.cuda.device(device):
        check(load().fda_group_reduce_cast(imgs, gsize, group_rank, outs, world, rank, num_elements, DTYPE_CODE[dtype],
                                           torch.cuda.current_stream(device).cuda_stream))
    _count(1)


def head_slice_cast_push(image_ptr, output_ptrs, rank, cell_begin, cell_count, slice_elements, full_elements,
                         head_offset_elements, dtype, device):
    """``fda_head_slice_cast_push``: ``image_ptr`` = this rank's compact fp32 image of one batch element (int address),
    ``output_ptrs`` = address of that batch element inside every rank's full gradient."""
    world = len(output_ptrs)
    outs = (ctypes.c_void_p * world)(*output_ptrs)
    with torch.cuda.device(device):
        check(load().fda_head_slice_cast_push(image_ptr, outs, world, rank, cell_begin, cell_count, slice_elements, full_elements,
                                              head_offset_elements, DTYPE_CODE[dtype], torch.cuda.current_stream(device).cuda_stream))
    _count(1)


def multimem_reduce_cast(mc_image_ptr, mc_output_ptr, world, rank, num_elements, dtype, device, byte_offsets=(0, 0)):
    """``fda_multimem_reduce_cast`` on the multicast addresses of two symmetric-memory allocations."""
    with torch.cuda.device(device):
        check(load().fda_multimem_reduce_cast(mc_image_ptr + byte_offsets[0], mc_output_ptr + byte_offsets[1], world, rank,
                                              num_elements, DTYPE_CODE[dtype], torch.cuda.current_stream(device).cuda_stream))
    _count(1)


def peer_push_partials(image_ptr, staging_ptrs, slot_stride, rank, num_elements, device):
    """``fda_peer_push_partials``: ``image_ptr`` = local image (int address, already offset to the range),
    ``staging_ptrs`` = per-rank staging addresses."""
    world = len(staging_ptrs)
    st = (ctypes.c_void_p * world)(*staging_ptrs)
    with torch.cuda.device(device):
        check(load().fda_peer_push_partials(image_ptr, st, slot_stride, world, rank, num_elements,
                                            torch.cuda.current_stream(device).cuda_stream))
    _count(1)


def peer_reduce_staged_cast(image_ptr, staging_ptr, slot_stride, output_ptrs, rank, num_elements, dtype, device):
    world = len(output_ptrs)
    outs = (ctypes.c_void_p * world)(*output_ptrs)
    with torch.cuda.device(device):
        check(load().fda_peer_reduce_staged_cast(image_ptr, staging_ptr, slot_stride, outs, world, rank, num_elements,
                                                 DTYPE_CODE[dtype], torch.cuda.current_stream(device).cuda_stream))
    _count(1)


def pack_sampling(offsets, reference_points, logits, shapes):
    """``fda_pack_sampling``: offsets ``[B,Q,G,L,K,3]``, reference points ``[B,Q,L,3]``, logits ``[B,Q,G,L,K]``
    (one dtype, contiguous, CUDA) -> packed ``[B,Q,G,L*K*4]`` fp32."""
    B, Q, G, L, K, _ = offsets.shape
    packed = torch.empty(B, Q, G, L * K * 4, dtype=torch.float32, device=offsets.device)
    with torch.cuda.device(offsets.device):
        check(load().fda_pack_sampling(offsets.data_ptr(), reference_points.data_ptr(), logits.data_ptr(), shapes.data_ptr(),
                                       packed.data_ptr(), B, Q, G, L, K, DTYPE_CODE[offsets.dtype], _stream(offsets)))
    _count(1)
    return packed


def pack_sampling_backward(grad_packed, shapes, B, Q, G, L, K, dtype):
    """``fda_pack_sampling_backward``: ``grad_packed`` fp32 ``[B,Q,G,L*K*4]`` -> ``(grad_offsets [B,Q,G,L,K,3],
    grad_reference_points [B,Q,L,3], grad_logits [B,Q,G,L,K])`` in ``dtype``."""
    dev = grad_packed.device
    g_off = torch.empty(B, Q, G, L, K, 3, dtype=dtype, device=dev)
    g_ref = torch.empty(B, Q, L, 3, dtype=dtype, device=dev)
    g_logit = torch.empty(B, Q, G, L, K, dtype=dtype, device=dev)
    with torch.cuda.device(dev):
        check(load().fda_pack_sampling_backward(grad_packed.data_ptr(), shapes.data_ptr(), g_off.data_ptr(), g_ref.data_ptr(),
                                                g_logit.data_ptr(), B, Q, G, L, K, DTYPE_CODE[dtype], _stream(grad_packed)))
    _count(1)
    return g_off, g_ref, g_logit


def _triple(v):
    arr = (ctypes.c_int * 3)(*[int(x) for x in v])
    return arr


def dcnv4_output_size(size_in, kernel, stride, pad, dilation):
    """``(depth_out, height_out, width_out)`` of a DCNv4-3D layer (all triples in (d, h, w) order)."""
    out = [ctypes.c_int(0) for _ in range(3)]
    check(load().fda_dcnv4_output_size(*[int(x) for x in size_in], _triple(kernel), _triple(stride), _triple(pad),
                                       _triple(dilation), *[ctypes.addressof(o) for o in out]))
    return tuple(o.value for o in out)


def dcnv4_forward(value, p_offset, kernel, stride, pad, dilation, group, group_channels, offset_scale, remove_center,
                  softmax, im2col_step=64):
    """``fda_dcnv4_forward``: value ``[B, Din, Hin, Win, G*Dg]``, p_offset ``[B, Do, Ho, Wo, padded]`` ->
    ``[B, Do, Ho, Wo, G*Dg]``."""
    B, Din, Hin, Win, C = value.shape
    Do, Ho, Wo = dcnv4_output_size((Din, Hin, Win), kernel, stride, pad, dilation)
    out = torch.empty(B, Do, Ho, Wo, C, dtype=value.dtype, device=value.device)
    with torch.cuda.device(value.device):
        check(load().fda_dcnv4_forward(value.data_ptr(), p_offset.data_ptr(), out.data_ptr(), B, Din, Hin, Win, group,
                                       group_channels, _triple(kernel), _triple(stride), _triple(pad), _triple(dilation),
                                       float(offset_scale), int(remove_center), int(bool(softmax)), p_offset.shape[-1],
                                       DTYPE_CODE[value.dtype], im2col_step, _stream(value)))
    _count(1)
    return out


def dcnv4_backward(value, p_offset, grad_output, kernel, stride, pad, dilation, group, group_channels, offset_scale,
                   remove_center, softmax, im2col_step=64):
    """``fda_dcnv4_backward`` -> ``(grad_value, grad_offset)`` in the inputs' dtype."""
    B, Din, Hin, Win, C = value.shape
    grad_value, grad_offset = torch.empty_like(value), torch.empty_like(p_offset)
    need = int(load().fda_dcnv4_backward_workspace_bytes(B, Din, Hin, Win, group, group_channels, DTYPE_CODE[value.dtype]))
    ws = torch.empty((need + 3) // 4, dtype=torch.float32, device=value.device) if need else None
    with torch.cuda.device(value.device):
        check(load().fda_dcnv4_backward(value.data_ptr(), p_offset.data_ptr(), grad_output.data_ptr(), grad_value.data_ptr(),
                                        grad_offset.data_ptr(), ws.data_ptr() if ws is not None else None, need, B, Din, Hin,
                                        Win, group, group_channels, _triple(kernel), _triple(stride), _triple(pad),
                                        _triple(dilation), float(offset_scale), int(remove_center), int(bool(softmax)),
                                        p_offset.shape[-1], DTYPE_CODE[value.dtype], im2col_step, _stream(value)))
    _count(1 + (1 if need else 0))
    return grad_value, grad_offset


def roi_align3d_forward(features, rois, output_size, spatial_scale, sampling_ratio, order):
    """``fda_roi_align3d_forward``: features ``[N,C,D,H,W]``, rois ``[n,7]`` (same dtype) -> ``[n,C,pd,ph,pw]``."""
    N, C, D, H, W = features.shape
    pd, ph, pw = output_size
    out = torch.empty(rois.shape[0], C, pd, ph, pw, dtype=features.dtype, device=features.device)
    with torch.cuda.device(features.device):
        check(load().fda_roi_align3d_forward(features.data_ptr(), rois.data_ptr(), out.data_ptr(), rois.shape[0], C, D, H, W,
                                             pd, ph, pw, float(spatial_scale), int(sampling_ratio), int(order),
                                             DTYPE_CODE[features.dtype], _stream(features)))
    _count(1)
    return out


def roi_align3d_backward(grad_output, rois, feature_shape, spatial_scale, sampling_ratio, order):
    """``fda_roi_align3d_backward`` -> fp32 ``grad_features`` of ``feature_shape``."""
    N, C, D, H, W = feature_shape
    n, _, pd, ph, pw = grad_output.shape
    grad = torch.zeros(N, C, D, H, W, dtype=torch.float32, device=grad_output.device)
    with torch.cuda.device(grad_output.device):
        check(load().fda_roi_align3d_backward(grad_output.data_ptr(), rois.data_ptr(), grad.data_ptr(), n, C, D, H, W, pd, ph, pw,
                                              float(spatial_scale), int(sampling_ratio), int(order),
                                              DTYPE_CODE[grad_output.dtype], _stream(grad_output)))
    _count(1)
    return grad


def nms3d(boxes_sorted, iou_threshold):
    """``fda_nms3d`` on fp32 boxes ``[n,6]`` already sorted by decreasing score -> positions of the kept boxes."""
    n = boxes_sorted.shape[0]
    dev = boxes_sorted.device
    keep = torch.empty(max(n, 1), dtype=torch.int64, device=dev)
    num = torch.zeros(1, dtype=torch.int32, device=dev)
    need = int(load().fda_nms3d_workspace_bytes(n))
    ws = torch.empty(max(need // 8, 1), dtype=torch.int64, device=dev)
    with torch.cuda.device(dev):
        check(load().fda_nms3d(boxes_sorted.data_ptr(), n, float(iou_threshold), ws.data_ptr(), need, keep.data_ptr(),
                               num.data_ptr(), _stream(boxes_sorted)))
    _count(2 if n else 0)
    return keep[: int(num.item())]
