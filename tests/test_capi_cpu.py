"""CPU-side checks of the C ABI: the library loads, exports everything the header declares, and
rejects bad arguments before touching a device (no kernel is launched here)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from ops3d_b200 import capi


def declared_functions():
    text = open(os.path.join(ROOT, "include", "fda_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fda_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = capi.load()
    names = declared_functions()
    assert {"fda_forward", "fda_backward", "fda_backward_workspace_bytes"} <= set(names)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/fda_b200.h but not exported"
    assert set(capi.EXPORTS) <= set(names)


def test_version_and_status_strings():
    lib = capi.load()
    assert lib.fda_version() >= 1000
    assert lib.fda_status_string(0) == b"ok"
    for code in range(1, 12):
        assert lib.fda_status_string(code) not in (b"ok", b"unknown status")
    assert lib.fda_status_string(999) == b"unknown status"


def _fwd(lib, ptr=16, B=1, N=8, G=1, D=8, L=1, Q=1, K=4, vdt=2, pdt=0, step=64):
    p = ctypes.c_void_p(ptr)
    return lib.fda_forward(p, p, p, p, p, B, N, G, D, L, Q, K, vdt, pdt, step, 8, 0, 1, None)


def test_forward_argument_validation_happens_on_the_host():
    lib = capi.load()
    assert _fwd(lib, ptr=0) == 1                      # null pointer
    assert _fwd(lib, vdt=7) == 2                      # unknown dtype
    assert _fwd(lib, vdt=0, pdt=2) == 2               # bf16 offsets with fp32 value: not in the envelope
    assert _fwd(lib, vdt=1, pdt=2) == 2               # mixed 16-bit types
    assert _fwd(lib, L=0) == 3 and _fwd(lib, L=6) == 3
    assert _fwd(lib, K=5) == 4 and _fwd(lib, K=16) == 4
    assert _fwd(lib, D=12) == 5                       # not a multiple of 8 bf16 channels
    assert _fwd(lib, D=264) == 5                      # head row longer than 512 bytes
    assert _fwd(lib, Q=0) == 6 and _fwd(lib, B=-1) == 6
    assert _fwd(lib, N=1 << 30, G=8, D=32) == 6       # 32-bit offsets inside one batch element
    assert _fwd(lib, B=5, step=2) == 7                # reference: batch % min(batch, im2col_step) != 0
    assert _fwd(lib, ptr=8) == 9                      # misaligned base address


def test_backward_workspace_contract():
    lib = capi.load()
    # arguments: B, N, G, D, L, Q, K, value dtype, packed dtype (0 = f32, 1 = f16, 2 = bf16)
    assert lib.fda_backward_workspace_bytes(2, 100, 8, 32, 2, 50, 4, 0, 0) == 0    # fp32 accumulates in place
    assert lib.fda_backward_workspace_bytes(2, 100, 8, 32, 2, 50, 4, 2, 0) == 2 * 100 * 8 * 32 * 4
    assert lib.fda_backward_workspace_bytes(2, 100, 8, 32, 2, 50, 4, 2, 2) == 2 * 100 * 8 * 32 * 4  # no hand-over: no plane
    assert lib.fda_backward_scratch_bytes(2, 100, 8, 32, 2, 50, 4, 0) == 0         # image fits L2: no binning
    # 16-bit offsets: fp32 plane [B][Q*G][L*K] for the logit gradients handed from launch to launch
    assert lib.fda_backward_scratch_bytes(2, 100, 8, 32, 2, 50, 4, 2) == 2 * 50 * 8 * 2 * 4 * 4
    # image of one batch element (598016 x 256 x 4 B) exceeds L2: counters + one 8-byte entry per (row, point)
    big = lib.fda_backward_scratch_bytes(2, 598016, 8, 32, 3, 1000, 8, 0)
    assert big == 3 * 2 * 128 * 4 + 2 * 1000 * 8 * 8 * 8
    assert lib.fda_backward_workspace_bytes(2, 598016, 8, 32, 3, 1000, 8, 2, 0) == 2 * 598016 * 256 * 4 + big
    plane = 2 * 1000 * 8 * 3 * 8 * 4
    assert lib.fda_backward_scratch_bytes(2, 598016, 8, 32, 3, 1000, 8, 2) == big + plane
    assert lib.fda_backward_workspace_bytes(2, 598016, 8, 32, 3, 1000, 8, 2, 2) == 2 * 598016 * 256 * 4 + big + plane
    p = ctypes.c_void_p(16)
    args = (1, 8, 1, 8, 1, 1, 4, 2, 0, 64, 1, 0, None)
    assert lib.fda_backward(p, p, p, p, p, p, p, None, 0, *args) == 8        # workspace missing
    assert lib.fda_backward(p, p, p, p, p, p, p, p, 16, *args) == 8          # workspace too small
    assert lib.fda_backward(p, p, p, p, p, None, p, p, 1 << 20, *args) == 1  # null output


def test_level_range_and_slab_part_validation():
    lib = capi.load()
    p = ctypes.c_void_p(256)
    dims = (1, 8, 1, 8, 2, 1, 4, 2, 0, 64)  # B, N, G, D, L, Q, K, value bf16, packed f32, im2col_step
    # empty / reversed / out-of-range level ranges
    for lb, le in ((1, 1), (2, 1), (0, 3), (-1, 1)):
        assert lib.fda_backward_accumulate_levels(p, p, p, p, p, p, p, *dims, lb, le, 5, None, 0, None) == 3
    # slab-part launches need scratch and a problem whose image exceeds L2
    assert lib.fda_backward_binned_part(p, p, p, p, p, p, p, *dims, 0, 4, 1, None, 0, None) == 8
    assert lib.fda_backward_binned_part(p, p, p, p, p, p, p, *dims, 4, 4, 1, p, 1 << 30, None) == 6  # part >= parts
    # BINNED_DONE without usable scratch is a caller error, not a silent full recomputation
    assert lib.fda_backward_accumulate_levels(p, p, p, p, p, p, p, *dims, 0, 2, 2 | 4 | 8, None, 0, None) == 8


def test_cell_sorted_path_selection_and_scratch_size():
    """Which backward a problem takes, and what the cell-sorted one needs: pure host functions of the shape."""
    lib = capi.load()
    B, N, G, D, L, Q, K = 2, 598016, 8, 32, 3, 598016, 8
    points, bins = B * Q * G * L * K, B * N * G
    r256 = lambda n: (n + 255) // 256 * 256  # noqa: E731
    tiles = (bins + 8191) // 8192
    want = r256(bins * 4) + r256(tiles * 4) + r256(points * 32) + r256(points * 16)
    assert lib.fda_backward_sorted_scratch_bytes(B, N, G, D, L, Q, K, 2) == want     # bf16: counters, scan, records, results
    assert lib.fda_backward_sorted_scratch_bytes(B, N, G, D, L, Q, K, 1) == want     # fp16 too
    assert lib.fda_backward_path(B, N, G, D, L, Q, K, 2) == 2
    assert lib.fda_backward_workspace_bytes(B, N, G, D, L, Q, K, 2, 0) == B * N * G * D * 4 + want
    assert lib.fda_backward_sorted_scratch_bytes(B, N, G, D, L, Q, K, 0) == 0        # fp32 values: not this path
    assert lib.fda_backward_path(B, N, G, D, L, Q, K, 0) == 1                        # ... but the image exceeds L2: brick-binned
    assert lib.fda_backward_sorted_scratch_bytes(B, N, G, 64, L, Q, K, 2) == 0       # 64 channels per head: not this path
    assert lib.fda_backward_sorted_scratch_bytes(B, N, G, D, L, Q // 16, K, 2) == 0  # 1.5 points per cell and head: too sparse
    assert lib.fda_backward_path(B, N, G, D, L, Q // 16, K, 2) == 1
    assert lib.fda_backward_sorted_scratch_bytes(1, 288, 4, 32, 2, 288, 4, 2) == 0   # a few thousand points: too small
    assert lib.fda_backward_path(1, 288, 4, 32, 2, 288, 4, 2) == 0
    # forward row order: head groups of 2 when 8 heads x 598016 cells x 64 B exceed the L2 budget and the call is large
    assert lib.fda_forward_head_group(N, G, D, L, Q, K, 2) == 2
    assert lib.fda_forward_head_group(N, 2, D, L, Q, K, 2) == 2        # a rank's 2-head slice fits: plain order (= all its heads)
    assert lib.fda_forward_head_group(N, G, D, L, 1000, K, 2) == G     # small call: plain row order
    assert lib.fda_forward_head_group(4608, G, D, 2, 4608, 4, 2) == G  # volume fits L2: plain row order
    # one rank of a head-split job at 8 GPUs: one batch element, 2 heads, every query -- as dense as the whole problem
    assert lib.fda_backward_path(1, N, 2, D, L, Q, K, 2) == 2


def test_sparse_image_handling_selection_and_validation(fda_env):
    """When fda_backward zeroes and converts only the image rows that points touch: a pure host function of the shape
    (8 corner rows per point against num_value rows per head: at most 60 % of the image)."""
    lib = capi.load()
    assert lib.fda_backward_touched_rows(4, 37376, 8, 32, 3, 200, 4, 2) == 1      # 200 object queries over 37 376 cells
    assert lib.fda_backward_touched_rows(4, 37376, 8, 32, 3, 200, 4, 1) == 1      # fp16 too
    assert lib.fda_backward_touched_rows(4, 37376, 8, 32, 3, 200, 4, 0) == 0      # fp32 accumulates in grad_value itself
    assert lib.fda_backward_touched_rows(4, 37376, 8, 32, 3, 400, 4, 2) == 0      # twice the queries: dense is cheaper
    assert lib.fda_backward_touched_rows(2, 4608, 8, 32, 2, 4608, 4, 2) == 0      # self-attention: every cell touched
    assert lib.fda_backward_touched_rows(2, 598016, 8, 32, 3, 598016, 8, 2) == 0  # cell-sorted path
    assert lib.fda_backward_touched_rows(2, 598016, 8, 32, 3, 100, 8, 2) == 1     # a 1.2 GB image for 100 queries
    assert lib.fda_backward_touched_rows(0, 37376, 8, 32, 3, 200, 4, 2) == 0
    fda_env(FDA_BWD_TOUCHED="0")
    assert lib.fda_backward_touched_rows(4, 37376, 8, 32, 3, 200, 4, 2) == 0
    fda_env(FDA_BWD_TOUCHED="2")
    assert lib.fda_backward_touched_rows(2, 4608, 8, 32, 2, 4608, 4, 2) == 1
    assert lib.fda_backward_touched_rows(2, 4608, 8, 32, 2, 4608, 4, 0) == 0
    # the conversion validates on the host: null pointers, an fp32 value (no separate image), alignment
    call = lambda a, g, pk, vdt: lib.fda_cast_grad_value_touched(a, g, 256, 256, pk, 1, 100, 2, 32, 1, 5, 4, vdt, 0, None)  # noqa: E731
    assert call(None, 256, 256, 2) == 1
    assert call(256, 256, None, 2) == 1
    assert call(256, 256, 256, 0) == 2
    assert call(256, 264, 256, 2) == 9


def test_exchange_kernels_validate_before_launch():
    lib = capi.load()
    ptrs = (ctypes.c_void_p * 2)(256, 512)
    assert lib.fda_peer_reduce_cast(None, ptrs, 2, 0, 64, 2, None) == 1
    assert lib.fda_peer_reduce_cast(ptrs, ptrs, 2, 2, 64, 2, None) == 6      # rank outside world
    assert lib.fda_peer_reduce_cast(ptrs, ptrs, 2, 0, 60, 2, None) == 6      # not a multiple of 8 elements
    assert lib.fda_peer_reduce_cast(ptrs, ptrs, 17, 0, 64, 2, None) == 6     # more than 16 ranks
    bad = (ctypes.c_void_p * 2)(256, 520)
    assert lib.fda_peer_reduce_cast(bad, ptrs, 2, 0, 64, 2, None) == 9       # misaligned peer buffer
    assert lib.fda_multimem_reduce_cast(None, ctypes.c_void_p(256), 2, 0, 64, 2, None) == 1
    assert lib.fda_peer_push_partials(ctypes.c_void_p(256), ptrs, 16, 2, 0, 64, None) == 6  # slot shorter than a slice
    img = ctypes.c_void_p(256)
    assert lib.fda_head_slice_cast_push(None, ptrs, 2, 0, 0, 10, 64, 256, 64, 2, None) == 1
    assert lib.fda_head_slice_cast_push(img, ptrs, 2, 0, 0, 10, 64, 256, 224, 2, None) == 6   # slice does not fit behind the offset
    assert lib.fda_head_slice_cast_push(img, ptrs, 2, 0, 0, 10, 60, 256, 64, 2, None) == 6    # not a multiple of 8 elements
    assert lib.fda_head_slice_cast_push(img, bad, 2, 0, 0, 10, 64, 256, 64, 2, None) == 9     # misaligned peer buffer
    assert lib.fda_head_slice_cast_push(img, ptrs, 2, 0, 0, 0, 64, 256, 64, 2, None) == 0     # nothing to do: no launch
    assert lib.fda_pack_sampling(None, None, None, None, None, 1, 1, 1, 1, 4, 0, None) == 1
    assert lib.fda_pack_sampling(ctypes.c_void_p(256), ctypes.c_void_p(256), ctypes.c_void_p(256), ctypes.c_void_p(256),
                                 ctypes.c_void_p(256), 1, 1, 1, 6, 4, 0, None) == 3


def test_bin_plan_is_a_pure_host_function():
    import torch

    shapes = torch.tensor([(32, 64, 256), (16, 32, 128), (8, 16, 64)])
    assert capi.bin_plan(shapes, (2, 598016, 8, 32), 598016, 8) == (0, 32, 1)
    assert capi.bin_plan(shapes.flip(0), (1, 598016, 8, 32), 1000, 4) == (2, 32, 1)   # largest level last
    assert capi.bin_plan(torch.tensor([(16, 32, 128), (8, 16, 64)]), (1, 73728, 8, 32), 73728, 4) is None  # 75 MB image fits
