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
    assert lib.fda_backward_workspace_bytes(2, 100, 8, 32, 50, 4, 0) == 0    # fp32 accumulates in place
    assert lib.fda_backward_workspace_bytes(2, 100, 8, 32, 50, 4, 2) == 2 * 100 * 8 * 32 * 4
    assert lib.fda_backward_scratch_bytes(2, 100, 8, 32, 50, 4) == 0         # image fits L2: no binning
    # image of one batch element (598016 x 256 x 4 B) exceeds L2: counters + one 8-byte entry per (row, point)
    big = lib.fda_backward_scratch_bytes(2, 598016, 8, 32, 1000, 8)
    assert big == 3 * 2 * 64 * 4 + 2 * 1000 * 8 * 8 * 8
    assert lib.fda_backward_workspace_bytes(2, 598016, 8, 32, 1000, 8, 2) == 2 * 598016 * 256 * 4 + big
    p = ctypes.c_void_p(16)
    args = (1, 8, 1, 8, 1, 1, 4, 2, 0, 64, 1, 0, None)
    assert lib.fda_backward(p, p, p, p, p, p, p, None, 0, *args) == 8        # workspace missing
    assert lib.fda_backward(p, p, p, p, p, p, p, p, 16, *args) == 8          # workspace too small
    assert lib.fda_backward(p, p, p, p, p, None, p, p, 1 << 20, *args) == 1  # null output
