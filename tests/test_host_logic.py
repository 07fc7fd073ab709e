"""Host-side mirror of the reference's Python interface (no device needed)."""
import pytest
import torch

import ops3d_b200
from ops3d_b200 import FlashDeformAttnFunction
from ops3d_b200.flash_deform_attn import findspec, findspec_bwd

# (B, Q, G, C) -> (findspec, findspec_bwd) as returned by the reference's own functions
# (ops3d/flash_deform_attn.py:26-62) for these arguments.
REFERENCE_SPECS = {
    (1, 288, 4, 16): ((8, 384), (1, 256)),
    (2, 4608, 8, 32): ((8, 512), (1, 256)),
    (4, 200, 8, 32): ((8, 512), (1, 256)),
    (1, 4096, 8, 64): ((8, 512), (2, 256)),
    (1, 294912, 8, 48): ((8, 432), (2, 192)),
    (5, 64, 4, 32): ((8, 512), (1, 256)),
    (64, 64, 4, 32): ((8, 512), (1, 256)),
    (1, 1, 4, 32): ((8, 16), (1, 128)),
    (3, 7, 2, 8): ((8, 42), (1, 112)),
}


@pytest.mark.parametrize("shape,want", sorted(REFERENCE_SPECS.items()))
def test_launch_hints_equal_the_reference(shape, want):
    assert findspec(*shape) == want[0]
    assert findspec_bwd(*shape) == want[1]


def test_launch_hints_are_cheap_at_full_size():
    import time
    t = time.perf_counter()
    findspec(2, 598016, 8, 32), findspec_bwd(2, 598016, 8, 32)
    assert time.perf_counter() - t < 0.05  # the reference's divisor scan takes ~40 ms here per call


def test_public_names():
    assert ops3d_b200._C is not None, "torch binding not built"
    assert hasattr(ops3d_b200._C, "flash_deform_attn_forward") and hasattr(ops3d_b200._C, "flash_deform_attn_backward")
    assert callable(FlashDeformAttnFunction.apply)


def test_reference_import_lines_resolve():
    """The import lines of the reference's callers and tests work unchanged (reference
    tests/test_flash_deform_attn_wrapper.py:12-13, tests/test_extension.py:26-29,
    tests/benchmark_flash_deform_attn.py:513)."""
    import importlib

    from ops3d import FlashDeformAttnFunction as F1
    from ops3d import _C as C1
    from ops3d.flash_deform_attn import FlashDeformAttnFunction as F2
    from ops3d.flash_deform_attn import factors, findspec as fs, findspec_bwd as fsb

    assert F1 is FlashDeformAttnFunction and F2 is FlashDeformAttnFunction
    assert C1 is ops3d_b200._C and importlib.import_module("ops3d._C") is C1
    assert hasattr(C1, "flash_deform_attn_forward") and hasattr(C1, "flash_deform_attn_backward")
    # the rest of the reference's binding (reference tests/test_extension.py:16-24, csrc/vision.cpp:15-21)
    for name in ("nms_3d", "roi_align_3d_forward", "roi_align_3d_backward", "dcnv4_forward", "dcnv4_backward"):
        assert hasattr(C1, name), name
    from ops3d import RoIAlign, RoIAlign3DFunction, nms_nd, roi_align_3d  # reference ops3d/__init__.py:8-25

    assert callable(nms_nd) and callable(roi_align_3d) and RoIAlign((2, 2, 2), 1.0).dim == 3 and RoIAlign3DFunction is not None
    assert fs is findspec and fsb is findspec_bwd
    assert factors(12) == [1, 2, 3, 4, 6, 12] and factors(1) == [1] and factors(49) == [1, 7, 49]


def _cpu_inputs(L=2, K=4, L_packed=None):
    shapes = torch.tensor([[4, 4, 4]] * L, dtype=torch.long)
    lsi = torch.cat((shapes.new_zeros(1), shapes.prod(1).cumsum(0)[:-1]))
    value = torch.rand(1, int(shapes.prod(1).sum()), 4, 32)
    Lp = L if L_packed is None else L_packed
    packed = torch.rand(1, 16, 4, Lp * K * 4)
    return value, shapes, lsi, packed


def test_last_dimension_mismatch_raises_value_error():
    value, shapes, lsi, packed = _cpu_inputs(L=2, L_packed=1)
    with pytest.raises(ValueError, match="does not match"):
        FlashDeformAttnFunction.apply(value, shapes, lsi, packed, 1, 4, True)


def test_cpu_tensors_raise_instead_of_falling_back():
    value, shapes, lsi, packed = _cpu_inputs()
    with pytest.raises((RuntimeError, AssertionError)):
        FlashDeformAttnFunction.apply(value, shapes, lsi, packed, 1, 4, True)


def test_product_package_never_touches_the_oracle():
    """The oracle is test infrastructure: nothing under ops3d_b200/ (Python or C++/CUDA) may import,
    include, load or call it, and the package has no CPU code path to fall back to."""
    import os
    import re

    import ops3d

    offenders = []
    roots = [os.path.dirname(os.path.abspath(m.__file__)) for m in (ops3d_b200, ops3d)]
    for root, (dirpath, _, files) in ((r, w) for r in roots for w in os.walk(r)):
        for name in files:
            if not name.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                continue
            text = open(os.path.join(dirpath, name), encoding="utf-8").read()
            pattern = r"\b(import|from)\s+oracle\b|oracle/|fda_oracle|libfda_oracle"
            if name.endswith(".py"):
                pattern += r"|grid_sample\("  # no PyTorch re-implementation of the operator inside the package
            if re.search(pattern, text):
                offenders.append(os.path.relpath(os.path.join(dirpath, name), root))
    assert offenders == []


def test_operator_fails_loudly_without_the_extension(monkeypatch):
    import ops3d_b200.flash_deform_attn as mod

    monkeypatch.setattr(mod, "_C", None)
    value, shapes, lsi, packed = _cpu_inputs()
    with pytest.raises(RuntimeError, match="extension not built"):
        FlashDeformAttnFunction.apply(value, shapes, lsi, packed, 1, 4, True)
