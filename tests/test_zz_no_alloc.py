"""The allocation-free backward entry point (``fda_backward_noalloc``) against the regular one and
against the CPU oracle.

Collected last on purpose (file name): if it fails under ``-x``, every other test has already run.
Both entry points run the same kernels; they differ in where the fp32 accumulation image lives
(caller's workspace vs. a fixed array inside the library), so results agree up to the order of the
floating-point atomics -- checked with the suite's 16-bit tolerance (2e-2 of the reference's
largest magnitude) and, for fp32 values, the fp32 tolerance (1e-4).  The same bounds are then
applied against the oracle, so the check does not rest on the other CUDA path being right.
"""
import pytest
import torch

from oracle import fda_oracle
from ops3d_b200 import capi

pytestmark = pytest.mark.gpu


def _inputs(shapes, B, Q, G, D, K, seed, vdt, dev="cuda"):
    value, sh, lsi, packed, grad_out = fda_oracle.make_inputs(shapes, B, Q, G, D, K, seed=seed)
    return value.to(dev, vdt), sh.to(dev), lsi.to(dev), packed.to(dev), grad_out.to(dev, vdt)


def _compare(args, K, tol):
    value, sh, lsi, packed, grad_out = args
    want_gv, want_gp = capi.backward(value, sh, lsi, packed, grad_out, K)
    # outputs pre-allocated by the caller and pre-filled with garbage: the call must overwrite all of it
    got_gv = torch.full_like(value, 7.0)
    got_gp = torch.full_like(packed, -3.0)
    capi.backward_noalloc(value, sh, lsi, packed, grad_out, K, got_gv, got_gp)
    torch.cuda.synchronize()
    _, ref_gv, ref_gp = fda_oracle.fused_forward_backward(value.cpu(), sh.cpu(), packed.cpu(), grad_out.cpu(), K)
    for got, want, ref in ((got_gv, want_gv, ref_gv), (got_gp, want_gp, ref_gp)):
        scale = max(1.0, ref.abs().max().item())
        assert (got.float() - want.float()).abs().max().item() <= tol * scale
        assert (got.float().cpu() - ref).abs().max().item() <= tol * scale


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    # first call: the larger problem, leaves its sums behind in the shared image ...
    first = _inputs([(8, 16, 32), (4, 8, 16)], 2, 300, 8, 32, 4, seed=21, vdt=torch.bfloat16)
    _compare(first, 4, 2e-2)
    # ... second call right after it: smaller, other shape and dtype; stale sums must not leak in
    second = _inputs([(4, 4, 8), (2, 2, 4), (1, 1, 2)], 1, 77, 4, 16, 8, seed=22, vdt=torch.float16)
    _compare(second, 8, 2e-2)
    # and the first problem again: what the second call left behind must not matter either
    _compare(first, 4, 2e-2)


def test_fp32_values_need_no_image_and_have_no_limit():
    args = _inputs([(4, 8, 8), (2, 4, 4)], 1, 64, 4, 16, 4, seed=23, vdt=torch.float32)
    _compare(args, 4, 1e-4)


def test_repeated_calls_return_the_same_status_and_result():
    """The first call on a device resolves the image's address; later calls reuse it and must behave the same."""
    args = _inputs([(4, 4, 8), (2, 2, 4)], 1, 40, 4, 16, 4, seed=24, vdt=torch.bfloat16)
    value, sh, lsi, packed, grad_out = args
    results = []
    for _ in range(3):
        gv, gp = torch.empty_like(value), torch.empty_like(packed)
        capi.backward_noalloc(value, sh, lsi, packed, grad_out, 4, gv, gp)  # raises on any non-zero status
        torch.cuda.synchronize()
        results.append((gv, gp))
    for gv, gp in results[1:]:
        assert torch.equal(gp, results[0][1])  # row-local, no atomics: bit-identical
        assert (gv.float() - results[0][0].float()).abs().max().item() <= 2e-2 * max(1.0, gv.float().abs().max().item())


def test_problem_larger_than_the_image_is_rejected():
    # 16-bit grad_value with more elements than the built-in image holds: refused before any launch
    N = capi.NOALLOC_MAX_ELEMENTS // (8 * 32) + 1
    dev = "cuda"
    value = torch.zeros(1, N, 8, 32, dtype=torch.bfloat16, device=dev)
    sh = torch.tensor([[1, 1, N]], dtype=torch.long, device=dev)
    lsi = torch.zeros(1, dtype=torch.long, device=dev)
    packed = torch.zeros(1, 4, 8, 16, device=dev)
    grad_out = torch.zeros(1, 4, 8 * 32, dtype=torch.bfloat16, device=dev)
    with pytest.raises(capi.FdaError) as info:
        capi.backward_noalloc(value, sh, lsi, packed, grad_out, 4, torch.empty_like(value), torch.empty_like(packed))
    assert info.value.status == 11
