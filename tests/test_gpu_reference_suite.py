"""The reference's own GPU test recipes (tests/test_flash_deform_attn.py, _stress.py and _wrapper.py
of cell-observatory/ops3d) re-stated against this package: same shapes, seeds, value
distributions and tolerances (rtol 1e-2 / atol 1e-3; bf16 atol 1e-2), same entry points
(``FlashDeformAttnFunction.apply`` and the raw ``_C`` binding), and the reference's own import lines
(tests/test_flash_deform_attn.py:9-12, tests/test_flash_deform_attn_wrapper.py:12-13):
``ms_deform_attn_core_pytorch_3d`` is attached to ``ops3d`` by tests/conftest.py from the CPU oracle."""
import pytest
import torch
import torch.nn.functional as F

from ops3d import FlashDeformAttnFunction, ms_deform_attn_core_pytorch_3d
from ops3d import _C as _C
from ops3d.flash_deform_attn import findspec, findspec_bwd
from oracle.fda_oracle import fused_forward_backward, level_start_index_of

pytestmark = pytest.mark.gpu
DEV = "cuda"


def make(N, M, D, Lq, L, K, shapes, dtype=torch.float32, seed=42, device=DEV):
    shapes_t = shapes if isinstance(shapes, torch.Tensor) else torch.tensor(shapes, dtype=torch.long, device=device)
    lsi = level_start_index_of(shapes_t)
    S = int(shapes_t.prod(1).sum())
    torch.manual_seed(seed)
    value = torch.rand(N, S, M, D, device=device, dtype=dtype) * 0.01
    loc = torch.rand(N, Lq, M, L, K, 3, device=device, dtype=dtype)
    logits = torch.rand(N, Lq, M, L, K, device=device, dtype=dtype) + 1e-5
    soft = F.softmax(logits.flatten(-2, -1), dim=-1).unflatten(-1, (L, K))
    packed = torch.cat([loc.reshape(N, Lq, M, L * K * 3), logits.reshape(N, Lq, M, L * K)], dim=-1)
    return value, loc, soft, packed, shapes_t, lsi


def oracle(value, shapes_t, loc, soft):
    return ms_deform_attn_core_pytorch_3d(value.float().cpu(), shapes_t.cpu(), loc.float().cpu(), soft.float().cpu())


@torch.no_grad()
def test_forward_half_default_shape():
    # reference default_forward_params: N=1, M=8, D=64, Lq=4096, L=4 (64^3 .. 8^3), K=8
    shapes = [[64] * 3, [32] * 3, [16] * 3, [8] * 3]
    value, loc, soft, packed, sh, lsi = make(1, 8, 64, 4096, 4, 8, shapes)
    out = FlashDeformAttnFunction.apply(value.half(), sh, lsi, packed.half(), 128, 8, True)
    ref = oracle(value, sh, loc, soft)
    assert not torch.isnan(out).any() and not torch.isinf(out).any()
    assert torch.allclose(out.float().cpu(), ref, rtol=1e-2, atol=1e-3)


def test_backward_half_default_shape():
    # reference default_backward_params (tests/conftest.py:60-87) at its own size: N=1, M=8, D=48,
    # Lq = 64^3 + 32^3 = 294912, L=2 (64^3, 32^3), K=4; loss = out.sum() / 10, i.e. grad_output = 0.1.
    # The oracle side is evaluated query-chunked (same autograd recipe per chunk) to bound host memory.
    shapes = [[64] * 3, [32] * 3]
    N, M, D, L, K, Lq = 1, 8, 48, 2, 4, 64 ** 3 + 32 ** 3
    sh = torch.tensor(shapes, dtype=torch.long, device=DEV)
    lsi = level_start_index_of(sh)
    S = int(sh.prod(1).sum())
    torch.manual_seed(42)
    value = (torch.rand(N, S, M, D, device=DEV) * 0.01).half().requires_grad_(True)
    loc = torch.rand(N, Lq, M, L, K, 3, device=DEV).half()
    logits = (torch.rand(N, Lq, M, L, K, device=DEV) + 1e-5).half()
    packed = torch.cat([loc.reshape(N, Lq, M, L * K * 3), logits.reshape(N, Lq, M, L * K)], dim=-1).requires_grad_(True)
    out = FlashDeformAttnFunction.apply(value, sh, lsi, packed, 64, K, True)
    (out.sum() / 10).backward()

    ref, ref_gv, ref_gp = fused_forward_backward(value.detach().cpu(), sh.cpu(), packed.detach().cpu(),
                                                 torch.full((N, Lq, M * D), 0.1), K, chunk=32768)
    assert torch.allclose(out.float().cpu(), ref, rtol=1e-2, atol=1e-3)
    assert torch.allclose(value.grad.float().cpu(), ref_gv, rtol=1e-2, atol=1e-3)
    g = packed.grad.float().cpu()
    assert torch.allclose(g[..., : L * K * 3], ref_gp[..., : L * K * 3], rtol=1e-2, atol=1e-3)
    assert torch.allclose(g[..., L * K * 3:], ref_gp[..., L * K * 3:], rtol=1e-2, atol=1e-3)


@torch.no_grad()
def test_raw_binding_signature():
    """Nine positional arguments each, hints taken from findspec / findspec_bwd."""
    shapes = [[16] * 3, [8] * 3]
    value, loc, soft, packed, sh, lsi = make(2, 8, 32, 256, 2, 4, shapes)
    d_stride, threads = findspec(2, 256, 8, 32)
    out = _C.flash_deform_attn_forward(value, sh, lsi, packed, 64, 4, d_stride, threads, True)
    assert out.shape == (2, 256, 8 * 32)
    assert torch.allclose(out.cpu(), oracle(value, sh, loc, soft), rtol=1e-2, atol=1e-3)
    d_b, t_b = findspec_bwd(2, 256, 8, 32)
    gv, gp = _C.flash_deform_attn_backward(value, sh, lsi, packed, torch.ones_like(out), 64, 4, d_b, t_b)
    assert gv.shape == value.shape and gp.shape == packed.shape


EDGE = [
    (1, (1, 1, 1), 1), (1, (4, 4, 4), 1), (1, (7, 7, 7), 1), (1, (8, 8, 8), 1), (1, (16, 16, 16), 1),
    (2, (4, 4, 4), 1), (2, (8, 8, 8), 1), (3, (4, 4, 4), 1), (3, (16, 16, 16), 1), (4, (8, 8, 8), 2),
    (5, (4, 4, 4), 1), (1, (32, 16, 8), 1), (2, (16, 8, 4), 1), (1, (8, 4, 2), 1), (2, (32, 16, 8), 1),
    (1, (8, 8, 8), 64),
]


@pytest.mark.parametrize("K", [4, 8])
@pytest.mark.parametrize("L,spatial,B", EDGE)
@torch.no_grad()
def test_forward_edge_shapes(L, spatial, B, K):
    M, D = 4, 32
    Lq = max(1, min(64, spatial[0] * spatial[1] * spatial[2]))
    value, loc, soft, packed, sh, lsi = make(B, M, D, Lq, L, K, [list(spatial)] * L)
    out = FlashDeformAttnFunction.apply(value, sh, lsi, packed, B, K, True)
    ref = oracle(value, sh, loc, soft)
    assert not torch.isnan(out).any() and not torch.isinf(out).any()
    assert torch.allclose(out.cpu(), ref, rtol=1e-2, atol=1e-3)


@pytest.mark.parametrize("shapes", [[[1, 1, 1], [64, 64, 64]], [[32, 16, 8], [16, 8, 4]]])
@torch.no_grad()
def test_forward_uneven_and_anisotropic_levels(shapes):
    value, loc, soft, packed, sh, lsi = make(1, 4, 32, 64, 2, 4, shapes)
    out = FlashDeformAttnFunction.apply(value, sh, lsi, packed, 1, 4, True)
    assert torch.allclose(out.cpu(), oracle(value, sh, loc, soft), rtol=1e-2, atol=1e-3)


def test_invalid_batch_not_divisible_by_im2col_step():
    value, _, _, packed, sh, lsi = make(5, 4, 32, 64, 2, 4, [[4, 4, 4]] * 2)
    with pytest.raises((RuntimeError, AssertionError)):
        FlashDeformAttnFunction.apply(value, sh, lsi, packed, 2, 4, True)


def test_invalid_six_levels():
    value, _, _, packed, sh, lsi = make(1, 4, 32, 64, 6, 4, [[4, 4, 4]] * 6)
    with pytest.raises((RuntimeError, ValueError)):
        FlashDeformAttnFunction.apply(value, sh, lsi, packed, 1, 4, True)


def test_invalid_point_count_is_a_value_error():
    value, _, _, packed, sh, lsi = make(1, 4, 32, 64, 2, 2, [[4, 4, 4]] * 2)
    with pytest.raises(ValueError):
        FlashDeformAttnFunction.apply(value, sh, lsi, packed, 1, 2, True)


def test_invalid_cpu_tensors():
    value, _, _, packed, sh, lsi = make(1, 4, 32, 64, 2, 4, [[4, 4, 4]] * 2, device="cpu")
    with pytest.raises((RuntimeError, AssertionError)):
        FlashDeformAttnFunction.apply(value, sh, lsi, packed, 1, 4, True)


def test_invalid_non_contiguous():
    value, _, _, packed, sh, lsi = make(1, 4, 32, 64, 2, 4, [[4, 4, 4]] * 2)
    with pytest.raises(RuntimeError):
        FlashDeformAttnFunction.apply(value.transpose(2, 3), sh, lsi, packed, 1, 4, True)


def test_invalid_shape_mismatch():
    value, _, _, _, sh, lsi = make(1, 4, 32, 64, 2, 4, [[4, 4, 4]] * 2)
    wrong = torch.rand(1, 64, 4, 1 * 4 * 4, device=DEV)
    with pytest.raises(ValueError, match="does not match"):
        FlashDeformAttnFunction.apply(value, sh, lsi, wrong, 1, 4, True)


def _stress(dtype=torch.float32):
    return make(1, 4, 32, 64, 1, 4, [[4, 4, 4]], dtype=dtype)


@torch.no_grad()
def test_numeric_zeros():
    sh = torch.tensor([[4, 4, 4]], dtype=torch.long, device=DEV)
    lsi = level_start_index_of(sh)
    value = torch.zeros(1, 64, 4, 32, device=DEV)
    loc = torch.full((1, 64, 4, 1, 4, 3), 0.5, device=DEV)
    soft = torch.full((1, 64, 4, 1, 4), 0.25, device=DEV)
    packed = torch.cat([loc.reshape(1, 64, 4, 12), soft.reshape(1, 64, 4, 4)], dim=-1)
    out = FlashDeformAttnFunction.apply(value, sh, lsi, packed, 1, 4, True)
    assert not torch.isnan(out).any() and not torch.isinf(out).any()
    assert torch.allclose(out.cpu(), oracle(value, sh, loc, soft), rtol=1e-5, atol=1e-6)


@torch.no_grad()
def test_numeric_small_values():
    value, loc, soft, packed, sh, lsi = _stress()
    value = value * 1e-6
    loc = loc * 1e-6 + 0.5
    # as the reference's test: the packed logits slot carries the already soft-maxed weights
    packed = torch.cat([loc.reshape(1, 64, 4, 12), soft.reshape(1, 64, 4, 4)], dim=-1)
    out = FlashDeformAttnFunction.apply(value, sh, lsi, packed, 1, 4, True)
    assert torch.allclose(out.cpu(), oracle(value, sh, loc, soft), rtol=1e-2, atol=1e-4)


@torch.no_grad()
def test_numeric_large_values_fp32():
    value, loc, soft, packed, sh, lsi = _stress()
    value = value * 1e4
    out = FlashDeformAttnFunction.apply(value, sh, lsi, packed, 1, 4, True)
    assert torch.allclose(out.cpu(), oracle(value, sh, loc, soft), rtol=1e-2, atol=1e-1)


@pytest.mark.parametrize("dtype,atol", [(torch.float16, 1e-3), (torch.bfloat16, 1e-2)])
@torch.no_grad()
def test_numeric_16bit_everything(dtype, atol):
    value, loc, soft, packed, sh, lsi = _stress(dtype)
    out = FlashDeformAttnFunction.apply(value, sh, lsi, packed, 1, 4, True)
    assert out.dtype == dtype
    assert torch.allclose(out.float().cpu(), oracle(value, sh, loc, soft), rtol=1e-2, atol=atol)


def test_gradient_zero_grad_output():
    value, _, _, packed, sh, lsi = make(1, 4, 32, 64, 2, 4, [[4, 4, 4]] * 2)
    value.requires_grad_(True)
    packed.requires_grad_(True)
    out = FlashDeformAttnFunction.apply(value, sh, lsi, packed, 1, 4, True)
    out.backward(torch.zeros_like(out))
    assert value.grad is not None and value.grad.abs().max() == 0
    assert packed.grad is not None and packed.grad.abs().max() == 0
