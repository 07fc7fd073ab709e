"""DCNv4-3D kernels (through the C ABI and through ``ops3d._C`` / ``DCNv4Function``) against fixtures produced by the
reference's own CUDA kernels (``tests/golden/dcnv4_*.npz``) and against the CPU oracle (``oracle/dcnv4_oracle.py``: a
PyTorch restatement of those kernels, pinned to the same fixtures).  Tolerances as for the attention operator: fp32 max-abs <= 1e-4 * max(1, |ref|max),
16-bit <= 2e-2 * |ref|max against the fp32 oracle on the same rounded inputs.

Sampling positions are kept off the voxel grid (``oracle.keep_positions_off_the_grid``): with 16-bit offsets many positions
are exact integers (offset == stencil centre - stencil index), where trilinear interpolation has a left and a right
derivative and the oracle (which passes positions through grid_sample's normalise / un-normalise round trip) may pick the
other one."""
import pytest
import torch

from conftest import dcnv4_golden_names, load_dcnv4_golden
from oracle import dcnv4_oracle as oracle
from ops3d_b200 import capi

pytestmark = pytest.mark.gpu

CASES = [
    # B, (Din, Hin, Win), G, Dg, kernel, stride, pad, dilation, remove_center, softmax
    (2, (5, 6, 7), 4, 16, (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 0, False),
    (1, (6, 5, 8), 2, 32, (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, True),    # 26 points, soft-maxed masks
    (2, (7, 8, 9), 3, 8, (3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), 0, True),     # stride 2
    (1, (8, 7, 6), 4, 16, (3, 3, 3), (1, 1, 1), (2, 2, 2), (2, 2, 2), 1, False),   # dilation 2
    (1, (4, 6, 5), 8, 32, (1, 3, 3), (1, 1, 1), (0, 1, 1), (1, 1, 1), 0, True),    # flat stencil, 8 groups x 32 channels
    (3, (3, 3, 3), 1, 64, (3, 3, 3), (1, 1, 1), (0, 0, 0), (1, 1, 1), 0, False),   # single output cell, no padding
]


def _tol(dtype, ref):
    return (1e-4 if dtype == torch.float32 else 2e-2) * max(1.0 if dtype == torch.float32 else 1e-6, ref.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16], ids=["f32", "bf16", "f16"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: f"B{c[0]}_{'x'.join(map(str, c[1]))}_G{c[2]}x{c[3]}_k{'x'.join(map(str, c[4]))}_s{c[5][0]}_d{c[7][0]}_rc{c[8]}_sm{int(c[9])}")
def test_dcnv4_matches_oracle(case, dtype):
    B, size_in, G, Dg, kernel, stride, pad, dilation, rc, softmax = case
    if dtype != torch.float32 and Dg % 8:
        pytest.skip("16-bit values need group_channels % 8 == 0")
    value, rows, grad_out = oracle.make_inputs(B, size_in, G, Dg, kernel, stride, pad, dilation, rc, seed=3)
    dev = "cuda"
    rows = oracle.keep_positions_off_the_grid(rows.to(dtype), size_in, kernel, stride, pad, dilation, G, 0.37, rc)
    v, o, go = value.to(dev, dtype), rows.to(dev), grad_out.to(dev, dtype)
    args = (kernel, stride, pad, dilation, G, Dg, 0.37, rc, softmax)
    out = capi.dcnv4_forward(v, o, *args)
    gv, goff = capi.dcnv4_backward(v, o, go, *args)
    torch.cuda.synchronize()
    ref_out, ref_gv, ref_goff = oracle.dcnv4_forward_backward(v.cpu(), o.cpu(), go.cpu(), *args)
    assert out.shape == ref_out.shape and out.dtype == dtype
    assert (out.float().cpu() - ref_out).abs().max().item() <= _tol(dtype, ref_out)
    assert (gv.float().cpu() - ref_gv).abs().max().item() <= _tol(dtype, ref_gv)
    assert (goff.float().cpu() - ref_goff).abs().max().item() <= _tol(dtype, ref_goff)
    K = kernel[0] * kernel[1] * kernel[2] - rc
    assert goff[..., G * K * 4:].abs().max().item() == 0 if goff.shape[-1] > G * K * 4 else True  # padding gets zero gradient


@pytest.mark.parametrize("name", dcnv4_golden_names())
def test_dcnv4_matches_reference_kernel_fixtures(name):
    g = load_dcnv4_golden(name)
    kernel, stride, pad, dilation, G, Dg, scale, rc, softmax = g["args"]
    dev = "cuda"
    v, o, go = g["value"].to(dev), g["offset"].to(dev), g["grad_out"].to(dev)
    out = capi.dcnv4_forward(v, o, kernel, stride, pad, dilation, G, Dg, scale, rc, softmax)
    gv, goff = capi.dcnv4_backward(v, o, go, kernel, stride, pad, dilation, G, Dg, scale, rc, softmax)
    torch.cuda.synchronize()
    assert (out.cpu() - g["out"]).abs().max().item() <= 1e-4 * max(1.0, g["out"].abs().max().item())
    if g["backward_stored"]:  # else: the reference's backward is not run on that case (see the fixture generator)
        assert (gv.cpu() - g["grad_value"]).abs().max().item() <= 1e-4 * max(1.0, g["grad_value"].abs().max().item())
        assert (goff.cpu() - g["grad_offset"]).abs().max().item() <= 1e-4 * max(1.0, g["grad_offset"].abs().max().item())


def test_binding_and_autograd_wrapper():
    """``ops3d._C.dcnv4_forward / dcnv4_backward`` with the reference's positional arguments, and the autograd wrapper."""
    from ops3d import _C
    from ops3d_b200.dcnv4 import DCNv4Function

    B, size_in, G, Dg = 2, (6, 6, 6), 4, 16
    kernel, stride, pad, dilation = (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1)
    value, rows, grad_out = oracle.make_inputs(B, size_in, G, Dg, kernel, stride, pad, dilation, 0, seed=5)
    dev = "cuda"
    v, o = value.to(dev).requires_grad_(True), rows.to(dev).requires_grad_(True)
    out = _C.dcnv4_forward(v.detach(), o.detach(), *kernel, *stride, *pad, *dilation, G, Dg, 1.0, 64, 0, 8, 256, True)
    gv, goff = _C.dcnv4_backward(v.detach(), o.detach(), *kernel, *stride, *pad, *dilation, G, Dg, 1.0, 64, grad_out.to(dev), 0,
                                 8, 256, True)
    out2 = DCNv4Function.apply(v, o, kernel, stride, pad, dilation, G, Dg, 1.0, 64, 0, True)
    out2.backward(grad_out.to(dev))
    torch.cuda.synchronize()
    ref_out, ref_gv, ref_goff = oracle.dcnv4_forward_backward(value, rows, grad_out, kernel, stride, pad, dilation, G, Dg, 1.0, 0, True)
    assert torch.equal(out, out2)
    for got, ref in ((out, ref_out), (gv, ref_gv), (goff, ref_goff), (v.grad, ref_gv), (o.grad, ref_goff)):
        assert (got.cpu() - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())
    with pytest.raises(RuntimeError):
        _C.dcnv4_forward(v.detach().cpu(), o.detach().cpu(), *kernel, *stride, *pad, *dilation, G, Dg, 1.0, 64, 0, 8, 256, True)


def test_larger_volume_bf16():
    """A 3x3x3 layer over a 16x32x32 volume with 8 groups x 32 channels, the shape class the attention benchmark uses."""
    B, size_in, G, Dg = 1, (16, 32, 32), 8, 32
    kernel, stride, pad, dilation = (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1)
    value, rows, grad_out = oracle.make_inputs(B, size_in, G, Dg, kernel, stride, pad, dilation, 1, seed=9, offset_std=1.5)
    dev = "cuda"
    rows = oracle.keep_positions_off_the_grid(rows.bfloat16(), size_in, kernel, stride, pad, dilation, G, 0.73, 1)
    v, o, go = value.to(dev, torch.bfloat16), rows.to(dev), grad_out.to(dev, torch.bfloat16)
    args = (kernel, stride, pad, dilation, G, Dg, 0.73, 1, True)
    out = capi.dcnv4_forward(v, o, *args)
    gv, goff = capi.dcnv4_backward(v, o, go, *args)
    torch.cuda.synchronize()
    ref_out, ref_gv, ref_goff = oracle.dcnv4_forward_backward(v.cpu(), o.cpu(), go.cpu(), *args)
    for got, ref in ((out, ref_out), (gv, ref_gv), (goff, ref_goff)):
        assert (got.float().cpu() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
