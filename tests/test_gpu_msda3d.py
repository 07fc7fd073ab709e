"""The layer around the operator (``MSDeformAttn3D``) and its fused packing kernel against a plain PyTorch
composition that ends in the CPU oracle: forward and all parameter / input gradients."""
import pytest
import torch
import torch.nn.functional as F

from oracle.fda_oracle import level_start_index_of, ms_deform_attn_core_pytorch_3d

pytestmark = pytest.mark.gpu


def torch_layer(m, query, ref, src, shapes):
    """Same layer with separate PyTorch ops and the oracle (fp32, CPU)."""
    B, Q, _ = query.shape
    G, L, K = m.n_heads, m.n_levels, m.n_points
    value = m.value_proj(src).view(B, src.shape[1], G, -1)
    off = m.sampling_offsets(query).view(B, Q, G, L, K, 3)
    logits = m.attention_weights(query).view(B, Q, G, L, K)
    extent = shapes.flip(-1).to(off.dtype)  # (W, H, D)
    loc = ref[:, :, None, :, None, :] + off / extent[None, None, None, :, None, :]
    attn = F.softmax(logits.flatten(-2), -1).view(B, Q, G, L, K)
    return m.output_proj(ms_deform_attn_core_pytorch_3d(value, shapes, loc, attn))


@pytest.mark.parametrize("fused", [True, False], ids=["fused-gemm", "pack-kernel"])
@pytest.mark.parametrize("K", [4, 8])
def test_layer_matches_pytorch_composition(K, fused):
    from ops3d_b200.msda3d import MSDeformAttn3D

    torch.manual_seed(0)
    shapes = torch.tensor([(6, 8, 10), (3, 4, 5)])
    lsi = level_start_index_of(shapes)
    N = int(shapes.prod(1).sum())
    B, Q, C = 2, 37, 64
    ref_layer = MSDeformAttn3D(C, 2, 4, K)
    with torch.no_grad():  # non-trivial projections for the test
        ref_layer.sampling_offsets.weight.normal_(0, 0.05)
        ref_layer.attention_weights.weight.normal_(0, 0.3)
    query = torch.randn(B, Q, C, requires_grad=True)
    src = torch.randn(B, N, C, requires_grad=True)
    ref = torch.rand(B, Q, 2, 3, requires_grad=True)
    want = torch_layer(ref_layer, query, ref, src, shapes)
    gout = torch.randn_like(want)
    want.backward(gout)
    want_grads = [query.grad.clone(), src.grad.clone(), ref.grad.clone()] + [p.grad.clone() for p in ref_layer.parameters()]

    dev = "cuda"
    layer = MSDeformAttn3D(C, 2, 4, K, fused_projection=fused).to(dev)
    layer.load_state_dict(ref_layer.state_dict())
    q2, s2, r2 = (t.detach().to(dev).requires_grad_(True) for t in (query, src, ref))
    got = layer(q2, r2, s2, shapes.to(dev), lsi.to(dev))
    got.backward(gout.to(dev))
    got_grads = [q2.grad, s2.grad, r2.grad] + [p.grad for p in layer.parameters()]
    assert (got.cpu() - want).abs().max().item() <= 1e-4 * max(1.0, want.abs().max().item())
    for a, b in zip(got_grads, want_grads):
        assert (a.cpu() - b).abs().max().item() <= 2e-4 * max(1.0, b.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_packing_kernel(dtype):
    from ops3d_b200 import capi

    torch.manual_seed(1)
    dev = "cuda"
    shapes = torch.tensor([(4, 5, 6), (2, 3, 3), (1, 2, 2)], device=dev)
    B, Q, G, L, K = 2, 19, 3, 3, 4
    off = torch.randn(B, Q, G, L, K, 3, device=dev).to(dtype)
    ref = torch.rand(B, Q, L, 3, device=dev).to(dtype)
    logits = torch.randn(B, Q, G, L, K, device=dev).to(dtype)
    packed = capi.pack_sampling(off, ref, logits, shapes)
    extent = shapes.flip(-1).float()
    loc = ref.float()[:, :, None, :, None, :] + off.float() / extent[None, None, None, :, None, :]
    want = torch.cat([loc.reshape(B, Q, G, -1), logits.float().reshape(B, Q, G, -1)], -1)
    assert packed.dtype == torch.float32
    assert torch.allclose(packed, want, rtol=1e-6, atol=1e-6)


def test_fused_projection_bf16_matches_fp32_composition():
    """The one-GEMM projection + packing in bf16 against the fp32 composition on the same (bf16-rounded) tensors:
    coordinates to 2e-2 of a voxel-normalised unit, i.e. within the 16-bit tolerance of the operator's inputs, and
    the reference points themselves carried exactly (three 16-bit terms)."""
    from ops3d_b200.msda3d import project_and_pack

    torch.manual_seed(2)
    dev = "cuda"
    B, Q, C, G, L, K = 2, 50, 64, 4, 3, 4
    shapes = torch.tensor([(8, 16, 32), (4, 8, 16), (2, 4, 8)], device=dev)
    q = torch.randn(B, Q, C, device=dev).bfloat16()
    ref = torch.rand(B, Q, L, 3, device=dev)
    wo = (torch.randn(G * L * K * 3, C, device=dev) * 0.1).bfloat16()
    bo = torch.randn(G * L * K * 3, device=dev).bfloat16()
    wl = (torch.randn(G * L * K, C, device=dev) * 0.1).bfloat16()
    bl = torch.randn(G * L * K, device=dev).bfloat16()
    packed = project_and_pack(q, ref, wo, bo, wl, bl, shapes, G, K)
    off = (q.float() @ wo.float().t() + bo.float()).view(B, Q, G, L, K, 3)
    lg = (q.float() @ wl.float().t() + bl.float()).view(B, Q, G, L, K)
    loc = ref[:, :, None, :, None, :] + off / shapes.flip(-1).float()[None, None, None, :, None, :]
    want = torch.cat([loc.reshape(B, Q, G, -1), lg.reshape(B, Q, G, -1)], -1)
    assert packed.dtype == torch.float32 and packed.shape == want.shape
    assert (packed - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    # zero weights and biases: the packed coordinates are the reference points, to fp32 rounding
    z = project_and_pack(q, ref, wo * 0, bo * 0, wl * 0, bl * 0, shapes, G, K)
    want_ref = ref[:, :, None, :, None, :].expand(B, Q, G, L, K, 3).reshape(B, Q, G, -1)
    assert (z[..., : L * K * 3] - want_ref).abs().max().item() <= 3e-7
