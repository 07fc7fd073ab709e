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


@pytest.mark.parametrize("K", [4, 8])
def test_layer_matches_pytorch_composition(K):
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
    layer = MSDeformAttn3D(C, 2, 4, K).to(dev)
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
