"""Full-size checks (the benchmark's largest configuration: 256x512x2048 tile at strides 8/16/32, B=2,
N=Lq=598016, G=8, D=32, K=8, bf16 value, fp32 offsets) through properties that need no oracle run:

* interpolation and soft-max weights each sum to one, so with all sampling points strictly inside the
  volume a constant value field c gives out == c, zero coordinate gradients and zero logit gradients;
* for the same reason the column sums of grad_value equal the column sums of grad_output per
  (batch, head, channel) -- a checksum of checksums over 230 M sampling points and 1.8 G scattered rows;
* soft-max backward: the logit gradients of every row sum to zero;
* linearity in value: forward(v1 + v2) == forward(v1) + forward(v2).

This is also the only place where the slab-binned backward runs on its real workload (the gradient
image of one batch element, 612 MB, exceeds L2).
"""
import pytest
import torch

from ops3d_b200 import capi

pytestmark = pytest.mark.gpu

SHAPES = [(32, 64, 256), (16, 32, 128), (8, 16, 64)]
B, G, D, K = 2, 8, 32, 8
L = len(SHAPES)


@pytest.fixture(scope="module")
def problem():
    if torch.cuda.get_device_properties(0).total_memory < 40e9:
        pytest.skip("needs a GPU with > 40 GB")
    dev = torch.device("cuda")
    shapes = torch.tensor(SHAPES, dtype=torch.long, device=dev)
    sizes = shapes.prod(1)
    lsi = torch.cat((sizes.new_zeros(1), sizes.cumsum(0)[:-1]))
    N = int(sizes.sum())
    Q = N
    gen = torch.Generator(device=dev).manual_seed(5)
    packed = torch.empty(B, Q, G, L * K * 4, device=dev)
    # strictly interior for the smallest extent (8): x*S - 0.5 in [0, S-1]  <=>  x in [0.0625, 0.9375]
    packed[..., : L * K * 3] = torch.rand(B, Q, G, L * K * 3, generator=gen, device=dev) * 0.86 + 0.07
    packed[..., L * K * 3:] = torch.randn(B, Q, G, L * K, generator=gen, device=dev)
    grad_out = torch.randn(B, Q, G * D, generator=gen, device=dev).bfloat16()
    return dict(dev=dev, shapes=shapes, lsi=lsi, N=N, Q=Q, packed=packed, grad_out=grad_out, gen=gen)


def test_constant_field_and_gradient_checksums(problem):
    p = problem
    value = torch.full((B, p["N"], G, D), 1.5, dtype=torch.bfloat16, device=p["dev"])
    out = capi.forward(value, p["shapes"], p["lsi"], p["packed"], K)
    assert (out.float() - 1.5).abs().max().item() <= 1.5 * 2 ** -7  # one bf16 rounding of a sum of weights ~ 1
    del out
    assert capi.scratch_bytes(value, p["packed"], K) > 0  # the slab-binned path is what runs here
    gv, gp = capi.backward(value, p["shapes"], p["lsi"], p["packed"], p["grad_out"], K)
    torch.cuda.synchronize()
    # constant field: every sample equals c, so d out / d coordinate = 0 and d out / d logit = 0
    go_scale = p["grad_out"].float().abs().max().item()
    assert gp.abs().max().item() <= 2e-2 * go_scale * 256  # coordinate gradients carry a factor of the level size
    assert gp[..., : L * K * 3].abs().mean().item() <= 1e-3
    assert gp[..., L * K * 3:].abs().max().item() <= 1e-4 * go_scale * D
    # column sums: sum_n grad_value[b, n, g, d] == sum_q grad_out[b, q, g, d]
    want = p["grad_out"].float().view(B, p["Q"], G, D).double().sum(1)
    got = gv.double().sum(1)
    rms = want.pow(2).mean().sqrt().item()
    assert (got - want).abs().max().item() <= 2e-2 * rms  # bf16 rounding of 598016 cells per column
    # and nothing is wildly off anywhere: the largest element is bounded by the number of contributions
    assert torch.isfinite(gv.float()).all()


def test_logit_gradients_sum_to_zero_and_forward_is_linear(problem):
    p = problem
    gen = p["gen"]
    v1 = torch.randn(B, p["N"], G, D, generator=gen, device=p["dev"]).bfloat16()
    v2 = torch.randn(B, p["N"], G, D, generator=gen, device=p["dev"]).bfloat16()
    o1 = capi.forward(v1, p["shapes"], p["lsi"], p["packed"], K).float()
    o2 = capi.forward(v2, p["shapes"], p["lsi"], p["packed"], K).float()
    v12 = (v1.float() + v2.float()).bfloat16()
    o12 = capi.forward(v12, p["shapes"], p["lsi"], p["packed"], K).float()
    # v1 + v2 is itself rounded to bf16 (relative 2^-9 per element) before the gather
    scale = o12.abs().max().item()
    assert (o12 - (o1 + o2)).abs().max().item() <= 2e-2 * scale
    del o1, o2, o12, v2, v12
    gv, gp = capi.backward(v1, p["shapes"], p["lsi"], p["packed"], p["grad_out"], K)
    torch.cuda.synchronize()
    logit_grads = gp[..., L * K * 3:]
    row_sums = logit_grads.sum(-1)
    assert row_sums.abs().max().item() <= 1e-3 * max(1.0, logit_grads.abs().max().item())
    assert torch.isfinite(gp).all() and torch.isfinite(gv.float()).all()
