"""Generates the golden fixtures in this directory by running the REFERENCE package.

Run where the reference checkout is available (it is not on the GPU machines):

    python tests/golden/make_golden.py --reference /path/to/ops3d

It imports ``ops3d.ms_deform_attn_core_pytorch_3d`` from that checkout (the
reference's own CPU implementation of the operator, ``ops3d/flash_deform_attn.py:139-165``;
the package imports without its compiled extension), feeds it seeded inputs and
stores inputs and outputs as ``<case>.npz``:

    value [B,N,G,D] f32, shapes [L,3] i64, packed [B,Q,G,L*K*4] f32 (planar
    coords|logits), grad_out [B,Q,G*D] f32, K,
    out [B,Q,G*D], grad_value [B,N,G,D], grad_packed [B,Q,G,L*K*4]

Forward/backward follow the reference's own test recipe
(``tests/test_flash_deform_attn.py:106-136``): softmax over the flattened L*K
logits outside the oracle, autograd for the gradients.  Nothing of this repository
is imported here, so the fixtures are independent of the code they check.
"""
import argparse
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))

# name, shapes, B, Q, G, D, K, coords, value_rounding
CASES = [
    # BASELINE config 1: the CPU-plumbing case, fp32
    ("cfg1_fp32", [(4, 8, 8), (2, 4, 4)], 1, 288, 4, 16, 4, "uniform", None),
    # edge shapes of the reference's stress tests (tests/test_flash_deform_attn_stress.py:47-64)
    ("edge_l1_1x1x1_k4", [(1, 1, 1)], 1, 1, 2, 8, 4, "uniform", None),
    ("edge_l1_7x7x7_k8", [(7, 7, 7)], 1, 16, 2, 8, 8, "uniform", None),
    ("edge_l5_4x4x4_k4", [(4, 4, 4)] * 5, 1, 16, 2, 8, 4, "uniform", None),
    ("edge_aniso_l2_k4_b2", [(16, 8, 4), (8, 4, 2)], 2, 16, 2, 16, 4, "uniform", None),
    ("edge_uneven_l2_k8", [(1, 1, 1), (8, 8, 8)], 1, 16, 2, 8, 8, "uniform", None),
    # far out-of-range coordinates: whole points contribute nothing
    ("edge_far_oob_k4", [(4, 6, 8), (2, 3, 4)], 1, 32, 2, 8, 4, "wide", None),
    # down-scaled BASELINE config 2 (two levels, D=32, value rounded through bf16)
    ("cfg2_small_bf16value", [(4, 8, 16), (2, 4, 8)], 2, 48, 2, 32, 4, "uniform", "bf16"),
    # down-scaled BASELINE config 3 (cross-attention, clustered coordinates, 3 levels)
    ("cfg3_small_clustered", [(4, 8, 16), (2, 4, 8), (1, 2, 4)], 2, 20, 2, 32, 4, "clustered", "bf16"),
    # down-scaled BASELINE config 5 (three levels, K=8)
    ("cfg5_small_k8", [(4, 8, 16), (2, 4, 8), (1, 2, 4)], 2, 24, 2, 32, 8, "uniform", "bf16"),
]


def make_case(ref_fn, name, shapes, B, Q, G, D, K, coords, rounding, seed=0):
    gen = torch.Generator().manual_seed(seed)
    shapes_t = torch.tensor([list(s) for s in shapes], dtype=torch.long)
    L = len(shapes)
    N = int(shapes_t.prod(1).sum())
    value = torch.randn(B, N, G, D, generator=gen)
    if rounding == "bf16":
        value = value.bfloat16().float()
    if coords == "uniform":
        loc = torch.rand(B, Q, G, L, K, 3, generator=gen) * 1.1 - 0.05
    elif coords == "wide":
        loc = torch.rand(B, Q, G, L, K, 3, generator=gen) * 3.0 - 1.0
    else:
        centre = torch.rand(B, Q, 1, 1, 1, 3, generator=gen)
        loc = (centre + 0.05 * torch.randn(B, Q, G, L, K, 3, generator=gen)).clamp_(-0.05, 1.05)
    logits = torch.randn(B, Q, G, L, K, generator=gen)
    grad_out = torch.randn(B, Q, G * D, generator=torch.Generator().manual_seed(seed + 1))

    v = value.clone().requires_grad_(True)
    lc = loc.clone().requires_grad_(True)
    lg = logits.clone().requires_grad_(True)
    attn = F.softmax(lg.flatten(-2, -1), dim=-1).unflatten(-1, (L, K))
    out = ref_fn(v, shapes_t, lc, attn)
    out.backward(grad_out)
    packed = torch.cat([loc.reshape(B, Q, G, L * K * 3), logits.reshape(B, Q, G, L * K)], dim=-1)
    grad_packed = torch.cat([lc.grad.reshape(B, Q, G, L * K * 3), lg.grad.reshape(B, Q, G, L * K)], dim=-1)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        value=value.numpy(), shapes=shapes_t.numpy(), packed=packed.numpy(), grad_out=grad_out.numpy(),
        K=np.int64(K), out=out.detach().numpy(), grad_value=v.grad.numpy(), grad_packed=grad_packed.numpy(),
    )
    print(f"{name}: N={N} out|max|={out.abs().max():.4f}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout (contains ops3d/)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import ops3d  # the reference package; its compiled extension is not needed for this function

    assert os.path.realpath(os.path.dirname(ops3d.__file__)).startswith(os.path.realpath(args.reference))
    torch.set_num_threads(1)  # fixed summation order
    for case in CASES:
        make_case(ops3d.ms_deform_attn_core_pytorch_3d, *case)


if __name__ == "__main__":
    main()
