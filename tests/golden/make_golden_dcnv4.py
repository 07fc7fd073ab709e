"""Generates ``dcnv4_*.npz`` by running the REFERENCE's own DCNv4-3D CUDA kernels on a GPU.

The reference has no Python, CPU or test code for this operator, so its kernels are the only executable
statement of it.  They are compiled unmodified for sm_100a from the reference checkout
(``baseline/build_ref_cuda.sh <checkout> --dcnv4`` -> ``baseline/_ref/ops3d_ref_dcnv4.so``, git-ignored) and fed
seeded fp32 inputs; inputs and outputs are stored so that ``tests/test_oracle.py`` can pin the CPU oracle
(``oracle/dcnv4_oracle.py``) and ``tests/test_gpu_dcnv4.py`` the kernels of this repository to them:

    python tests/golden/make_golden_dcnv4.py --out <dir>          (on a machine with a GPU and the built .so)

    value [B,D,H,W,G*Dg] f32, offset [B,Do,Ho,Wo,padded] f32, grad_out, config (ints / floats),
    out, backward_stored and, where that is 1, grad_value, grad_offset

Only this script and the reference's binary are involved: nothing of this repository's kernels or oracle computes
the stored outputs (the oracle module is used for its seeded input generator alone).  The reference supports
3x3x3 stencils only (K = 27, or 26 with remove_center; csrc/cuda/dcnv4_im2col_cuda.cuh:418-445).
"""
import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

# name, B, (Din,Hin,Win), G, Dg, stride, pad, dilation, remove_center, softmax, offset_scale, run the reference's backward
#
# The last column: with soft-maxed masks and a channel-lane count that divides 32, the reference takes
# backward_kernel_dcn_warp_primitive, whose soft-max backward block sits INSIDE the outermost stencil loop
# (csrc/cuda/dcnv4_col2im_cuda.cuh:520-533: it runs after every kernel_w step, sums cache entries that were never
# written and advances the output pointer by K each time, i.e. up to 2K floats past the group's mask slots -- for the
# last group of the last cell that is past the end of grad_offset).  Its result is garbage and the store is out of
# bounds, so the reference's backward is NOT run on such a case: it pins ``out`` only.  The soft-max backward is pinned
# by the cases whose 12 channel lanes (48 channels / 4) select backward_kernel_dcn, where the block follows the loops
# (:225-237).
CASES = [
    ("dcnv4_k27_softmax", 2, (5, 6, 7), 4, 16, (1, 1, 1), (1, 1, 1), (1, 1, 1), 0, True, 0.37, False),
    ("dcnv4_k26_plain", 1, (6, 5, 8), 2, 32, (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, False, 0.73, True),
    ("dcnv4_k27_stride2_dil2", 2, (8, 7, 9), 4, 16, (2, 2, 2), (2, 2, 2), (2, 2, 2), 0, False, 1.0, True),
    ("dcnv4_k27_softmax_d48", 1, (5, 5, 6), 2, 48, (1, 1, 1), (1, 1, 1), (1, 1, 1), 0, True, 0.5, True),
    ("dcnv4_k26_softmax_d48", 1, (4, 6, 5), 2, 48, (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, True, 0.81, True),
]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--lib", default=os.path.join(ROOT, "baseline", "_ref", "ops3d_ref_dcnv4.so"))
    args = ap.parse_args()
    from oracle import dcnv4_oracle as gen  # seeded input generator only

    spec = importlib.util.spec_from_file_location("ops3d_ref_dcnv4", args.lib)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    os.makedirs(args.out, exist_ok=True)
    kernel = (3, 3, 3)
    for name, B, size_in, G, Dg, stride, pad, dilation, rc, softmax, scale, run_backward in CASES:
        value, rows, grad_out = gen.make_inputs(B, size_in, G, Dg, kernel, stride, pad, dilation, rc, seed=11)
        rows = gen.keep_positions_off_the_grid(rows, size_in, kernel, stride, pad, dilation, G, scale, rc)
        v, o, go = value.cuda(), rows.cuda(), grad_out.cuda()
        d_stride = 4                      # fp32: 16-byte transfers
        block_thread = (Dg // d_stride) * G   # one (batch, cell) per block: no block straddles two batch elements
        out = ref.dcnv4_forward(v, o, *kernel, *stride, *pad, *dilation, G, Dg, scale, 64, rc, d_stride, block_thread, softmax)
        stored = dict(
            value=value.numpy(), offset=rows.numpy(), grad_out=grad_out.numpy(),
            size_in=np.array(size_in), group=np.int64(G), group_channels=np.int64(Dg), kernel=np.array(kernel),
            stride=np.array(stride), pad=np.array(pad), dilation=np.array(dilation), remove_center=np.int64(rc),
            softmax=np.int64(int(softmax)), offset_scale=np.float64(scale), backward_stored=np.int64(int(run_backward)),
            out=out.cpu().numpy())
        if run_backward:
            assert not (softmax and 32 % (Dg // d_stride) == 0), "the reference's warp-primitive soft-max backward stores out of bounds"
            gv, goff = ref.dcnv4_backward(v, o, *kernel, *stride, *pad, *dilation, G, Dg, scale, 64, go, rc, d_stride,
                                          block_thread, softmax)
            stored.update(grad_value=gv.float().cpu().numpy(), grad_offset=goff.float().cpu().numpy())
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(args.out, name + ".npz"), **stored)
        print(f"{name}: out|max|={out.abs().max().item():.4f}" + (
            f" grad_value|max|={gv.abs().max().item():.4f} grad_offset|max|={goff.abs().max().item():.4f}" if run_backward else ""))


if __name__ == "__main__":
    main()
