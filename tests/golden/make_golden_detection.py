"""Generates ``roi_align3d_*.npz`` and ``nms3d_*.npz`` by running the REFERENCE's own CUDA kernels on a GPU.

The reference has no CPU path for ROI-Align 3D or NMS 3D, so its kernels are compiled unmodified for sm_100a from the
reference checkout (``baseline/build_ref_cuda.sh <checkout> --detection`` -> ``baseline/_ref/ops3d_ref_detection.so``,
git-ignored) and fed seeded fp32 inputs; inputs and outputs are stored so that ``tests/test_oracle.py`` can pin the
CPU oracles (``oracle/detection_oracle.py``) and ``tests/test_gpu_detection_ops.py`` this repository's kernels to them:

    python tests/golden/make_golden_detection.py --out <dir>      (on a machine with a GPU and the built .so)

Nothing of this repository computes the stored outputs.  NMS scores are distinct, so the reference's unstable sort
cannot reorder ties.
"""
import argparse
import importlib.util
import os

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

# name, N, C, (D, H, W), rois, output_size, spatial_scale, sampling_ratio, order
ROI_CASES = [
    ("roi_align3d_linear_s2", 2, 5, (6, 7, 9), 7, (2, 3, 2), 0.5, 2, 1),
    ("roi_align3d_linear_adaptive", 2, 3, (8, 8, 8), 6, (2, 2, 2), 1.0, 0, 1),
    ("roi_align3d_nearest", 1, 4, (5, 6, 7), 5, (3, 2, 2), 1.0, 1, 0),
]
NMS_CASES = [("nms3d_300", 300, 0.1), ("nms3d_1000", 1000, 0.25), ("nms3d_65", 65, 0.3)]


def rois_for(n, N, D, H, W, seed):
    gen = torch.Generator().manual_seed(seed)
    lo = torch.rand(n, 3, generator=gen) * torch.tensor([W, H, D]) * 0.6 - 1.0     # some start outside the volume
    ext = torch.rand(n, 3, generator=gen) * torch.tensor([W, H, D]) * 0.7 + 0.3
    batch = torch.randint(0, N, (n, 1), generator=gen).float()
    return torch.cat([batch, lo, lo + ext], 1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--lib", default=os.path.join(ROOT, "baseline", "_ref", "ops3d_ref_detection.so"))
    args = ap.parse_args()
    spec = importlib.util.spec_from_file_location("ops3d_ref_detection", args.lib)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    os.makedirs(args.out, exist_ok=True)
    for name, N, C, (D, H, W), n, osize, scale, ratio, order in ROI_CASES:
        gen = torch.Generator().manual_seed(17)
        feats = torch.randn(N, C, D, H, W, generator=gen)
        rois = rois_for(n, N, D, H, W, seed=19)
        gout = torch.randn(n, C, *osize, generator=gen)
        out = torch.zeros(n, C, *osize, device="cuda")
        ref.roi_align_3d_forward(feats.cuda(), rois.cuda(), out, *osize, scale, ratio, order)
        grad = torch.zeros(N, C, D, H, W, device="cuda")
        ref.roi_align_3d_backward(gout.cuda(), rois.cuda(), grad, *osize, scale, ratio, order)
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(args.out, name + ".npz"), features=feats.numpy(), rois=rois.numpy(), grad_out=gout.numpy(),
                            output_size=np.array(osize), spatial_scale=np.float64(scale), sampling_ratio=np.int64(ratio),
                            order=np.int64(order), out=out.cpu().numpy(), grad_features=grad.cpu().numpy())
        print(f"{name}: out|max|={out.abs().max().item():.4f} grad|max|={grad.abs().max().item():.4f}")
    for name, n, thr in NMS_CASES:
        gen = torch.Generator().manual_seed(n)
        centre = torch.rand(n, 3, generator=gen) * 40
        size = torch.rand(n, 3, generator=gen) * 12 + 2
        boxes = torch.cat([centre - size / 2, centre + size / 2], 1)
        scores = torch.randperm(n, generator=gen).float() / n      # distinct
        keep = ref.nms_3d(boxes.cuda(), scores.cuda(), thr)
        np.savez_compressed(os.path.join(args.out, name + ".npz"), boxes=boxes.numpy(), scores=scores.numpy(),
                            threshold=np.float64(thr), keep=keep.cpu().numpy())
        print(f"{name}: kept {keep.numel()} of {n}")


if __name__ == "__main__":
    main()
