"""ROI-Align 3D and NMS 3D kernels against their CPU oracles (``oracle/detection_oracle.py``) and the reference's own
known-answer tests for NMS (reference ``tests/test_nms.py:17-50``, same inputs, same expectations), through the
reference's import surface: ``ops3d._C.nms_3d``, ``ops3d.nms_nd``, ``ops3d.RoIAlign`` / ``roi_align_3d``."""
import numpy as np
import pytest
import torch

import ops3d
from conftest import detection_golden
from ops3d import _C
from oracle import detection_oracle as oracle

pytestmark = pytest.mark.gpu


def test_nms3d_suppresses_high_iou_duplicates():
    # one high-score box duplicated 1000x: all IoUs = 1, only the top-score box remains
    box0 = torch.tensor([0, 0, 0, 100, 100, 100], device="cuda", dtype=torch.float32)
    boxes = box0.unsqueeze(0).repeat(1000, 1)
    scores = torch.cat([torch.tensor([0.9], device="cuda"), torch.zeros(999, device="cuda")])
    keep = _C.nms_3d(boxes, scores, 0.1)
    assert keep.cpu().tolist() == [0]


def test_nms3d_keeps_non_overlapping_boxes():
    box_a = torch.tensor([0, 0, 0, 10, 10, 10], device="cuda", dtype=torch.float32)
    box_b = torch.tensor([20, 20, 20, 30, 30, 30], device="cuda", dtype=torch.float32)
    keep = _C.nms_3d(torch.stack([box_a, box_b]), torch.tensor([0.6, 0.7], device="cuda"), 0.5)
    assert set(keep.cpu().tolist()) == {0, 1} and keep.cpu().tolist() == [1, 0]  # decreasing score


@pytest.mark.parametrize("n,thr", [(1, 0.5), (63, 0.3), (64, 0.3), (65, 0.3), (300, 0.1), (1000, 0.25), (2500, 0.5)])
def test_nms3d_matches_oracle(n, thr):
    gen = torch.Generator().manual_seed(n)
    centre = torch.rand(n, 3, generator=gen) * 40
    size = torch.rand(n, 3, generator=gen) * 12 + 2
    boxes = torch.cat([centre - size / 2, centre + size / 2], 1)
    scores = torch.rand(n, generator=gen)
    keep = _C.nms_3d(boxes.cuda(), scores.cuda(), thr).cpu().tolist()
    assert keep == oracle.nms3d(boxes.numpy(), scores.numpy(), thr)
    kept2, dets = ops3d.nms_nd(torch.cat([boxes, scores[:, None]], 1).cuda(), thr)
    assert kept2.cpu().tolist() == keep and dets.shape == (n, 7)


def test_nms3d_empty_and_cpu_inputs():
    assert _C.nms_3d(torch.zeros(0, 6, device="cuda"), torch.zeros(0, device="cuda"), 0.5).numel() == 0
    with pytest.raises(RuntimeError):
        _C.nms_3d(torch.zeros(2, 6), torch.zeros(2), 0.5)


def _rois(n, N, D, H, W, seed):
    gen = torch.Generator().manual_seed(seed)
    lo = torch.rand(n, 3, generator=gen) * torch.tensor([W, H, D]) * 0.6 - 1.0     # some start outside the volume
    ext = torch.rand(n, 3, generator=gen) * torch.tensor([W, H, D]) * 0.7 + 0.3
    batch = torch.randint(0, N, (n, 1), generator=gen).float()
    return torch.cat([batch, lo, lo + ext], 1)


@pytest.mark.parametrize("order", [1, 0])
@pytest.mark.parametrize("sampling_ratio", [2, 0])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_roi_align3d_matches_oracle(dtype, sampling_ratio, order):
    N, C, D, H, W = 2, 5, 6, 7, 9
    torch.manual_seed(4)
    feats = torch.randn(N, C, D, H, W)
    rois = _rois(7, N, D, H, W, seed=5)
    out_size, scale = (2, 3, 2), 0.5 if dtype == torch.float32 else 1.0
    f = feats.to(dtype).cuda().requires_grad_(True)
    r = rois.to(dtype)  # the forward reads rois in the features' dtype, as the reference does
    out = ops3d.roi_align_3d(f, r.cuda(), out_size, scale, sampling_ratio, order)
    gout = torch.randn(out.shape)
    out.backward(gout.to(dtype).cuda())
    want = oracle.roi_align3d_forward(f.detach().float().cpu().numpy(), r.float().numpy(), out_size, scale, sampling_ratio, order)
    want_g = oracle.roi_align3d_backward(gout.to(dtype).float().numpy(), r.float().numpy(), (N, C, D, H, W), scale, sampling_ratio, order)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert out.shape == (7, C) + out_size and out.dtype == dtype
    assert np.abs(out.detach().float().cpu().numpy() - want).max() <= tol * max(1.0, np.abs(want).max())
    assert np.abs(f.grad.float().cpu().numpy() - want_g).max() <= tol * max(1.0, np.abs(want_g).max())


def test_roi_align_module_and_binding_contract():
    """``ops3d.RoIAlign`` (order passed at call time; nearest uses one sample per bin) and the raw binding's
    caller-allocated tensors."""
    N, C, D, H, W = 1, 3, 5, 5, 5
    feats = torch.randn(N, C, D, H, W, device="cuda")
    rois = torch.tensor([[0, 0.0, 0.0, 0.0, 4.0, 4.0, 4.0], [0, 1.0, 2.0, 0.5, 3.5, 4.5, 2.5]], device="cuda")
    layer = ops3d.RoIAlign((2, 2, 2), 1.0, sampling_ratio=2)
    for order in (1, 0):
        got = layer(feats, rois, order=order)
        want = oracle.roi_align3d_forward(feats.cpu().numpy(), rois.cpu().numpy(), (2, 2, 2), 1.0, 1 if order == 0 else 2, order)
        assert np.abs(got.cpu().numpy() - want).max() <= 1e-5
    out = torch.full((2, C, 2, 2, 2), 7.0, device="cuda")
    _C.roi_align_3d_forward(feats, rois, out, 2, 2, 2, 1.0, 2, 1)
    assert torch.equal(out, layer(feats, rois, order=1))
    grad_in = torch.zeros(N, C, D, H, W, device="cuda")
    _C.roi_align_3d_backward(torch.ones_like(out), rois, grad_in, 2, 2, 2, 1.0, 2, 1)
    assert abs(grad_in.sum().item() - out.numel()) <= 1e-3  # interpolation weights of in-range samples sum to one
    with pytest.raises(RuntimeError):
        _C.roi_align_3d_forward(feats, rois[:, :6].contiguous(), out, 2, 2, 2, 1.0, 2, 1)


@pytest.mark.parametrize("name,z", detection_golden("roi_align3d_"), ids=lambda v: v if isinstance(v, str) else "")
def test_roi_align3d_matches_reference_kernel_fixtures(name, z):
    size = tuple(int(v) for v in z["output_size"])
    scale, ratio, order = float(z["spatial_scale"]), int(z["sampling_ratio"]), int(z["order"])
    feats = torch.from_numpy(z["features"]).cuda().requires_grad_(True)
    out = ops3d.roi_align_3d(feats, torch.from_numpy(z["rois"]).cuda(), size, scale, ratio, order)
    out.backward(torch.from_numpy(z["grad_out"]).cuda())
    assert np.abs(out.detach().cpu().numpy() - z["out"]).max() <= 1e-5
    assert np.abs(feats.grad.cpu().numpy() - z["grad_features"]).max() <= 1e-4


@pytest.mark.parametrize("name,z", detection_golden("nms3d_"), ids=lambda v: v if isinstance(v, str) else "")
def test_nms3d_matches_reference_kernel_fixtures(name, z):
    keep = _C.nms_3d(torch.from_numpy(z["boxes"]).cuda(), torch.from_numpy(z["scores"]).cuda(), float(z["threshold"]))
    assert keep.cpu().tolist() == z["keep"].tolist()
