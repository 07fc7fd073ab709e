"""Pins the CPU oracle (both restatements) to fixtures produced by the reference itself."""
import pytest
import torch

from conftest import golden_names, load_golden
from oracle import c_oracle, fda_oracle


@pytest.mark.parametrize("name", golden_names())
def test_torch_restatement_matches_reference_fixture(name):
    g = load_golden(name)
    out, gv, gp = fda_oracle.fused_forward_backward(g["value"], g["shapes"], g["packed"], g["grad_out"], g["K"])
    assert torch.allclose(out, g["out"], rtol=0, atol=2e-6)
    assert torch.allclose(gv, g["grad_value"], rtol=1e-5, atol=2e-6)
    assert torch.allclose(gp, g["grad_packed"], rtol=1e-5, atol=2e-5)


@pytest.mark.parametrize("name", golden_names())
def test_torch_restatement_chunked_equals_unchunked(name):
    g = load_golden(name)
    a = fda_oracle.fused_forward_backward(g["value"], g["shapes"], g["packed"], g["grad_out"], g["K"], chunk=7)
    b = fda_oracle.fused_forward_backward(g["value"], g["shapes"], g["packed"], g["grad_out"], g["K"])
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-5)
    assert torch.allclose(fda_oracle.fused_forward(g["value"], g["shapes"], g["packed"], g["K"], chunk=5), b[0], atol=2e-6)


@pytest.mark.parametrize("name", golden_names())
def test_c_restatement_matches_reference_fixture(name):
    g = load_golden(name)
    out = c_oracle.forward(g["value"], g["shapes"], g["lsi"], g["packed"], g["K"])
    gv, gp = c_oracle.backward(g["value"], g["shapes"], g["lsi"], g["packed"], g["grad_out"], g["K"])
    # fp32 max-abs bound of the operator's parity contract is 1e-4; the C loops
    # (double accumulation) sit far inside it.
    assert (out - g["out"]).abs().max() <= 5e-6
    assert (gv - g["grad_value"]).abs().max() <= 2e-5
    scale = g["grad_packed"].abs().max().clamp_min(1.0)
    assert (gp - g["grad_packed"]).abs().max() <= 2e-5 * scale


def test_known_answers():
    """Closed-form cases (no reference needed): constant volume, voxel centres, zero value."""
    shapes = torch.tensor([[3, 4, 5]])
    lsi = torch.zeros(1, dtype=torch.long)
    B, G, D, K, L, Q = 1, 2, 8, 4, 1, 6
    N = 60
    gen = torch.Generator().manual_seed(3)
    # all sampling points strictly inside [0.5/S, 1-0.5/S]: interpolation weights sum to 1
    loc = torch.rand(B, Q, G, L, K, 3, generator=gen) * 0.5 + 0.25
    logits = torch.randn(B, Q, G, L, K, generator=gen)
    packed = fda_oracle.pack_loc_attn(loc, logits)
    const = torch.full((B, N, G, D), 2.5)
    for fwd in (lambda v: fda_oracle.fused_forward(v, shapes, packed, K),
                lambda v: c_oracle.forward(v, shapes, lsi, packed, K)):
        assert torch.allclose(fwd(const), torch.full((B, Q, G * D), 2.5), atol=1e-5)
        assert fwd(torch.zeros(B, N, G, D)).abs().max() == 0
    # every point on the centre of voxel (z=1,y=2,x=3): out = value[voxel]
    centre = torch.tensor([(3 + 0.5) / 5, (2 + 0.5) / 4, (1 + 0.5) / 3])
    loc_c = centre.expand(B, Q, G, L, K, 3).contiguous()
    packed_c = fda_oracle.pack_loc_attn(loc_c, logits)
    value = torch.randn(B, N, G, D, generator=gen)
    want = value[:, (1 * 4 + 2) * 5 + 3].reshape(B, 1, G * D).expand(B, Q, G * D)
    assert torch.allclose(fda_oracle.fused_forward(value, shapes, packed_c, K), want, atol=1e-5)
    assert torch.allclose(c_oracle.forward(value, shapes, lsi, packed_c, K), want, atol=1e-5)


def test_dcnv4_oracle_known_answers():
    """The DCNv4-3D oracle on cases with a closed-form answer: a 3x3x3 stencil whose mask selects the centre point
    reproduces the input; an extra offset of one voxel along x shifts it (zero beyond the edge); soft-maxed equal
    masks over a constant volume give the constant away from the border."""
    from oracle import dcnv4_oracle as o

    B, size, G, Dg = 1, (4, 5, 6), 2, 8
    k, s, p, d = (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1)
    v, rows, _ = o.make_inputs(B, size, G, Dg, k, s, p, d, 0, seed=1)
    pts = o.stencil_points(k, 0)
    K, c = len(pts), pts.index((1, 1, 1))
    assert K == 27 and rows.shape[-1] == 216 and o.output_size(size, k, s, p, d) == size
    rows.zero_()
    body = rows[..., : G * K * 4].reshape(B, *size, G, K * 4)
    body[..., 3 * K + c] = 1.0
    out = o.dcnv4_forward(v, rows, k, s, p, d, G, Dg, 1.0, 0, False)
    assert (out - v).abs().max().item() < 1e-6
    body[..., 3 * c] = 1.0
    out = o.dcnv4_forward(v, rows, k, s, p, d, G, Dg, 1.0, 0, False)
    assert (out[:, :, :, :-1] - v[:, :, :, 1:]).abs().max().item() < 1e-6 and out[:, :, :, -1].abs().max().item() == 0
    rows.zero_()
    out = o.dcnv4_forward(torch.full_like(v, 2.0), rows, k, s, p, d, G, Dg, 1.0, 1, True)
    assert len(o.stencil_points(k, 1)) == 26
    assert (out[:, 1:-1, 1:-1, 1:-1] - 2.0).abs().max().item() < 1e-6


def test_detection_oracles_known_answers():
    """NMS oracle on the reference's own known-answer cases (reference tests/test_nms.py:17-50) and ROI-Align oracle on
    closed-form cases: a constant volume pools to the constant; the backward of ones spreads exactly one unit per output
    element while every sample lies inside the volume."""
    import numpy as np

    from oracle import detection_oracle as o

    boxes = np.tile(np.array([0, 0, 0, 100, 100, 100], np.float32), (1000, 1))
    scores = np.zeros(1000, np.float32)
    scores[0] = 0.9
    assert o.nms3d(boxes, scores, 0.1) == [0]
    two = np.array([[0, 0, 0, 10, 10, 10], [20, 20, 20, 30, 30, 30]], np.float32)
    assert o.nms3d(two, np.array([0.6, 0.7], np.float32), 0.5) == [1, 0]
    assert abs(o.iou3d([0, 0, 0, 2, 2, 2], [1, 1, 1, 3, 3, 3]) - 1 / 15) < 1e-6
    feats = np.full((1, 2, 4, 5, 6), 3.0)
    rois = np.array([[0, 0.5, 0.5, 0.5, 4.2, 3.7, 2.9]], np.float32)
    for order in (0, 1):
        out = o.roi_align3d_forward(feats, rois, (2, 2, 2), 1.0, 2, order)
        assert np.abs(out - 3.0).max() < 1e-9
        grad = o.roi_align3d_backward(np.ones((1, 2, 2, 2, 2)), rois, (1, 2, 4, 5, 6), 1.0, 2, order)
        assert abs(grad.sum() - 16.0) < 1e-9
    # a roi of one voxel around a cell centre returns that cell (nearest and linear agree at integer positions)
    vol = np.arange(2 * 3 * 4 * 5, dtype=np.float64).reshape(1, 2, 3, 4, 5)
    roi = np.array([[0, 1.5, 0.5, 0.5, 2.5, 1.5, 1.5]], np.float32)   # x in [1.5,2.5] -> sample at x = 2, y = 1, z = 1
    for order in (0, 1):
        out = o.roi_align3d_forward(vol, roi, (1, 1, 1), 1.0, 1, order)
        assert np.allclose(out[0, :, 0, 0, 0], vol[0, :, 1, 1, 2])


def test_dcnv4_oracle_matches_reference_kernel_outputs():
    """The DCNv4-3D oracle against what the reference's own CUDA kernels produced on a B200 (fp32; fixtures and their
    generator in tests/golden/).  One case stores the forward only: the reference's backward is not run on it (a defect
    of its warp-primitive soft-max backward, see the generator); the soft-max backward is pinned by the other cases."""
    from conftest import dcnv4_golden_names, load_dcnv4_golden
    from oracle import dcnv4_oracle as o

    names = dcnv4_golden_names()
    assert len(names) >= 5
    pinned_softmax_backward = False
    for name in names:
        g = load_dcnv4_golden(name)
        out, gv, goff = o.dcnv4_forward_backward(g["value"], g["offset"], g["grad_out"], *g["args"])
        assert (out - g["out"]).abs().max().item() <= 2e-5 * max(1.0, g["out"].abs().max().item())
        if g["backward_stored"]:
            assert (gv - g["grad_value"]).abs().max().item() <= 2e-5 * max(1.0, g["grad_value"].abs().max().item())
            assert (goff - g["grad_offset"]).abs().max().item() <= 2e-5 * max(1.0, g["grad_offset"].abs().max().item())
            pinned_softmax_backward |= g["args"][-1]
    assert pinned_softmax_backward


def test_detection_oracles_match_reference_kernel_outputs():
    """ROI-Align 3D and NMS 3D oracles against what the reference's own CUDA kernels produced on a B200."""
    import numpy as np

    from conftest import detection_golden
    from oracle import detection_oracle as o

    rois = detection_golden("roi_align3d_")
    assert len(rois) >= 3 and {int(z["order"]) for _, z in rois} == {0, 1}
    for name, z in rois:
        size = tuple(int(v) for v in z["output_size"])
        scale, ratio, order = float(z["spatial_scale"]), int(z["sampling_ratio"]), int(z["order"])
        out = o.roi_align3d_forward(z["features"], z["rois"], size, scale, ratio, order)
        grad = o.roi_align3d_backward(z["grad_out"], z["rois"], z["features"].shape, scale, ratio, order)
        assert np.abs(out - z["out"]).max() <= 2e-6, name
        assert np.abs(grad - z["grad_features"]).max() <= 5e-6, name
    nms = detection_golden("nms3d_")
    assert len(nms) >= 3
    for name, z in nms:
        assert o.nms3d(z["boxes"], z["scores"], float(z["threshold"])) == z["keep"].tolist(), name


@pytest.mark.parametrize("coords", ["uniform", "clustered"])
def test_grad_value_is_zero_outside_the_corner_rows_of_the_points(coords):
    """The rule behind the sparse handling of the gradient image (zero and convert only the rows that points touch): the
    oracle's grad_value is exactly zero in every head row that is not one of the 8 corner cells of some sampling point of
    that head, with the corners taken as the kernels take them (voxel = ((2*loc - 1 + 1) * size - 1) / 2 rounded step by
    step in fp32, floor, index inside the level)."""
    import numpy as np

    shapes = [(6, 7, 9), (3, 4, 5)]
    B, Q, G, D, K = 2, 5, 3, 8, 4
    value, sh, lsi, packed, grad_out = fda_oracle.make_inputs(shapes, B, Q, G, D, K, seed=47, coords=coords, lo=-0.2, hi=1.2)
    _, gv, _ = fda_oracle.fused_forward_backward(value, sh, packed, grad_out, K)
    L = len(shapes)
    loc = packed[..., : 3 * L * K].reshape(B, Q, G, L, K, 3).numpy().astype(np.float32)
    touched = np.zeros((B, value.shape[1], G), dtype=bool)
    one, half = np.float32(1.0), np.float32(0.5)
    for l, (Dz, H, W) in enumerate(shapes):
        vox = []
        for axis, size in ((0, W), (1, H), (2, Dz)):   # packed order is x, y, z
            g = np.float32(2.0) * loc[:, :, :, l, :, axis] - one
            vox.append(((g + one) * np.float32(size) - one) * half)
        x0, y0, z0 = (np.floor(v).astype(np.int64) for v in vox)
        b_idx, _, g_idx, _ = np.meshgrid(np.arange(B), np.arange(Q), np.arange(G), np.arange(K), indexing="ij")
        for dz in (0, 1):
            for dy in (0, 1):
                for dx in (0, 1):
                    x, y, z = x0 + dx, y0 + dy, z0 + dz
                    ok = (x >= 0) & (x < W) & (y >= 0) & (y < H) & (z >= 0) & (z < Dz)
                    cell = int(lsi[l]) + (z * H + y) * W + x
                    touched[b_idx[ok], cell[ok], g_idx[ok]] = True
    support = (gv != 0).any(dim=-1).numpy()
    assert support.any() and not touched.all()
    assert not (support & ~touched).any()
    assert touched.sum() <= B * Q * G * L * K * 8
