"""Shared pytest configuration: markers, import path, golden-fixture loader."""
import glob
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def _inject_reference_debug_function():
    """The reference package also exports its PyTorch implementation, ``ms_deform_attn_core_pytorch_3d``, and
    its tests import it from ``ops3d``.  The product package deliberately ships no PyTorch implementation of
    the operator; for the tests the CPU oracle's restatement is attached under the reference's names."""
    import ops3d
    import ops3d.flash_deform_attn
    from oracle.fda_oracle import ms_deform_attn_core_pytorch_3d

    ops3d.ms_deform_attn_core_pytorch_3d = ms_deform_attn_core_pytorch_3d
    ops3d.flash_deform_attn.ms_deform_attn_core_pytorch_3d = ms_deform_attn_core_pytorch_3d


_inject_reference_debug_function()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def golden_names():
    """Fixtures of the attention operator (made by the reference's PyTorch implementation)."""
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz"))
                  if not os.path.basename(p).startswith(("dcnv4_", "roi_align3d_", "nms3d_")))


def dcnv4_golden_names():
    """Fixtures of DCNv4-3D (made by the reference's CUDA kernels, tests/golden/make_golden_dcnv4.py)."""
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "dcnv4_*.npz")))


def load_dcnv4_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    d = {k: torch.from_numpy(z[k]) for k in ("value", "offset", "grad_out", "out")}
    d["backward_stored"] = bool(z["backward_stored"])   # False: the generator did not run the reference's backward
    if d["backward_stored"]:
        d.update({k: torch.from_numpy(z[k]) for k in ("grad_value", "grad_offset")})
    d["args"] = (tuple(int(v) for v in z["kernel"]), tuple(int(v) for v in z["stride"]), tuple(int(v) for v in z["pad"]),
                 tuple(int(v) for v in z["dilation"]), int(z["group"]), int(z["group_channels"]), float(z["offset_scale"]),
                 int(z["remove_center"]), bool(z["softmax"]))
    return d


def load_golden(name):
    """One fixture as a dict of CPU tensors (+ ints K, L and level_start_index)."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    d = {k: torch.from_numpy(z[k]) for k in ("value", "shapes", "packed", "grad_out", "out", "grad_value", "grad_packed")}
    d["K"] = int(z["K"])
    d["L"] = int(d["shapes"].shape[0])
    sizes = d["shapes"].prod(1)
    d["lsi"] = torch.cat((sizes.new_zeros(1), sizes.cumsum(0)[:-1]))
    return d


@pytest.fixture
def fda_env():
    """``fda_env(NAME="value", ...)`` sets ``FDA_*`` knobs for one test and makes the library re-read them
    (it reads its environment once, when loaded); everything is restored afterwards."""
    from ops3d_b200 import capi

    saved = {}

    def set_knobs(**knobs):
        for name, val in knobs.items():
            if name not in saved:
                saved[name] = os.environ.get(name)
            if val is None:
                os.environ.pop(name, None)
            else:
                os.environ[name] = str(val)
        capi.reload_config()

    yield set_knobs
    for name, old in saved.items():
        if old is None:
            os.environ.pop(name, None)
        else:
            os.environ[name] = old
    capi.reload_config()


def detection_golden(prefix):
    """Fixtures of ROI-Align 3D (``roi_align3d_``) or NMS 3D (``nms3d_``), made by the reference's CUDA kernels
    (tests/golden/make_golden_detection.py): ``[(name, dict of numpy arrays)]``."""
    out = []
    for path in sorted(glob.glob(os.path.join(GOLDEN_DIR, prefix + "*.npz"))):
        z = np.load(path)
        out.append((os.path.basename(path)[:-4], {k: z[k] for k in z.files}))
    return out
