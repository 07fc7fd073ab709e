"""ctypes front-end of the plain-C restatement in ``oracle/fda_oracle.c``.

TEST INFRASTRUCTURE ONLY (see the header of the C file).  Tensors in, tensors
out; everything is converted to contiguous fp32 / int64 on the CPU first.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfda_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "fda_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libfda_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(_LIB_PATH)
        p = ctypes.c_void_p
        i = ctypes.c_int
        lib.fda_oracle_forward.argtypes = [p, p, p, p, i, i, i, i, i, i, i, p]
        lib.fda_oracle_forward.restype = i
        lib.fda_oracle_backward.argtypes = [p, p, p, p, p, i, i, i, i, i, i, i, p, p]
        lib.fda_oracle_backward.restype = i
        _lib = lib
    return _lib


def _prep(value, shapes, lsi, packed):
    value = value.detach().cpu().float().contiguous()
    shapes = torch.as_tensor(shapes).cpu().long().contiguous()
    lsi = torch.as_tensor(lsi).cpu().long().contiguous()
    packed = packed.detach().cpu().float().contiguous()
    return value, shapes, lsi, packed


def forward(value, shapes, lsi, packed, K: int) -> torch.Tensor:
    value, shapes, lsi, packed = _prep(value, shapes, lsi, packed)
    B, N, G, D = value.shape
    Q, L = packed.shape[1], shapes.shape[0]
    assert packed.shape[-1] == L * K * 4
    out = torch.empty(B, Q, G * D)
    rc = _load().fda_oracle_forward(value.data_ptr(), shapes.data_ptr(), lsi.data_ptr(), packed.data_ptr(),
                                    B, N, G, D, L, K, Q, out.data_ptr())
    if rc:
        raise RuntimeError(f"fda_oracle_forward failed ({rc})")
    return out


def backward(value, shapes, lsi, packed, grad_out, K: int):
    value, shapes, lsi, packed = _prep(value, shapes, lsi, packed)
    grad_out = grad_out.detach().cpu().float().contiguous()
    B, N, G, D = value.shape
    Q, L = packed.shape[1], shapes.shape[0]
    grad_value = torch.empty_like(value)
    grad_packed = torch.empty_like(packed)
    rc = _load().fda_oracle_backward(value.data_ptr(), shapes.data_ptr(), lsi.data_ptr(), packed.data_ptr(),
                                     grad_out.data_ptr(), B, N, G, D, L, K, Q,
                                     grad_value.data_ptr(), grad_packed.data_ptr())
    if rc:
        raise RuntimeError(f"fda_oracle_backward failed ({rc})")
    return grad_value, grad_packed
