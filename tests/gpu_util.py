"""Helpers shared by the GPU parity tests (torch only supplies device memory here)."""
import ctypes as C

import numpy as np
import torch

from nectarml_b200 import _lib, _nectarml
from nectarml_b200.ops import ConvGeometry

DEV = "cuda:0"
F32, F16 = _nectarml.DType.Float32, _nectarml.DType.Float16


def geometry(case):
    transposed, geom, _, _ = case
    B, Ci, H, W, Co, KH, KW, s, p, d, op = geom
    return ConvGeometry(B, Ci, H, W, Co, KH, KW, tuple(s), tuple(p), tuple(d), tuple(op), transposed)


def dev(a, dtype=torch.float32, nhwc=False):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dtype)
    if nhwc:
        t = t.permute(0, 2, 3, 1)
    return t.contiguous()


def host(t, nhwc=False):
    if nhwc:
        t = t.permute(0, 3, 1, 2)
    return t.float().cpu().numpy()


def fetch(ptr, shape, dtype=np.float32):
    """Reads a result pointer of the reference-shaped API back to the host and releases it."""
    out = np.empty(shape, dtype)
    _lib.check(_lib.load().nml_debug_copy_to_host(out.ctypes.data_as(C.c_void_p), ptr, out.nbytes))
    _nectarml.free_cuda(ptr, out.size, None)
    return out


def rel_max(a, b):
    """max|a-b| / max|b| -- the norm the fp32 tolerance is stated in (elementwise relative error
    is meaningless at zero crossings)."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def assert_f32(a, b, what, tol=1e-5):
    r = rel_max(a, b)
    assert r <= tol, f"{what}: max|a-b|/max|b| = {r:.3e} > {tol:g}"


def assert_f16(a, b, what, rtol=1e-2, atol=1e-3):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    bad = np.abs(a - b) > atol + rtol * np.abs(b)
    assert not bad.any(), f"{what}: {int(bad.sum())} of {a.size} outside {rtol:g} rel / {atol:g} abs; " \
                          f"worst |a-b| = {np.abs(a - b).max():.3e}"
