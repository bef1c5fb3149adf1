"""The forward entry point that allocates nothing (`nml_conv_forward_static`).

Some hosts cannot call cudaMalloc where they call this library -- a server whose own pool already
owns all free HBM, or a loop that cannot afford the device-wide synchronisation an allocation
implies -- so this variant keeps its conversion scratch in a 64 MiB array inside the library
image.  The test calls it through the C ABI twice in a row, the second time on a different layer
so that whatever the first call left in the shared scratch would show, and compares each result
with the ordinary entry point's.  It also checks that a layer too large for the built-in scratch
is refused with a message instead of being run.  This file is named to be collected last.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from nectarml_b200 import _lib, ops
from nectarml_b200.ops import ConvGeometry

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_both(g, seed, with_bias):
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.standard_normal(g.act_shape("in", "nchw"), dtype=np.float32)).to(DEV)
    w = torch.from_numpy((rng.standard_normal(g.weight_shape(), dtype=np.float32) * 0.1).astype(np.float32)).to(DEV)
    b = torch.from_numpy(rng.standard_normal(g.c_out, dtype=np.float32)).to(DEV) if with_bias else None
    ref = ops.conv_forward(g, x, w, b, math="3xtf32")  # existing entry point, caller workspace
    out = torch.full_like(ref, float("nan"))
    d = g.desc(_lib.NML_F32, "nchw", _lib.NML_F32, "nchw", _lib.NML_F32, "3xtf32", False)
    lib = _lib.load()
    st = lib.nml_conv_forward_static(C.byref(d), x.data_ptr(), w.data_ptr(), b.data_ptr() if b is not None else None,
                                     out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0, lib.nml_status_string(st)
    assert lib.nml_conv_forward_static(None, None, None, None, None, None) == 0  # no give-up recorded
    ops.device_status()
    return out.cpu().numpy(), ref.cpu().numpy()


def test_static_scratch_forward_matches_workspace_forward_twice():
    first = ConvGeometry(4, 72, 20, 20, 40, 3, 3, (1, 1), (1, 1))
    second = ConvGeometry(2, 10, 9, 13, 24, 3, 3, (2, 2), (1, 1))  # smaller: lands on top of the first call's leftovers
    for g, seed, bias in ((first, 11, True), (second, 12, False)):
        got, ref = _run_both(g, seed, bias)
        assert np.isfinite(got).all()
        rel = np.abs(got.astype(np.float64) - ref).max() / np.abs(ref).max()
        assert rel <= 1e-5, f"static-scratch forward differs from the workspace forward: {rel:.3e}"


def test_layer_beyond_the_built_in_scratch_is_refused():
    g = ConvGeometry(64, 256, 128, 128, 256, 3, 3, (1, 1), (1, 1))  # 2 x 1 GiB of converted input
    d = g.desc(_lib.NML_F32, "nchw", _lib.NML_F32, "nchw", _lib.NML_F32, "3xtf32", False)
    lib = _lib.load()
    one = torch.zeros(1, device=DEV)  # never read: the size check comes before anything is launched
    st = lib.nml_conv_forward_static(C.byref(d), one.data_ptr(), one.data_ptr(), None, one.data_ptr(), None)
    assert st == 2
    msg = lib.nml_status_string(st).decode()
    assert "67108864" in msg and "scratch" in msg
