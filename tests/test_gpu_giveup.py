"""The give-up path of the kernels, exercised without faulting, trapping or hanging the GPU.

Every wait inside the kernels is bounded: when it runs out the kernel records which wait it was in a
status word, unwinds (lets copies in flight land, frees TMEM) and returns, and the host learns of it
from `nml_device_status` (NML_ERR_DEVICE).  Two ways to make a wait run out on purpose:

* `nml_debug_wait_timeout`: one warp waits on an mbarrier that nothing ever arrives on, 1 ms limit;
* `nml_debug_stalled_linear_forward`: the contraction kernel itself on a small Linear layer whose
  activation boxes are encoded half as tall as the kernel expects, so no stage ever holds all its
  bytes; 2 ms limit.  This runs the kernel's own unwinding in every role.
Afterwards the context is intact and ordinary calls give correct results.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from nectarml_b200 import _lib, ops
from nectarml_b200.ops import ConvGeometry

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NML_ERR_DEVICE = 5
WAIT_CODES = {101, 102, 103, 104, 105}


def _status():
    code = C.c_int(0)
    st = _lib.load().nml_device_status(C.byref(code))
    return st, code.value


def _linear_still_correct():
    gen = torch.Generator(device=DEV).manual_seed(9)
    x = torch.randn(300, 128, device=DEV, generator=gen).half()
    w = (torch.randn(96, 128, device=DEV, generator=gen) * 0.1).half()
    y = ops.linear_forward(x, w)
    ops.device_status()
    assert torch.allclose(y.double(), x.double() @ w.double().t(), rtol=1e-2, atol=1e-3)


def test_bounded_wait_runs_out_and_is_reported_once():
    lib = _lib.load()
    assert _status() == (0, 0)
    assert lib.nml_debug_wait_timeout(1_000_000, 0, None) == 0
    st, code = _status()
    assert st == NML_ERR_DEVICE and code == 102
    assert b"102" in lib.nml_status_string(st)
    assert _status() == (0, 0), "the status word is cleared by the call that reported it"
    with pytest.raises(_lib.NectarB200Error):
        lib.nml_debug_wait_timeout(1_000_000, 0, None)
        ops.device_status()
    _linear_still_correct()


def test_static_entry_point_has_its_own_status_word():
    lib = _lib.load()
    assert lib.nml_conv_forward_static(None, None, None, None, None, None) == 0
    assert lib.nml_debug_wait_timeout(1_000_000, 1, None) == 0
    assert _status() == (0, 0), "a give-up under the static entry point is not reported into the ordinary word"
    st = lib.nml_conv_forward_static(None, None, None, None, None, None)
    assert st == NML_ERR_DEVICE and b"102" in lib.nml_status_string(st)
    assert lib.nml_conv_forward_static(None, None, None, None, None, None) == 0


def test_contraction_kernel_unwinds_when_its_operands_never_land():
    lib = _lib.load()
    rows, fin, fout = 512, 256, 128
    x = torch.randn(rows, fin, device=DEV).half()
    w = torch.randn(fout, fin, device=DEV).half()
    y = torch.full((rows, fout), 7.0, device=DEV, dtype=torch.float16)
    d = _lib.LinearDesc()
    d.rows, d.in_features, d.out_features = rows, fin, fout
    d.in_dtype = d.out_dtype = d.w_dtype = _lib.NML_F16
    d.math = _lib.NML_MATH_F16
    assert _status() == (0, 0)
    st = lib.nml_debug_stalled_linear_forward(C.byref(d), x.data_ptr(), w.data_ptr(), y.data_ptr(), None, 0,
                                              2_000_000, torch.cuda.current_stream().cuda_stream)
    assert st == 0, lib.nml_status_string(st)
    st, code = _status()  # synchronises: the kernel has returned by itself
    assert st == NML_ERR_DEVICE and code in WAIT_CODES, (st, code)
    assert bool((y == 7.0).all()), "a launch that gave up stores nothing"
    assert _status() == (0, 0)
    _linear_still_correct()
    # and a convolution through the same kernel family
    g = ConvGeometry(2, 32, 12, 12, 48, 3, 3, (1, 1), (1, 1))
    xc = torch.randn(2, 12, 12, 32, device=DEV).half()
    wc = (torch.randn(48, 32, 3, 3, device=DEV) * 0.1).half()
    yc = ops.conv_forward(g, xc, wc, None, layout="nhwc")
    ops.device_status()
    ref = torch.nn.functional.conv2d(xc.permute(0, 3, 1, 2).float(), wc.float(), padding=1).permute(0, 2, 3, 1)
    assert torch.allclose(yc.float(), ref, rtol=1e-2, atol=1e-3)
