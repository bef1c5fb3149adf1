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


def _free_bytes():
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]  # cudaMemGetInfo: what the driver has left, not torch's cache


def test_static_scratch_forward_matches_workspace_forward_twice(oracle):
    first = ConvGeometry(4, 72, 20, 20, 40, 3, 3, (1, 1), (1, 1))
    second = ConvGeometry(2, 10, 9, 13, 24, 3, 3, (2, 2), (1, 1))  # smaller: lands on top of the first call's leftovers
    for g, seed, bias in ((first, 11, True), (second, 12, False)):
        got, ref = _run_both(g, seed, bias)
        assert np.isfinite(got).all()
        rel = np.abs(got.astype(np.float64) - ref).max() / np.abs(ref).max()
        assert rel <= 1e-5, f"static-scratch forward differs from the workspace forward: {rel:.3e}"
        rng = np.random.default_rng(seed)  # the same draws as _run_both
        x = rng.standard_normal(g.act_shape("in", "nchw"), dtype=np.float32)
        w = (rng.standard_normal(g.weight_shape(), dtype=np.float32) * 0.1).astype(np.float32)
        b = rng.standard_normal(g.c_out, dtype=np.float32) if bias else None
        want = oracle.conv2d(x, w, b, g.stride, g.padding, g.dilation)
        rel = np.abs(got.astype(np.float64) - want).max() / np.abs(want).max()
        assert rel <= 1e-5, f"static-scratch forward differs from the oracle: {rel:.3e}"


# (transposed, (B, C_in, H, W, C_out, KH, KW, stride, padding)): a transposed stride-2 layer producing 3 channels
# (phase-packed gather walk), a 4x4 stride-2 bottleneck layer with few pixels (K-split walk), an RGB stem (window walk)
FP16_NHWC_CASES = [
    (True, (2, 64, 9, 11, 3, 4, 4, (2, 2), (1, 1))),
    (False, (2, 256, 4, 4, 96, 4, 4, (2, 2), (1, 1))),
    (False, (2, 3, 30, 26, 64, 7, 7, (2, 2), (3, 3))),
]


@pytest.mark.parametrize("case", FP16_NHWC_CASES, ids=["convT_to_rgb", "k_split", "rgb_stem"])
def test_static_scratch_forward_fp16_nhwc_against_the_oracle(case, oracle):
    transposed, (B, Ci, H, W, Co, KH, KW, s, p) = case
    g = ConvGeometry(B, Ci, H, W, Co, KH, KW, s, p, transposed=transposed)
    rng = np.random.default_rng(21)
    r = oracle.round_f16
    x = r(rng.standard_normal((B, Ci, H, W), dtype=np.float32))
    w = r((rng.standard_normal(g.weight_shape(), dtype=np.float32) * 0.1).astype(np.float32))
    b = r(rng.standard_normal(Co, dtype=np.float32))
    want = (oracle.conv_transpose2d(x, w, b, s, p, (1, 1), (0, 0)) if transposed else oracle.conv2d(x, w, b, s, p, (1, 1)))
    xd = torch.from_numpy(x).to(DEV).half().permute(0, 2, 3, 1).contiguous()
    wd, bd = torch.from_numpy(w).to(DEV).half(), torch.from_numpy(b).to(DEV).half()
    d = g.desc(_lib.NML_F16, "nhwc", _lib.NML_F16, "nhwc", _lib.NML_F16, "f16", False)
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    free_before = None
    for call in range(2):
        out = torch.full(g.act_shape("out", "nhwc"), float("nan"), device=DEV, dtype=torch.float16)
        if call == 1:
            free_before = _free_bytes()
        st = lib.nml_conv_forward_static(C.byref(d), xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), out.data_ptr(), stream)
        assert st == 0, lib.nml_status_string(st)
        if call == 1:
            assert _free_bytes() == free_before, "the second call changed the amount of free device memory"
        outs.append(out)
    assert lib.nml_conv_forward_static(None, None, None, None, None, None) == 0
    assert torch.equal(outs[0], outs[1])
    got = outs[1].permute(0, 3, 1, 2).float().cpu().numpy()
    bad = np.abs(got - want) > 1e-3 + 1e-2 * np.abs(want)
    assert not bad.any(), f"{int(bad.sum())} of {got.size} outside 1e-2 rel / 1e-3 abs"


def test_layer_beyond_the_built_in_scratch_is_refused():
    g = ConvGeometry(64, 256, 128, 128, 256, 3, 3, (1, 1), (1, 1))  # 2 x 1 GiB of converted input
    d = g.desc(_lib.NML_F32, "nchw", _lib.NML_F32, "nchw", _lib.NML_F32, "3xtf32", False)
    lib = _lib.load()
    one = torch.zeros(1, device=DEV)  # never read: the size check comes before anything is launched
    st = lib.nml_conv_forward_static(C.byref(d), one.data_ptr(), one.data_ptr(), None, one.data_ptr(), None)
    assert st == 2
    msg = lib.nml_status_string(st).decode()
    assert "67108864" in msg and "scratch" in msg
