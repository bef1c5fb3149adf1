"""CPU-only checks of the C ABI: the shared library loads, exports every function the header
declares, and its host-side logic (output sizes, workspace sizing, argument validation) works
without a GPU.  No compute call is made here."""
import ctypes as C
import os
import re
import subprocess

import pytest

from nectarml_b200 import _lib
from nectarml_b200.ops import ConvGeometry

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "nectarml_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nml_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_binding_expects():
    assert declared_functions() == sorted(_lib.SYMBOLS)


def test_library_exports_every_declared_symbol(lib):
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True,
                         check=True).stdout
    exported = set(re.findall(r"\sT\s+(nml_[a-z0-9_]+)", out))
    missing = [f for f in declared_functions() if f not in exported]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_status_strings(lib):
    assert lib.nml_status_string(0) == b"ok"
    assert b"workspace" in lib.nml_status_string(2)
    assert lib.nml_status_string(99) == b"unknown status"


@pytest.mark.parametrize("geom,expect", [
    (ConvGeometry(8, 64, 56, 56, 64, 3, 3, (1, 1), (1, 1)), (56, 56)),
    (ConvGeometry(256, 3, 224, 224, 64, 7, 7, (2, 2), (3, 3)), (112, 112)),
    (ConvGeometry(256, 1024, 14, 14, 2048, 1, 1, (2, 2)), (7, 7)),
    (ConvGeometry(64, 3, 256, 256, 64, 4, 4, (2, 2), (1, 1)), (128, 128)),
    (ConvGeometry(64, 128, 128, 128, 3, 4, 4, (2, 2), (1, 1), transposed=True), (256, 256)),
    (ConvGeometry(2, 8, 8, 8, 4, 3, 3, (2, 2), (1, 1), (1, 1), (1, 1), transposed=True), (16, 16)),
])
def test_output_size_matches_reference_formula(lib, oracle, geom, expect):
    assert geom.out_hw() == expect
    if geom.transposed:
        ref = oracle.conv_transpose_out_hw(geom.h, geom.w, geom.kh, geom.kw, geom.stride, geom.padding,
                                           geom.dilation, geom.output_padding)
    else:
        ref = oracle.conv_out_hw(geom.h, geom.w, geom.kh, geom.kw, geom.stride, geom.padding, geom.dilation)
    assert geom.out_hw() == ref


def test_invalid_geometry_is_rejected(lib):
    bad = ConvGeometry(1, 3, 2, 2, 4, 5, 5)  # kernel larger than the padded input
    d = bad.desc(0, "nchw", 0, "nchw", 0, "f16", False)
    ho, wo = C.c_int(), C.c_int()
    assert lib.nml_conv_output_size(C.byref(d), C.byref(ho), C.byref(wo)) == 1
    n = C.c_size_t()
    assert lib.nml_conv_workspace_size(C.byref(d), 0, C.byref(n)) == 1
    assert lib.nml_conv_workspace_size(None, 0, C.byref(n)) == 1


def test_workspace_sizes(lib):
    g = ConvGeometry(8, 64, 56, 56, 64, 3, 3, (1, 1), (1, 1))
    n = C.c_size_t()
    # native fp16 NHWC forward: only the repacked weights (64 x 9 taps x 64 ch x 2 B)
    d = g.desc(_lib.NML_F16, "nhwc", _lib.NML_F16, "nhwc", _lib.NML_F16, "f16", False)
    assert lib.nml_conv_workspace_size(C.byref(d), 0, C.byref(n)) == 0
    assert 64 * 9 * 64 * 2 <= n.value <= 64 * 9 * 64 * 2 + 1024
    # reference-shaped fp32 NCHW forward in 3xTF32: hi+lo planes of x and of the weights
    d = g.desc(_lib.NML_F32, "nchw", _lib.NML_F32, "nchw", _lib.NML_F32, "3xtf32", False)
    assert lib.nml_conv_workspace_size(C.byref(d), 0, C.byref(n)) == 0
    x_bytes = 8 * 64 * 56 * 56 * 4
    assert 2 * x_bytes <= n.value <= 2 * x_bytes + 2 * 64 * 9 * 64 * 4 + 4096
    # weight gradient converts both x and dy
    assert lib.nml_conv_workspace_size(C.byref(d), 2, C.byref(n)) == 0
    assert n.value >= 4 * x_bytes
    # native fp16 Linear: the operands are used in place; forward only sets aside room to widen
    # an fp16 bias to fp32
    ld = _lib.LinearDesc(4096, 512, 2048, _lib.NML_F16, _lib.NML_F16, _lib.NML_F16, _lib.NML_MATH_F16, 0)
    assert lib.nml_linear_workspace_size(C.byref(ld), 0, C.byref(n)) == 0
    assert n.value == 2048 * 4
    assert lib.nml_linear_workspace_size(C.byref(ld), 1, C.byref(n)) == 0
    assert n.value == 0
    # weight gradient: one fp32 plane of dW per K slice (the slices are added in a fixed order by a second
    # kernel) plus the rows of partial column sums behind the bias gradient
    assert lib.nml_linear_workspace_size(C.byref(ld), 2, C.byref(n)) == 0
    dw_bytes = 2048 * 512 * 4
    assert 2 * dw_bytes <= n.value <= 16 * dw_bytes


def test_unsupported_requests(lib):
    # the reference asserts groups == 1 on CUDA (nectarml/cuda/tensor/conv.py:120-121); so do we
    out = C.c_size_t()
    st = lib.nml_ref_conv2d(0, 0, 0, 0, 0, 0, 0, 1, 4, 8, 8, 4, 3, 3, 1, 1, 1, 1, 1, 1, 2, 0, 0, C.byref(out))
    assert st == 4
    # only float32 / float16 (nectarml/csrc/ops/tensor/matmul.cpp:47)
    st = lib.nml_ref_conv2d(0, 0, 0, 0, 0, 0, 0, 1, 4, 8, 8, 4, 3, 3, 1, 1, 1, 1, 1, 1, 1, 3, 0, C.byref(out))
    assert st == 1


def test_shim_rejects_bad_dtype():
    from nectarml_b200 import _nectarml
    with pytest.raises(RuntimeError):
        _nectarml.tensor.matmul(0, 0, [2, 2], [2, 2], _nectarml.DType.Int32)
    assert int(_nectarml.DType.Float32) == 0 and int(_nectarml.DType.Float16) == 1


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "nectarml_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, f"{f} mentions the oracle"


def test_workspace_sizes_of_special_walks(lib):
    """Workspace requests are computed without a device: the K-split forward walk asks for one fp32 plane of
    partial sums per K slice, the phase-packed gather walk for its packed weights and replicated bias."""
    n = C.c_size_t()
    # 4x4 s2 512->512 on a 4x4 image, batch 64: planes of 64 x 2 x 2 output pixels x 512 channels of fp32 partial
    # sums (one per K slice, at most 148 SMs / 4 tiles of them) beside the repacked weights (512 x 16 taps x 512 ch x 2 B)
    g = ConvGeometry(64, 512, 4, 4, 512, 4, 4, (2, 2), (1, 1))
    d = g.desc(_lib.NML_F16, "nhwc", _lib.NML_F16, "nhwc", _lib.NML_F16, "f16", False)
    assert lib.nml_conv_workspace_size(C.byref(d), 0, C.byref(n)) == 0
    weights, partial = 512 * 16 * 512 * 2, 64 * 2 * 2 * 512 * 4
    assert weights + 2 * partial <= n.value <= weights + 37 * partial + 4096
    # input gradient of a 7x7 s2 3->64 stem: four output phases x 3 channels = 12 packed columns over 16 union
    # taps of 64 channels (fp16), no bias; then the usual repack of those weights (16 columns of 64-wide K blocks)
    g = ConvGeometry(4, 3, 32, 32, 64, 7, 7, (2, 2), (3, 3))
    d = g.desc(_lib.NML_F16, "nhwc", _lib.NML_F16, "nhwc", _lib.NML_F16, "f16", False)
    assert lib.nml_conv_workspace_size(C.byref(d), 1, C.byref(n)) == 0
    packed = 12 * 64 * 16 * 2
    assert 2 * packed <= n.value <= 2 * packed + 4096
    # the same gradient into an NCHW tensor does not take the packed walk (one pass per phase instead)
    d = g.desc(_lib.NML_F16, "nhwc", _lib.NML_F16, "nchw", _lib.NML_F16, "f16", False)
    d.in_layout, d.out_layout = 1, 0  # dY NHWC, dX NCHW
    assert lib.nml_conv_workspace_size(C.byref(d), 1, C.byref(n)) == 0
