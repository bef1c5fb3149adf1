"""ctypes binding of the C ABI in ``include/nectarml_b200.h``.

The shared library is built in-tree by :mod:`nectarml_b200.build` (nvcc, sm_100a).  There is no
CPU or library fallback: if the library is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnectarml_b200.so")

NML_OK = 0
NML_F32, NML_F16 = 0, 1
NML_NCHW, NML_NHWC = 0, 1
NML_MATH_F16, NML_MATH_3XTF32, NML_MATH_TF32 = 0, 1, 2
NML_PASS_FORWARD, NML_PASS_BACKWARD_DATA, NML_PASS_BACKWARD_WEIGHT = 0, 1, 2


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "batch", "c_in", "h", "w", "c_out", "kh", "kw", "stride_h", "stride_w", "pad_h", "pad_w",
        "dil_h", "dil_w", "outpad_h", "outpad_w", "transposed", "in_dtype", "in_layout",
        "out_dtype", "out_layout", "w_dtype", "math", "round_out_f16")]


class LinearDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "rows", "in_features", "out_features", "in_dtype", "out_dtype", "w_dtype", "math",
        "round_out_f16")]


# name -> (restype, argtypes); every symbol the header declares is listed here and checked at load.
_VP, _SZ, _UP = C.c_void_p, C.c_size_t, C.c_size_t  # uintptr_t == size_t on this ABI
_I = C.c_int
_ref_fwd_common = [_UP, _SZ, _UP, _SZ, _UP, _SZ, _SZ] + [_I] * 13
_ref_bwd_common = [_UP, _UP] + [_I] * 15
SYMBOLS = {
    "nml_status_string": (C.c_char_p, [_I]),
    "nml_conv_output_size": (_I, [C.POINTER(ConvDesc), C.POINTER(_I), C.POINTER(_I)]),
    "nml_conv_workspace_size": (_I, [C.POINTER(ConvDesc), _I, C.POINTER(_SZ)]),
    "nml_linear_workspace_size": (_I, [C.POINTER(LinearDesc), _I, C.POINTER(_SZ)]),
    "nml_conv_forward": (_I, [C.POINTER(ConvDesc), _VP, _VP, _VP, _VP, _VP, _SZ, _VP]),
    "nml_conv_forward_static": (_I, [C.POINTER(ConvDesc), _VP, _VP, _VP, _VP, _VP]),
    "nml_conv_backward_data": (_I, [C.POINTER(ConvDesc), _VP, _VP, _VP, _VP, _SZ, _VP]),
    "nml_conv_backward_weight": (_I, [C.POINTER(ConvDesc), _VP, _VP, _VP, _VP, _VP, _SZ, _VP]),
    "nml_linear_forward": (_I, [C.POINTER(LinearDesc), _VP, _VP, _VP, _VP, _VP, _SZ, _VP]),
    "nml_linear_backward_data": (_I, [C.POINTER(LinearDesc), _VP, _VP, _VP, _VP, _SZ, _VP]),
    "nml_linear_backward_weight": (_I, [C.POINTER(LinearDesc), _VP, _VP, _VP, _VP, _VP, _SZ, _VP]),
    "nml_init": (_I, []),
    "nml_set_sm_limit": (_I, [_I]),
    "nml_device_status": (_I, [C.POINTER(_I)]),
    "nml_launch_count": (C.c_longlong, []),
    "nml_layers_launch_count": (C.c_longlong, []),
    "nml_bn_workspace_size": (_I, [C.c_longlong, _I, C.POINTER(_SZ)]),
    "nml_bn_forward": (_I, [_VP, C.c_longlong, _I, _VP, _VP, _VP, _I, C.c_float, C.c_float, _VP, _VP, _VP, _VP, _SZ, _VP]),
    "nml_bn_backward": (_I, [_VP, _VP, _VP, C.c_longlong, _I, _VP, _VP, _VP, _I, C.c_float, _VP, _VP, _VP, _VP, _VP, _SZ, _VP]),
    "nml_maxpool_forward": (_I, [_VP, _I, _I, _I, _I, _I, _I, _I, _VP, _VP, _VP]),
    "nml_maxpool_backward": (_I, [_VP, _VP, _I, _I, _I, _I, _I, _I, _I, _VP, _VP]),
    "nml_grads_check": (_I, [_VP, _SZ, C.c_float, _VP, _VP]),
    "nml_sgd_momentum_step": (_I, [_VP, _VP, _VP, _VP, _SZ, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, _VP, _VP]),
    "nml_profile_begin": (_I, [_I]),
    "nml_profile_end": (_I, [C.POINTER(C.c_float), _I, C.POINTER(_I)]),
    # conv2d: ... dilation_w, groups, dtype, half_precision, result
    "nml_ref_conv2d": (_I, _ref_fwd_common + [_I, _I, _I, C.POINTER(_UP)]),
    # conv_transpose2d: ... dilation_w, outpad_h, outpad_w, groups, dtype, half_precision, result
    "nml_ref_conv_transpose2d": (_I, _ref_fwd_common + [_I, _I, _I, _I, _I, C.POINTER(_UP)]),
    # backward_input: 15 ints + groups + dtype + result
    "nml_ref_conv2d_backward_input": (_I, _ref_bwd_common + [_I, _I, C.POINTER(_UP)]),
    "nml_ref_conv_transpose2d_backward_input": (_I, _ref_bwd_common + [_I, _I, C.POINTER(_UP)]),
    # backward_weight: 15 ints + dtype + result
    "nml_ref_conv2d_backward_weight": (_I, _ref_bwd_common + [_I, C.POINTER(_UP)]),
    "nml_ref_conv_transpose2d_backward_weight": (_I, _ref_bwd_common + [_I, C.POINTER(_UP)]),
    # 1-D: (ptr, ptr, bias) + B, C_in, L, C_out, K, stride, padding, dilation[, output_padding], groups, dtype, result
    "nml_ref_conv1d": (_I, [_UP, _UP, _UP] + [_I] * 10 + [C.POINTER(_UP)]),
    "nml_ref_conv_transpose1d": (_I, [_UP, _UP, _UP] + [_I] * 11 + [C.POINTER(_UP)]),
    "nml_ref_conv1d_backward_input": (_I, [_UP, _UP] + [_I] * 11 + [C.POINTER(_UP)]),
    "nml_ref_conv_transpose1d_backward_input": (_I, [_UP, _UP] + [_I] * 11 + [C.POINTER(_UP)]),
    "nml_ref_conv1d_backward_weight": (_I, [_UP, _UP] + [_I] * 10 + [C.POINTER(_UP)]),
    "nml_ref_conv_transpose1d_backward_weight": (_I, [_UP, _UP] + [_I] * 10 + [C.POINTER(_UP)]),
    "nml_ref_matmul": (_I, [_UP, _UP, C.POINTER(_I), _I, C.POINTER(_I), _I, _I, C.POINTER(_UP)]),
    "nml_ref_free": (_I, [_UP]),
    "nml_debug_copy_to_host": (_I, [_VP, _UP, _SZ]),
    "nml_debug_wait_timeout": (_I, [C.c_ulonglong, _I, _VP]),
    "nml_debug_stalled_linear_forward": (_I, [C.POINTER(LinearDesc), _VP, _VP, _VP, _VP, _SZ, C.c_ulonglong, _VP]),
    "nml_debug_tma_box": (_I, [_VP, _I, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I), C.POINTER(_I),
                               _VP, _SZ, _VP]),
}

_lib = None


class NectarB200Error(RuntimeError):
    """Raised for every non-zero status of the C ABI (the reference raises RuntimeError too)."""


def load() -> C.CDLL:
    """Loads the library once and binds every declared symbol; raises if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise NectarB200Error(
            f"{LIB_PATH} is missing: build it with `python -m nectarml_b200.build` "
            "(there is no fallback path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != NML_OK:
        msg = load().nml_status_string(status).decode()
        raise NectarB200Error(f"nectarml_b200 status {status}: {msg}")
