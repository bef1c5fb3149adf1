"""Drop-in for the part of the reference's pybind module ``_nectarml`` that this path covers.

The reference's Python wrappers call ``_nectarml.tensor.conv.conv2d(...)`` and friends with
device pointers as integers plus shape ints and get a device pointer back
(nectarml/cuda/tensor/conv.py:138-146, 157-171, 211-220, 232-247;
nectarml/cuda/tensor/matmul.py:9-10; registration in nectarml/csrc/python/bindings.cpp:41-51,
prototypes in nectarml/csrc/python/ops/tensor/conv.h:71-150 and matmul.h:10-16).  The same
names, argument order and error type (``RuntimeError``) are kept here and forwarded to the
``nml_ref_*`` entry points of the C ABI.  ``DType`` mirrors the reference's enum
(nectarml/csrc/include/common/dtype.h:15-21); only Float32 and Float16 are valid on this path.
"""
from __future__ import annotations

import ctypes as C
import enum
from typing import Sequence

from . import _lib


class DType(enum.IntEnum):
    Float32 = 0
    Float16 = 1
    UInt8 = 2
    Int32 = 3
    Bool = 4


def _dtype(dtype) -> int:
    v = int(dtype)
    if v not in (DType.Float32, DType.Float16):
        raise RuntimeError("conv / matmul only support float32 and float16")
    return v


def _call(fn, *args) -> int:
    out = C.c_size_t(0)
    status = fn(*args, C.byref(out))
    if status != 0:
        raise RuntimeError(f"nectarml_b200: {_lib.load().nml_status_string(status).decode()}")
    return int(out.value)


class _Conv:
    """``_nectarml.tensor.conv``"""

    @staticmethod
    def conv2d(input_ptr, input_size, weight_ptr, weight_size, bias_ptr, bias_size, output_size, B, C_in, H, W,
               C_out, KH, KW, stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w, groups, dtype,
               half_precision) -> int:
        return _call(_lib.load().nml_ref_conv2d, input_ptr, input_size, weight_ptr, weight_size, bias_ptr or 0,
                     bias_size, output_size, B, C_in, H, W, C_out, KH, KW, stride_h, stride_w, padding_h, padding_w,
                     dilation_h, dilation_w, groups, _dtype(dtype), int(bool(half_precision)))

    @staticmethod
    def conv_transpose2d(input_ptr, input_size, weight_ptr, weight_size, bias_ptr, bias_size, output_size, B, C_in,
                         H, W, C_out, KH, KW, stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w,
                         output_padding_h, output_padding_w, groups, dtype, half_precision) -> int:
        return _call(_lib.load().nml_ref_conv_transpose2d, input_ptr, input_size, weight_ptr, weight_size,
                     bias_ptr or 0, bias_size, output_size, B, C_in, H, W, C_out, KH, KW, stride_h, stride_w,
                     padding_h, padding_w, dilation_h, dilation_w, output_padding_h, output_padding_w, groups,
                     _dtype(dtype), int(bool(half_precision)))

    @staticmethod
    def conv2d_backward_input(out_grad_ptr, weight_ptr, B, C_in, H, W, C_out, KH, KW, H_out, W_out, stride_h,
                              stride_w, padding_h, padding_w, dilation_h, dilation_w, groups, dtype) -> int:
        return _call(_lib.load().nml_ref_conv2d_backward_input, out_grad_ptr, weight_ptr, B, C_in, H, W, C_out, KH,
                     KW, H_out, W_out, stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w, groups,
                     _dtype(dtype))

    @staticmethod
    def conv_transpose2d_backward_input(out_grad_ptr, weight_ptr, B, C_in, H, W, C_out, KH, KW, H_out, W_out,
                                        stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w, groups,
                                        dtype) -> int:
        return _call(_lib.load().nml_ref_conv_transpose2d_backward_input, out_grad_ptr, weight_ptr, B, C_in, H, W,
                     C_out, KH, KW, H_out, W_out, stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w,
                     groups, _dtype(dtype))

    @staticmethod
    def conv2d_backward_weight(out_grad_ptr, input_ptr, B, C_in, H, W, C_out, KH, KW, H_out, W_out, stride_h,
                               stride_w, padding_h, padding_w, dilation_h, dilation_w, dtype) -> int:
        return _call(_lib.load().nml_ref_conv2d_backward_weight, out_grad_ptr, input_ptr, B, C_in, H, W, C_out, KH,
                     KW, H_out, W_out, stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w,
                     _dtype(dtype))

    @staticmethod
    def conv_transpose2d_backward_weight(out_grad_ptr, input_ptr, B, C_in, H, W, C_out, KH, KW, H_out, W_out,
                                         stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w,
                                         dtype) -> int:
        return _call(_lib.load().nml_ref_conv_transpose2d_backward_weight, out_grad_ptr, input_ptr, B, C_in, H, W,
                     C_out, KH, KW, H_out, W_out, stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w,
                     _dtype(dtype))


    # 1-D convolutions (nectarml/csrc/python/ops/tensor/conv.h:11-68; callers nectarml/cuda/tensor/conv.py:12-106)
    @staticmethod
    def conv1d(input_ptr, weight_ptr, bias_ptr, B, C_in, L, C_out, K, stride, padding, dilation, groups, dtype) -> int:
        return _call(_lib.load().nml_ref_conv1d, input_ptr, weight_ptr, bias_ptr or 0, B, C_in, L, C_out, K, stride,
                     padding, dilation, groups, _dtype(dtype))

    @staticmethod
    def conv_transpose1d(input_ptr, weight_ptr, bias_ptr, B, C_in, L, C_out, K, stride, padding, dilation,
                         output_padding, groups, dtype) -> int:
        return _call(_lib.load().nml_ref_conv_transpose1d, input_ptr, weight_ptr, bias_ptr or 0, B, C_in, L, C_out, K,
                     stride, padding, dilation, output_padding, groups, _dtype(dtype))

    @staticmethod
    def conv1d_backward_input(out_grad_ptr, weight_ptr, B, C_in, L, C_out, K, L_out, stride, padding, dilation,
                              groups, dtype) -> int:
        return _call(_lib.load().nml_ref_conv1d_backward_input, out_grad_ptr, weight_ptr, B, C_in, L, C_out, K, L_out,
                     stride, padding, dilation, groups, _dtype(dtype))

    @staticmethod
    def conv_transpose1d_backward_input(out_grad_ptr, weight_ptr, B, C_in, L, C_out, K, L_out, stride, padding,
                                        dilation, groups, dtype) -> int:
        return _call(_lib.load().nml_ref_conv_transpose1d_backward_input, out_grad_ptr, weight_ptr, B, C_in, L, C_out,
                     K, L_out, stride, padding, dilation, groups, _dtype(dtype))

    @staticmethod
    def conv1d_backward_weight(out_grad_ptr, input_ptr, B, C_in, L, C_out, K, L_out, stride, padding, dilation,
                               dtype) -> int:
        return _call(_lib.load().nml_ref_conv1d_backward_weight, out_grad_ptr, input_ptr, B, C_in, L, C_out, K, L_out,
                     stride, padding, dilation, _dtype(dtype))

    @staticmethod
    def conv_transpose1d_backward_weight(out_grad_ptr, input_ptr, B, C_in, L, C_out, K, L_out, stride, padding,
                                         dilation, dtype) -> int:
        return _call(_lib.load().nml_ref_conv_transpose1d_backward_weight, out_grad_ptr, input_ptr, B, C_in, L, C_out,
                     K, L_out, stride, padding, dilation, _dtype(dtype))


class _Tensor:
    """``_nectarml.tensor``"""
    conv = _Conv()

    @staticmethod
    def matmul(a_ptr, b_ptr, a_shape: Sequence[int], b_shape: Sequence[int], dtype) -> int:
        a = (C.c_int * len(a_shape))(*[int(v) for v in a_shape])
        b = (C.c_int * len(b_shape))(*[int(v) for v in b_shape])
        return _call(_lib.load().nml_ref_matmul, a_ptr, b_ptr, a, len(a_shape), b, len(b_shape), _dtype(dtype))


tensor = _Tensor()


def free_cuda(ptr: int, n_elements: int = 0, dtype=None) -> None:
    """Releases a result pointer (the reference's ``_nectarml.free_cuda(ptr, n_elements, dtype)``)."""
    status = _lib.load().nml_ref_free(ptr)
    if status != 0:
        raise RuntimeError(f"nectarml_b200: {_lib.load().nml_status_string(status).decode()}")
