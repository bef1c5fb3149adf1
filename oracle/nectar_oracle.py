"""TEST INFRASTRUCTURE -- not part of the product.

CPU oracle for the Conv2d / ConvTranspose2d / Linear path: a ctypes front end to
``nectar_oracle.c`` (the C restatement of the reference's NumPy conv backend,
nectarml/cpu/conv/conv2d.py) plus the Linear arithmetic, which in the reference is NumPy itself
(``np.matmul`` in nectarml/cpu/math.py:80-81 under ``x @ W.transpose(1,0) + b``,
nectarml/nn/linear.py:44-47; gradients as written in
nectarml/core/_tensor/numerical.py:896-904 and :662-666).

Pinned by tests/golden/ (outputs of the reference's own functions, see make_golden.py there).
Only tests, the smoke check and the benchmark's CPU-baseline / reference legs may import this.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libnectar_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "nectar_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(_SO), exist_ok=True)
        subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-std=c99", "-o", _SO, src],
                       check=True)
    return _SO


def _load():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def conv_out_hw(H, W, KH, KW, stride, padding, dilation):
    """nectarml/nn/functional/conv.py:406-407."""
    return ((H + 2 * padding[0] - dilation[0] * (KH - 1) - 1) // stride[0] + 1,
            (W + 2 * padding[1] - dilation[1] * (KW - 1) - 1) // stride[1] + 1)


def conv_transpose_out_hw(H, W, KH, KW, stride, padding, dilation, output_padding):
    """nectarml/nn/functional/conv.py:479-482."""
    return ((H - 1) * stride[0] - 2 * padding[0] + dilation[0] * (KH - 1) + 1 + output_padding[0],
            (W - 1) * stride[1] - 2 * padding[1] + dilation[1] * (KW - 1) + 1 + output_padding[1])


def _ints(*v):
    return [C.c_int(int(x)) for x in v]


def conv2d(x, w, bias, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    x, w = _f32(x), _f32(w)
    bias = _f32(bias) if bias is not None else None
    B, Ci, H, W = x.shape
    Co, _, KH, KW = w.shape
    Ho, Wo = conv_out_hw(H, W, KH, KW, stride, padding, dilation)
    y = np.empty((B, Co, Ho, Wo), np.float32)
    _load().nml_oracle_conv2d(_p(x), _p(w), _p(bias), _p(y), *_ints(B, Ci, H, W, Co, KH, KW, Ho, Wo, *stride,
                                                                    *padding, *dilation))
    return y


def conv_transpose2d(x, w, bias, stride=(1, 1), padding=(0, 0), dilation=(1, 1), output_padding=(0, 0)):
    x, w = _f32(x), _f32(w)
    bias = _f32(bias) if bias is not None else None
    B, Ci, H, W = x.shape
    _, Co, KH, KW = w.shape
    Ho, Wo = conv_transpose_out_hw(H, W, KH, KW, stride, padding, dilation, output_padding)
    y = np.empty((B, Co, Ho, Wo), np.float32)
    _load().nml_oracle_conv_transpose2d(_p(x), _p(w), _p(bias), _p(y), *_ints(B, Ci, H, W, Co, KH, KW, *stride,
                                                                              *padding, *dilation, *output_padding))
    return y


def conv2d_backward_input(dy, w, x_shape, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    dy, w = _f32(dy), _f32(w)
    B, Ci, H, W = x_shape
    Co, _, KH, KW = w.shape
    Ho, Wo = dy.shape[2:]
    dx = np.empty((B, Ci, H, W), np.float32)
    _load().nml_oracle_conv2d_backward_input(_p(dy), _p(w), _p(dx), *_ints(B, Ci, H, W, Co, KH, KW, Ho, Wo, *stride,
                                                                           *padding, *dilation))
    return dx


def conv2d_backward_weight(dy, x, w_shape, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    dy, x = _f32(dy), _f32(x)
    B, Ci, H, W = x.shape
    Co, _, KH, KW = w_shape
    Ho, Wo = dy.shape[2:]
    dw = np.empty((Co, Ci, KH, KW), np.float32)
    _load().nml_oracle_conv2d_backward_weight(_p(dy), _p(x), _p(dw), *_ints(B, Ci, H, W, Co, KH, KW, Ho, Wo, *stride,
                                                                            *padding, *dilation))
    return dw


def conv_transpose2d_backward_input(dy, w, x_shape, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    dy, w = _f32(dy), _f32(w)
    B, Ci, H, W = x_shape
    _, Co, KH, KW = w.shape
    Ho, Wo = dy.shape[2:]
    dx = np.empty((B, Ci, H, W), np.float32)
    _load().nml_oracle_conv_transpose2d_backward_input(_p(dy), _p(w), _p(dx), *_ints(B, Ci, H, W, Co, KH, KW, Ho, Wo,
                                                                                     *stride, *padding, *dilation))
    return dx


def conv_transpose2d_backward_weight(dy, x, w_shape, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    dy, x = _f32(dy), _f32(x)
    B, Ci, H, W = x.shape
    _, Co, KH, KW = w_shape
    Ho, Wo = dy.shape[2:]
    dw = np.empty((Ci, Co, KH, KW), np.float32)
    _load().nml_oracle_conv_transpose2d_backward_weight(_p(dy), _p(x), _p(dw), *_ints(B, Ci, H, W, Co, KH, KW, Ho, Wo,
                                                                                      *stride, *padding, *dilation))
    return dw


# 1-D convolutions (nectarml/cpu/conv/conv1d.py:20-215) are the 2-D loops over an image of height 1: the
# reference's 1-D code accumulates in the same order (bias, then input channel, then kernel position).
def _up(a):
    return None if a is None else np.ascontiguousarray(np.asarray(a, np.float32)[:, :, None, :])


def conv1d(x, w, bias, stride=1, padding=0, dilation=1):
    return conv2d(_up(x), _up(w), bias, (1, stride), (0, padding), (1, dilation))[:, :, 0, :]


def conv_transpose1d(x, w, bias, stride=1, padding=0, dilation=1, output_padding=0):
    return conv_transpose2d(_up(x), _up(w), bias, (1, stride), (0, padding), (1, dilation), (0, output_padding))[:, :, 0, :]


def conv1d_backward_input(dy, w, x_shape, stride=1, padding=0, dilation=1):
    B, C, L = x_shape
    return conv2d_backward_input(_up(dy), _up(w), (B, C, 1, L), (1, stride), (0, padding), (1, dilation))[:, :, 0, :]


def conv1d_backward_weight(dy, x, w_shape, stride=1, padding=0, dilation=1):
    Co, Ci, K = w_shape
    return conv2d_backward_weight(_up(dy), _up(x), (Co, Ci, 1, K), (1, stride), (0, padding), (1, dilation))[:, :, 0, :]


def conv_transpose1d_backward_input(dy, w, x_shape, stride=1, padding=0, dilation=1):
    B, C, L = x_shape
    return conv_transpose2d_backward_input(_up(dy), _up(w), (B, C, 1, L), (1, stride), (0, padding),
                                           (1, dilation))[:, :, 0, :]


def conv_transpose1d_backward_weight(dy, x, w_shape, stride=1, padding=0, dilation=1):
    Ci, Co, K = w_shape
    return conv_transpose2d_backward_weight(_up(dy), _up(x), (Ci, Co, 1, K), (1, stride), (0, padding),
                                            (1, dilation))[:, :, 0, :]


def bias_grad(dy):
    dy = _f32(dy)
    B, Co, Ho, Wo = dy.shape
    db = np.empty(Co, np.float32)
    _load().nml_oracle_bias_grad(_p(dy), _p(db), *_ints(B, Co, Ho, Wo))
    return db


def linear_forward(x, w, bias):
    """``x @ W.transpose(1,0)`` then ``bias + y`` (nectarml/nn/linear.py:44-47)."""
    y = np.matmul(x, np.ascontiguousarray(w.T))
    return y if bias is None else bias + y


def linear_backward(x, w, dy):
    """dX = dY @ W, dW = X^T-contracted dY, db = dY.sum(0)
    (nectarml/core/_tensor/numerical.py:896-904, 662-666)."""
    return np.matmul(dy, w), np.matmul(np.ascontiguousarray(dy.T), x), dy.sum(axis=0)


def matmul(a, b):
    """nectarml/cpu/math.py:80-81."""
    return np.matmul(a, b)


def round_f16(a):
    """fp16 rounding of the operands, as the autocast forward applies before the contraction
    (nectarml/csrc/ops/tensor/conv/conv2d.cpp:415-419)."""
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)
