"""Tensor-level entry to the contraction path: torch tensors in (they only supply device memory
and the stream), the C ABI underneath.

Each function corresponds to one host op of the reference:

=============================  ================================================================
here                           reference
=============================  ================================================================
conv_forward                   nectar::conv2d / nectar::conv_transpose2d
                               (nectarml/csrc/ops/tensor/conv/conv2d.cpp:401-497)
conv_backward_data             conv2d_backward_input / conv_transpose2d_backward_input
                               (conv2d.cpp:499-542)
conv_backward_weight           conv2d_backward_weight / conv_transpose2d_backward_weight
                               (conv2d.cpp:544-583) + ``out_grad.sum(dim=(0,2,3))``
                               (nectarml/cuda/tensor/conv.py:175-176)
linear_forward / _backward_*   ``x @ W.T + b`` and its gradients
                               (nectarml/nn/linear.py:44-47,
                               nectarml/core/_tensor/numerical.py:864-907)
=============================  ================================================================
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import (NML_F16, NML_F32, NML_MATH_3XTF32, NML_MATH_F16, NML_MATH_TF32, NML_NCHW,
                   NML_NHWC, NML_PASS_BACKWARD_DATA, NML_PASS_BACKWARD_WEIGHT, NML_PASS_FORWARD,
                   ConvDesc, LinearDesc, check)

_MATH = {"f16": NML_MATH_F16, "3xtf32": NML_MATH_3XTF32, "tf32": NML_MATH_TF32}
_LAYOUT = {"nchw": NML_NCHW, "nhwc": NML_NHWC}


def _dt(t: torch.dtype) -> int:
    if t == torch.float32:
        return NML_F32
    if t == torch.float16:
        return NML_F16
    raise _lib.NectarB200Error(f"only float32 and float16 tensors are supported, got {t}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise _lib.NectarB200Error("tensors must live on a CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise _lib.NectarB200Error("tensors must be contiguous")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


@dataclass(frozen=True)
class ConvGeometry:
    """Shape of one Conv2d (``transposed=False``) or ConvTranspose2d layer, input side first."""
    batch: int
    c_in: int
    h: int
    w: int
    c_out: int
    kh: int
    kw: int
    stride: Tuple[int, int] = (1, 1)
    padding: Tuple[int, int] = (0, 0)
    dilation: Tuple[int, int] = (1, 1)
    output_padding: Tuple[int, int] = (0, 0)
    transposed: bool = False

    def out_hw(self) -> Tuple[int, int]:
        d = self.desc(NML_F32, "nchw", NML_F32, "nchw", NML_F32, "f16", False)
        ho, wo = C.c_int(), C.c_int()
        check(_lib.load().nml_conv_output_size(C.byref(d), C.byref(ho), C.byref(wo)))
        return ho.value, wo.value

    def desc(self, in_dtype, in_layout, out_dtype, out_layout, w_dtype, math, round_out_f16) -> ConvDesc:
        d = ConvDesc()
        d.batch, d.c_in, d.h, d.w = self.batch, self.c_in, self.h, self.w
        d.c_out, d.kh, d.kw = self.c_out, self.kh, self.kw
        d.stride_h, d.stride_w = self.stride
        d.pad_h, d.pad_w = self.padding
        d.dil_h, d.dil_w = self.dilation
        d.outpad_h, d.outpad_w = self.output_padding
        d.transposed = int(self.transposed)
        d.in_dtype, d.in_layout = in_dtype, _LAYOUT[in_layout]
        d.out_dtype, d.out_layout = out_dtype, _LAYOUT[out_layout]
        d.w_dtype = w_dtype
        d.math = _MATH[math]
        d.round_out_f16 = int(bool(round_out_f16))
        return d

    def act_shape(self, which: str, layout: str) -> Tuple[int, int, int, int]:
        """Shape of the layer input (``which='in'``) or output (``'out'``) in the given layout."""
        if which == "in":
            c, h, w = self.c_in, self.h, self.w
        else:
            c = self.c_out
            h, w = self.out_hw()
        return (self.batch, c, h, w) if layout == "nchw" else (self.batch, h, w, c)

    def weight_shape(self) -> Tuple[int, int, int, int]:
        if self.transposed:
            return (self.c_in, self.c_out, self.kh, self.kw)
        return (self.c_out, self.c_in, self.kh, self.kw)


class Workspace:
    """Grow-only device scratch buffer handed to the C ABI (which itself never allocates)."""

    def __init__(self) -> None:
        self.buf: Optional[torch.Tensor] = None

    def get(self, nbytes: int, device) -> Tuple[Optional[int], int]:
        if nbytes == 0:
            return None, 0
        if self.buf is None or self.buf.numel() < nbytes or self.buf.device != torch.device(device):
            self.buf = torch.empty(int(nbytes * 1.25) + 256, dtype=torch.uint8, device=device)
        return self.buf.data_ptr(), self.buf.numel()


_default_ws = Workspace()


def _conv_ws(d: ConvDesc, which: int, ws: Optional[Workspace], device):
    need = C.c_size_t()
    check(_lib.load().nml_conv_workspace_size(C.byref(d), which, C.byref(need)))
    return (ws or _default_ws).get(need.value, device)


def conv_forward(g: ConvGeometry, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
                 layout: str = "nchw", out_layout: Optional[str] = None, math: str = "f16",
                 out_dtype: Optional[torch.dtype] = None, round_out_f16: bool = False,
                 out: Optional[torch.Tensor] = None, ws: Optional[Workspace] = None) -> torch.Tensor:
    out_layout = out_layout or layout
    out_dtype = out_dtype or x.dtype
    assert tuple(x.shape) == g.act_shape("in", layout), (tuple(x.shape), g.act_shape("in", layout))
    assert tuple(w.shape) == g.weight_shape()
    if bias is not None:
        assert bias.dtype == w.dtype and bias.numel() == g.c_out
    if out is None:
        out = torch.empty(g.act_shape("out", out_layout), dtype=out_dtype, device=x.device)
    d = g.desc(_dt(x.dtype), layout, _dt(out.dtype), out_layout, _dt(w.dtype), math, round_out_f16)
    wp, wb = _conv_ws(d, NML_PASS_FORWARD, ws, x.device)
    check(_lib.load().nml_conv_forward(C.byref(d), _ptr(x), _ptr(w), _ptr(bias), _ptr(out), wp, wb, _stream()))
    return out


def conv_backward_data(g: ConvGeometry, dy: torch.Tensor, w: torch.Tensor, *, layout: str = "nchw",
                       out_layout: Optional[str] = None, math: str = "f16",
                       out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
                       ws: Optional[Workspace] = None) -> torch.Tensor:
    out_layout = out_layout or layout
    out_dtype = out_dtype or dy.dtype
    assert tuple(dy.shape) == g.act_shape("out", layout)
    assert tuple(w.shape) == g.weight_shape()
    if out is None:
        out = torch.empty(g.act_shape("in", out_layout), dtype=out_dtype, device=dy.device)
    d = g.desc(_dt(dy.dtype), layout, _dt(out.dtype), out_layout, _dt(w.dtype), math, False)
    wp, wb = _conv_ws(d, NML_PASS_BACKWARD_DATA, ws, dy.device)
    check(_lib.load().nml_conv_backward_data(C.byref(d), _ptr(dy), _ptr(w), _ptr(out), wp, wb, _stream()))
    return out


def conv_backward_weight(g: ConvGeometry, x: torch.Tensor, dy: torch.Tensor, *, layout: str = "nchw",
                         math: str = "f16", want_bias_grad: bool = True, dw: Optional[torch.Tensor] = None,
                         db: Optional[torch.Tensor] = None,
                         ws: Optional[Workspace] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """dw (fp32, weight-shaped) and db (fp32, c_out); pass ``dw`` / ``db`` to have them written in place, e.g.
    into the views of a flat gradient bucket."""
    assert tuple(x.shape) == g.act_shape("in", layout)
    assert tuple(dy.shape) == g.act_shape("out", layout)
    assert x.dtype == dy.dtype
    if dw is None:
        dw = torch.empty(g.weight_shape(), dtype=torch.float32, device=x.device)
    if db is None and want_bias_grad:
        db = torch.empty(g.c_out, dtype=torch.float32, device=x.device)
    assert dw.dtype == torch.float32 and dw.numel() == g.c_in * g.c_out * g.kh * g.kw
    d = g.desc(_dt(x.dtype), layout, NML_F32, layout, NML_F32, math, False)
    wp, wb = _conv_ws(d, NML_PASS_BACKWARD_WEIGHT, ws, x.device)
    check(_lib.load().nml_conv_backward_weight(C.byref(d), _ptr(x), _ptr(dy), _ptr(dw), _ptr(db), wp, wb,
                                               _stream()))
    return dw, db


def _linear_desc(rows, fin, fout, in_dtype, out_dtype, w_dtype, math, round_out_f16) -> LinearDesc:
    d = LinearDesc()
    d.rows, d.in_features, d.out_features = rows, fin, fout
    d.in_dtype, d.out_dtype, d.w_dtype = in_dtype, out_dtype, w_dtype
    d.math = _MATH[math]
    d.round_out_f16 = int(bool(round_out_f16))
    return d


def _linear_ws(d: LinearDesc, which: int, ws: Optional[Workspace], device):
    need = C.c_size_t()
    check(_lib.load().nml_linear_workspace_size(C.byref(d), which, C.byref(need)))
    return (ws or _default_ws).get(need.value, device)


def linear_forward(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, *, math: str = "f16",
                   out_dtype: Optional[torch.dtype] = None, round_out_f16: bool = False,
                   out: Optional[torch.Tensor] = None, ws: Optional[Workspace] = None) -> torch.Tensor:
    """y[rows, out] = x[rows, in] @ w[out, in].T + bias."""
    rows, fin = x.shape
    fout = w.shape[0]
    assert w.shape[1] == fin
    if out is None:
        out = torch.empty((rows, fout), dtype=out_dtype or x.dtype, device=x.device)
    d = _linear_desc(rows, fin, fout, _dt(x.dtype), _dt(out.dtype), _dt(w.dtype), math, round_out_f16)
    wp, wb = _linear_ws(d, NML_PASS_FORWARD, ws, x.device)
    check(_lib.load().nml_linear_forward(C.byref(d), _ptr(x), _ptr(w), _ptr(bias), _ptr(out), wp, wb, _stream()))
    return out


def linear_backward_data(dy: torch.Tensor, w: torch.Tensor, *, math: str = "f16",
                         out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
                         ws: Optional[Workspace] = None) -> torch.Tensor:
    """dx[rows, in] = dy[rows, out] @ w[out, in]."""
    rows, fout = dy.shape
    fin = w.shape[1]
    assert w.shape[0] == fout
    if out is None:
        out = torch.empty((rows, fin), dtype=out_dtype or dy.dtype, device=dy.device)
    d = _linear_desc(rows, fin, fout, _dt(dy.dtype), _dt(out.dtype), _dt(w.dtype), math, False)
    wp, wb = _linear_ws(d, NML_PASS_BACKWARD_DATA, ws, dy.device)
    check(_lib.load().nml_linear_backward_data(C.byref(d), _ptr(dy), _ptr(w), _ptr(out), wp, wb, _stream()))
    return out


def linear_backward_weight(x: torch.Tensor, dy: torch.Tensor, *, math: str = "f16", want_bias_grad: bool = True,
                           dw: Optional[torch.Tensor] = None, db: Optional[torch.Tensor] = None,
                           ws: Optional[Workspace] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """dw[out, in] = dy.T @ x (fp32), db[out] = dy.sum(0) (fp32)."""
    rows, fin = x.shape
    fout = dy.shape[1]
    assert dy.shape[0] == rows and x.dtype == dy.dtype
    if dw is None:
        dw = torch.empty((fout, fin), dtype=torch.float32, device=x.device)
    if db is None and want_bias_grad:
        db = torch.empty(fout, dtype=torch.float32, device=x.device)
    d = _linear_desc(rows, fin, fout, _dt(x.dtype), NML_F32, NML_F32, math, False)
    wp, wb = _linear_ws(d, NML_PASS_BACKWARD_WEIGHT, ws, x.device)
    check(_lib.load().nml_linear_backward_weight(C.byref(d), _ptr(x), _ptr(dy), _ptr(dw), _ptr(db), wp, wb,
                                                 _stream()))
    return dw, db


def device_status() -> int:
    """Synchronises and raises if a kernel abandoned a bounded wait since the last call."""
    code = C.c_int(0)
    st = _lib.load().nml_device_status(C.byref(code))
    if st != 0:
        raise _lib.NectarB200Error(f"device-side failure, code {code.value}: "
                                   f"{_lib.load().nml_status_string(st).decode()}")
    return 0


def set_sm_limit(sms: int) -> None:
    """Caps the SMs later launches occupy (0: all); used while a collective shares the GPU."""
    check(_lib.load().nml_set_sm_limit(int(sms)))


def launch_count() -> int:
    return int(_lib.load().nml_launch_count())


def profile_begin(max_records: int) -> None:
    """Start bracketing the next ``max_records`` contraction-kernel launches with CUDA events."""
    check(_lib.load().nml_profile_begin(int(max_records)))


def profile_end(max_records: int):
    """Synchronise and return the recorded per-launch durations (ms) in launch order."""
    buf = (C.c_float * max_records)()
    n = C.c_int(0)
    check(_lib.load().nml_profile_end(buf, max_records, C.byref(n)))
    return [float(buf[i]) for i in range(n.value)]


def tma_box(t: torch.Tensor, box, elem_strides, coords) -> torch.Tensor:
    """Test support: returns one TMA box of a 4-D tensor (``t.shape`` slowest-first, as torch
    prints it; ``box``/``elem_strides``/``coords`` fastest-first, as TMA takes them)."""
    assert t.dim() == 4 and t.is_contiguous()
    dims = list(reversed(t.shape))
    n = 1
    for b, s in zip(box, elem_strides):
        n *= (b + s - 1) // s
    out = torch.zeros(n, dtype=t.dtype, device=t.device)
    arr = lambda v: (C.c_int * 4)(*v)
    check(_lib.load().nml_debug_tma_box(_ptr(t), t.element_size(), arr(dims), arr(box), arr(elem_strides),
                                        arr(coords), _ptr(out), out.numel() * out.element_size(), _stream()))
    return out
