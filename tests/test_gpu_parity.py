"""CUDA path vs the CPU oracle and the reference-generated fixtures, all through the C ABI.

Three call styles are covered for every golden geometry:
  * reference-shaped fp32 (`_nectarml.tensor.conv.*`, 3xTF32)  -- tolerance 1e-5 of max|ref|
  * reference-shaped autocast forward (fp32 tensors, fp16 arithmetic) -- 1e-2 rel / 1e-3 abs
  * native fp16 NHWC (descriptor API)                              -- 1e-2 rel / 1e-3 abs
fp16 comparisons use the oracle on fp16-rounded inputs, which is what the arithmetic sees."""
import numpy as np
import pytest
import torch

import cases
from gpu_util import DEV, F16, F32, assert_f16, assert_f32, dev, fetch, geometry, host, rel_max
from nectarml_b200 import _nectarml, ops

pytestmark = pytest.mark.gpu
conv = _nectarml.tensor.conv


def oracle_all(oracle, case, x, w, b, dy):
    transposed, geom, _, _ = case
    B, Ci, H, W, Co, KH, KW, s, p, d, op = geom
    if not transposed:
        return (oracle.conv2d(x, w, b, s, p, d), oracle.conv2d_backward_input(dy, w, x.shape, s, p, d),
                oracle.conv2d_backward_weight(dy, x, w.shape, s, p, d), oracle.bias_grad(dy))
    return (oracle.conv_transpose2d(x, w, b, s, p, d, op), oracle.conv_transpose2d_backward_input(dy, w, x.shape, s, p, d),
            oracle.conv_transpose2d_backward_weight(dy, x, w.shape, s, p, d), oracle.bias_grad(dy))


def shim_forward(case, xd, wd, bd, dtype, half):
    transposed, geom, _, _ = case
    B, Ci, H, W, Co, KH, KW, s, p, d, op = geom
    Ho, Wo = cases.out_hw(transposed, geom)
    common = (xd.data_ptr(), xd.numel(), wd.data_ptr(), wd.numel(), bd.data_ptr() if bd is not None else 0,
              bd.numel() if bd is not None else 0, B * Co * Ho * Wo, B, Ci, H, W, Co, KH, KW, s[0], s[1], p[0], p[1],
              d[0], d[1])
    if transposed:
        ptr = conv.conv_transpose2d(*common, op[0], op[1], 1, dtype, half)
    else:
        ptr = conv.conv2d(*common, 1, dtype, half)
    return fetch(ptr, (B, Co, Ho, Wo), np.float32 if dtype == F32 else np.float16)


def shim_backward(case, dyd, xd, wd, dtype):
    transposed, geom, _, _ = case
    B, Ci, H, W, Co, KH, KW, s, p, d, op = geom
    Ho, Wo = cases.out_hw(transposed, geom)
    args = (B, Ci, H, W, Co, KH, KW, Ho, Wo, s[0], s[1], p[0], p[1], d[0], d[1])
    if transposed:
        dx = conv.conv_transpose2d_backward_input(dyd.data_ptr(), wd.data_ptr(), *args, 1, dtype)
        dw = conv.conv_transpose2d_backward_weight(dyd.data_ptr(), xd.data_ptr(), *args, dtype)
        wshape = (Ci, Co, KH, KW)
    else:
        dx = conv.conv2d_backward_input(dyd.data_ptr(), wd.data_ptr(), *args, 1, dtype)
        dw = conv.conv2d_backward_weight(dyd.data_ptr(), xd.data_ptr(), *args, dtype)
        wshape = (Co, Ci, KH, KW)
    return fetch(dx, (B, Ci, H, W)), fetch(dw, wshape)


@pytest.mark.parametrize("name", sorted(cases.CONV_CASES))
def test_reference_shaped_fp32(name, golden_small, oracle):
    case = cases.CONV_CASES[name]
    x, w, b, dy = cases.draw_conv(name, case)
    y_o, dx_o, dw_o, db_o = oracle_all(oracle, case, x, w, b, dy)
    xd, wd, dyd = dev(x), dev(w), dev(dy)
    bd = dev(b) if b is not None else None
    y = shim_forward(case, xd, wd, bd, F32, False)
    dx, dw = shim_backward(case, dyd, xd, wd, F32)
    ops.device_status()
    for got, orc, key in ((y, y_o, "y"), (dx, dx_o, "dx"), (dw, dw_o, "dw")):
        assert_f32(got, orc, f"{name} {key} vs oracle")
        assert_f32(got, golden_small[f"{name}__{key}"], f"{name} {key} vs reference fixture")


@pytest.mark.parametrize("name", sorted(cases.CONV_CASES))
def test_reference_shaped_autocast_forward(name, oracle):
    """half_precision=True: fp32 tensors, fp16 operands, fp32 result holding fp16-rounded values
    (nectarml/csrc/ops/tensor/conv/conv2d.cpp:415-435)."""
    case = cases.CONV_CASES[name]
    transposed, geom, _, _ = case
    x, w, b, dy = cases.draw_conv(name, case)
    r = oracle.round_f16
    y_o = oracle_all(oracle, case, r(x), r(w), r(b) if b is not None else None, dy)[0]
    y = shim_forward(case, dev(x), dev(w), dev(b) if b is not None else None, F32, True)
    ops.device_status()
    assert_f16(y, y_o, f"{name} autocast y")
    assert np.array_equal(y, y.astype(np.float16).astype(np.float32)), "result is not fp16-representable"


@pytest.mark.parametrize("name", sorted(cases.CONV_CASES))
def test_native_fp16_nhwc(name, oracle):
    case = cases.CONV_CASES[name]
    g = geometry(case)
    x, w, b, dy = cases.draw_conv(name, case)
    r = oracle.round_f16
    y_o, dx_o, dw_o, db_o = oracle_all(oracle, case, r(x), r(w), r(b) if b is not None else None, r(dy))
    xd, dyd = dev(x, torch.float16, nhwc=True), dev(dy, torch.float16, nhwc=True)
    wd = dev(w, torch.float16)
    bd = dev(b, torch.float16) if b is not None else None
    y = ops.conv_forward(g, xd, wd, bd, layout="nhwc", math="f16")
    dx = ops.conv_backward_data(g, dyd, wd, layout="nhwc", math="f16")
    dw, db = ops.conv_backward_weight(g, xd, dyd, layout="nhwc", math="f16")
    ops.device_status()
    assert_f16(host(y, nhwc=True), y_o, f"{name} y")
    assert_f16(host(dx, nhwc=True), dx_o, f"{name} dx")
    # gradients of the weights come out in fp32 from fp32 accumulation
    assert_f32(host(dw), dw_o, f"{name} dw", tol=2e-5)
    assert_f32(host(db), db_o, f"{name} db", tol=2e-5)


# Unit-stride multi-tap layers whose weights fit in shared memory take the patch walk (one haloed box
# per channel block, resident weights, two issuing warps); these shapes span several tiles in both
# image directions, ragged edges, two channel blocks, dilation and a transposed (gather) layer.
PATCH_SHAPES = {
    "p_3x3_64_96":   (False, (2, 64, 40, 27, 96, 3, 3, (1, 1), (1, 1), (1, 1), (0, 0)), True, "normal"),
    "p_3x3_128_32":  (False, (1, 128, 33, 50, 32, 3, 3, (1, 1), (1, 1), (1, 1), (0, 0)), True, "normal"),
    "p_5x5_dil":     (False, (2, 16, 37, 21, 24, 5, 5, (1, 1), (4, 4), (2, 2), (0, 0)), False, "normal"),
    "p_rect_nopad":  (False, (3, 40, 19, 45, 64, 2, 4, (1, 1), (0, 0), (1, 1), (0, 0)), True, "normal"),
    "p_t_3x3_s1":    (True,  (2, 48, 18, 29, 40, 3, 3, (1, 1), (1, 1), (1, 1), (0, 0)), True, "normal"),
}


# Few output pixels under a long K loop (U-Net bottleneck layers): the forward walk splits K over
# CTAs and adds partial sums into an fp32 scratch that a finishing pass turns into the output.
SPLIT_SHAPES = {
    "s_conv_k4_s2":  (False, (2, 256, 4, 4, 96, 4, 4, (2, 2), (1, 1), (1, 1), (0, 0)), True, "normal"),
    "s_convT_k4_s2": (True,  (2, 256, 2, 2, 72, 4, 4, (2, 2), (1, 1), (1, 1), (0, 0)), True, "normal"),
    "s_conv_3x3":    (False, (1, 320, 6, 5, 40, 3, 3, (1, 1), (0, 0), (1, 1), (0, 0)), False, "normal"),
}
WALK_SHAPES = {**PATCH_SHAPES, **SPLIT_SHAPES}


@pytest.mark.parametrize("name", sorted(WALK_SHAPES))
def test_patch_walk_shapes(name, oracle):
    case = WALK_SHAPES[name]
    g = geometry(case)
    x, w, b, dy = cases.draw_conv(name, case)
    r = oracle.round_f16
    y_o, dx_o, dw_o, db_o = oracle_all(oracle, case, r(x), r(w), r(b) if b is not None else None, r(dy))
    xd, dyd = dev(x, torch.float16, nhwc=True), dev(dy, torch.float16, nhwc=True)
    wd = dev(w, torch.float16)
    bd = dev(b, torch.float16) if b is not None else None
    y = ops.conv_forward(g, xd, wd, bd, layout="nhwc", math="f16")
    dx = ops.conv_backward_data(g, dyd, wd, layout="nhwc", math="f16")
    ops.device_status()
    assert_f16(host(y, nhwc=True), y_o, f"{name} y")
    assert_f16(host(dx, nhwc=True), dx_o, f"{name} dx")
    # the same layer in fp32 (3xTF32: patches per pass, weights streamed)
    y32_o, dx32_o, _, _ = oracle_all(oracle, case, x, w, b, dy)
    xd32, wd32, dyd32 = dev(x), dev(w), dev(dy)
    bd32 = dev(b) if b is not None else None
    y32 = shim_forward(case, xd32, wd32, bd32, F32, False)
    dx32, _ = shim_backward(case, dyd32, xd32, wd32, F32)
    ops.device_status()
    assert_f32(y32, y32_o, f"{name} y fp32")
    assert_f32(dx32, dx32_o, f"{name} dx fp32")


# Weight gradients whose taps each hold one 64-channel group (or, for few-channel inputs, one kernel row of
# packed windows) and whose other tensor has a multiple of 64 channels take the weight-gradient patch walk:
# all row tiles in TMEM, one haloed patch per 8 x 8 pixel K block.
WGRAD_PATCH_SHAPES = {
    "w_3x3_64_64":    (False, (2, 64, 23, 15, 64, 3, 3, (1, 1), (1, 1), (1, 1), (0, 0)), True, "normal"),
    "w_3x3_dil_128":  (False, (1, 32, 17, 24, 128, 3, 3, (1, 1), (2, 2), (2, 2), (0, 0)), True, "normal"),
    "w_stem_7x7_s2":  (False, (2, 3, 30, 26, 64, 7, 7, (2, 2), (3, 3), (1, 1), (0, 0)), True, "normal"),
    "w_rect_s21":     (False, (2, 48, 17, 19, 64, 2, 4, (2, 1), (0, 0), (1, 1), (0, 0)), False, "normal"),
    "w_convT_to_5":   (True,  (2, 64, 15, 16, 5, 4, 4, (2, 2), (1, 1), (1, 1), (0, 0)), True, "normal"),
    "w_5x5_192":      (False, (1, 40, 12, 16, 192, 5, 5, (1, 1), (2, 2), (1, 1), (0, 0)), True, "normal"),
}


@pytest.mark.parametrize("name", sorted(WGRAD_PATCH_SHAPES))
def test_wgrad_patch_walk_shapes(name, oracle):
    case = WGRAD_PATCH_SHAPES[name]
    g = geometry(case)
    x, w, b, dy = cases.draw_conv(name, case)
    r = oracle.round_f16
    _, _, dw_o, db_o = oracle_all(oracle, case, r(x), r(w), r(b) if b is not None else None, r(dy))
    xd, dyd = dev(x, torch.float16, nhwc=True), dev(dy, torch.float16, nhwc=True)
    dw, db = ops.conv_backward_weight(g, xd, dyd, layout="nhwc", math="f16")
    ops.device_status()
    assert_f32(host(dw), dw_o, f"{name} dw", tol=2e-5)
    assert_f32(host(db), db_o, f"{name} db", tol=2e-5)


@pytest.mark.parametrize("name", sorted(cases.CONV1D_CASES))
def test_reference_shaped_conv1d(name, golden_conv1d, oracle):
    """`_nectarml.tensor.conv.conv1d` ... `conv_transpose1d_backward_weight` in fp32 (3xTF32) against the
    oracle and the fixtures produced by the reference's own 1-D functions."""
    case = cases.CONV1D_CASES[name]
    transposed, (B, Ci, L, Co, K, s, p, d, op), _ = case
    x, w, b, dy = cases.draw_conv1d(name, case)
    Lo = dy.shape[2]
    if not transposed:
        y_o = oracle.conv1d(x, w, b, s, p, d)
        dx_o = oracle.conv1d_backward_input(dy, w, x.shape, s, p, d)
        dw_o = oracle.conv1d_backward_weight(dy, x, w.shape, s, p, d)
    else:
        y_o = oracle.conv_transpose1d(x, w, b, s, p, d, op)
        dx_o = oracle.conv_transpose1d_backward_input(dy, w, x.shape, s, p, d)
        dw_o = oracle.conv_transpose1d_backward_weight(dy, x, w.shape, s, p, d)
    xd, wd, dyd = dev(x), dev(w), dev(dy)
    bd = dev(b) if b is not None else None
    bp = bd.data_ptr() if bd is not None else 0
    if not transposed:
        y = fetch(conv.conv1d(xd.data_ptr(), wd.data_ptr(), bp, B, Ci, L, Co, K, s, p, d, 1, F32), (B, Co, Lo))
        dx = fetch(conv.conv1d_backward_input(dyd.data_ptr(), wd.data_ptr(), B, Ci, L, Co, K, Lo, s, p, d, 1, F32), (B, Ci, L))
        dw = fetch(conv.conv1d_backward_weight(dyd.data_ptr(), xd.data_ptr(), B, Ci, L, Co, K, Lo, s, p, d, F32), (Co, Ci, K))
    else:
        y = fetch(conv.conv_transpose1d(xd.data_ptr(), wd.data_ptr(), bp, B, Ci, L, Co, K, s, p, d, op, 1, F32), (B, Co, Lo))
        dx = fetch(conv.conv_transpose1d_backward_input(dyd.data_ptr(), wd.data_ptr(), B, Ci, L, Co, K, Lo, s, p, d, 1, F32),
                   (B, Ci, L))
        dw = fetch(conv.conv_transpose1d_backward_weight(dyd.data_ptr(), xd.data_ptr(), B, Ci, L, Co, K, Lo, s, p, d, F32),
                   (Ci, Co, K))
    ops.device_status()
    for got, orc, key in ((y, y_o, "y"), (dx, dx_o, "dx"), (dw, dw_o, "dw")):
        assert_f32(got, orc, f"{name} {key} vs oracle")
        assert_f32(got, golden_conv1d[f"{name}__{key}"], f"{name} {key} vs reference fixture")
    with pytest.raises(RuntimeError):  # grouped convolution is refused, as the reference asserts on CUDA
        conv.conv1d(xd.data_ptr(), wd.data_ptr(), bp, B, Ci, L, Co, K, s, p, d, 2, F32)


def test_config1_full_size(golden_config1, oracle):
    """benchmark configuration 1: Conv2d fp32 N=8 64->64 56x56 3x3 s1 p1, output, dX, dW and db."""
    case = cases.CONFIG1
    x, w, b, dy = cases.draw_conv("config1", case, cases.CONFIG1_SEED)
    y_o, dx_o, dw_o, db_o = oracle_all(oracle, case, x, w, b, dy)
    xd, wd, bd, dyd = dev(x), dev(w), dev(b), dev(dy)
    y = shim_forward(case, xd, wd, bd, F32, False)
    dx, dw = shim_backward(case, dyd, xd, wd, F32)
    g = geometry(case)
    db = host(ops.conv_backward_weight(g, xd, dyd, layout="nchw", math="3xtf32")[1])
    ops.device_status()
    assert_f32(y, y_o, "config1 y")
    assert_f32(dx, dx_o, "config1 dx")
    assert_f32(dw, dw_o, "config1 dw")
    assert_f32(db, db_o, "config1 db")
    gc = golden_config1
    assert_f32(y.reshape(-1)[gc["y_idx"]], gc["y_val"], "config1 y vs reference samples")
    assert_f32(dx.reshape(-1)[gc["dx_idx"]], gc["dx_val"], "config1 dx vs reference samples")
    assert_f32(dw.reshape(-1)[gc["dw_idx"]], gc["dw_val"], "config1 dw vs reference samples", tol=3e-5)
    assert_f32(db, gc["db"], "config1 db vs reference")


@pytest.mark.parametrize("name", sorted(cases.LINEAR_CASES))
def test_linear_fp32_and_fp16(name, golden_small, oracle):
    x, w, b, dy = cases.draw_linear(name, cases.LINEAR_CASES[name])
    xd, wd, bd, dyd = dev(x), dev(w), dev(b), dev(dy)
    y = host(ops.linear_forward(xd, wd, bd, math="3xtf32"))
    dx = host(ops.linear_backward_data(dyd, wd, math="3xtf32"))
    dw, db = [host(t) for t in ops.linear_backward_weight(xd, dyd, math="3xtf32")]
    ops.device_status()
    for got, key in ((y, "y"), (dx, "dx"), (dw, "dw"), (db, "db")):
        assert_f32(got, golden_small[f"{name}__{key}"], f"{name} {key}")
    r = oracle.round_f16
    y_o = oracle.linear_forward(r(x), r(w), r(b))
    dx_o, dw_o, db_o = oracle.linear_backward(r(x), r(w), r(dy))
    h = torch.float16
    y16 = host(ops.linear_forward(dev(x, h), dev(w, h), dev(b, h), math="f16"))
    dx16 = host(ops.linear_backward_data(dev(dy, h), dev(w, h), math="f16"))
    dw16, db16 = [host(t) for t in ops.linear_backward_weight(dev(x, h), dev(dy, h), math="f16")]
    ops.device_status()
    assert_f16(y16, y_o, f"{name} fp16 y")
    assert_f16(dx16, dx_o, f"{name} fp16 dx")
    assert_f32(dw16, dw_o, f"{name} fp16 dw", tol=2e-5)
    assert_f32(db16, db_o, f"{name} fp16 db", tol=2e-5)


@pytest.mark.parametrize("rows,d", [(4096, 512), (1000, 520)])
def test_linear_projection_shapes(rows, d, oracle):
    """benchmark configuration 2 family: X[rows, d] @ W^T[d, 4d] + b in fp16 with fp32 accumulation."""
    rng = np.random.default_rng(1236)
    x = rng.standard_normal((rows, d), dtype=np.float32)
    bound = np.sqrt(6.0 / (d + 4 * d))
    w = rng.uniform(-bound, bound, (4 * d, d)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, 4 * d).astype(np.float32)
    dy = rng.standard_normal((rows, 4 * d), dtype=np.float32)
    r = oracle.round_f16
    y_o = oracle.linear_forward(r(x), r(w), r(b))
    dx_o, dw_o, db_o = oracle.linear_backward(r(x), r(w), r(dy))
    h = torch.float16
    xd, wd, bd, dyd = dev(x, h), dev(w, h), dev(b, h), dev(dy, h)
    assert_f16(host(ops.linear_forward(xd, wd, bd)), y_o, "y")
    assert_f16(host(ops.linear_backward_data(dyd, wd)), dx_o, "dx")
    dw, db = ops.linear_backward_weight(xd, dyd)
    ops.device_status()
    assert_f32(host(dw), dw_o, "dw", tol=2e-5)
    assert_f32(host(db), db_o, "db", tol=2e-5)


def test_reference_shaped_matmul(oracle):
    """`_nectarml.tensor.matmul`: 2-D, the 4x8 @ 8x4 case of the reference's tests
    (tests/automatic/test_tensor_methods.py:237-249), and equal-batch 3-D operands."""
    rng = np.random.default_rng(5)
    for a_shape, b_shape in (((4, 8), (8, 4)), ((130, 72), (72, 200)), ((3, 33, 40), (3, 40, 24))):
        a = rng.standard_normal(a_shape, dtype=np.float32)
        b = rng.standard_normal(b_shape, dtype=np.float32)
        a32, b32 = dev(a), dev(b)
        ptr = _nectarml.tensor.matmul(a32.data_ptr(), b32.data_ptr(), list(a_shape), list(b_shape), F32)
        got = fetch(ptr, a_shape[:-1] + (b_shape[-1],))
        assert_f32(got, oracle.matmul(a, b), f"matmul {a_shape}x{b_shape}")
        a16, b16 = dev(a, torch.float16), dev(b, torch.float16)
        ptr = _nectarml.tensor.matmul(a16.data_ptr(), b16.data_ptr(), list(a_shape), list(b_shape), F16)
        got = fetch(ptr, a_shape[:-1] + (b_shape[-1],), np.float16)
        assert_f16(got, oracle.matmul(oracle.round_f16(a), oracle.round_f16(b)), f"matmul fp16 {a_shape}")
    ops.device_status()


def _twice(fn):
    a = fn()
    a = [t.clone() for t in (a if isinstance(a, tuple) else (a,))]
    b = fn()
    b = b if isinstance(b, tuple) else (b,)
    return all(torch.equal(u, v) for u, v in zip(a, b))


@pytest.mark.parametrize("name", ["c72", "s_conv_k4_s2", "s_convT_k4_s2", "w_3x3_64_64", "w_stem_7x7_s2", "w_convT_to_5",
                                  "p_3x3_128_32", "k4_s2"])
def test_every_result_is_bitwise_repeatable(name):
    """y, dx, dw and db of two identical calls are equal bit for bit, also where the K loop is split over
    CTAs (forward walk of the few-pixel layers, every weight gradient): the slices' partial sums go to
    planes that are added in a fixed order, never through atomics.  The reference's single cuBLAS GEMM per
    pass is repeatable too."""
    case = {**cases.CONV_CASES, **WALK_SHAPES, **WGRAD_PATCH_SHAPES}[name]
    g = geometry(case)
    x, w, b, dy = cases.draw_conv(name, case)
    h = torch.float16
    xd, dyd, wd = dev(x, h, nhwc=True), dev(dy, h, nhwc=True), dev(w, h)
    bd = dev(b, h) if b is not None else None
    assert _twice(lambda: ops.conv_forward(g, xd, wd, bd, layout="nhwc")), "y (fp16)"
    assert _twice(lambda: ops.conv_backward_data(g, dyd, wd, layout="nhwc")), "dx (fp16)"
    assert _twice(lambda: ops.conv_backward_weight(g, xd, dyd, layout="nhwc")), "dw, db (fp16)"
    x32, dy32, w32 = dev(x), dev(dy), dev(w)
    assert _twice(lambda: ops.conv_forward(g, x32, w32, dev(b) if b is not None else None, math="3xtf32")), "y (fp32)"
    assert _twice(lambda: ops.conv_backward_data(g, dy32, w32, math="3xtf32")), "dx (fp32)"
    assert _twice(lambda: ops.conv_backward_weight(g, x32, dy32, math="3xtf32")), "dw, db (fp32)"
    ops.device_status()


@pytest.mark.parametrize("rows,fin,fout", [(4096, 512, 2048), (3000, 264, 520)])
def test_linear_is_bitwise_repeatable(rows, fin, fout):
    """Linear at a split-K shape (the weight gradient of 4096 x 512 -> 2048 is cut into K slices)."""
    gen = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn(rows, fin, device=DEV, generator=gen).half()
    w = (torch.randn(fout, fin, device=DEV, generator=gen) * 0.05).half()
    b = torch.randn(fout, device=DEV, generator=gen).half()
    dy = torch.randn(rows, fout, device=DEV, generator=gen).half()
    assert _twice(lambda: ops.linear_forward(x, w, b))
    assert _twice(lambda: ops.linear_backward_data(dy, w))
    assert _twice(lambda: ops.linear_backward_weight(x, dy))
    ops.device_status()


@pytest.mark.parametrize("name", ["ref_basic", "ref_stride", "c72", "k4_s2", "k7_s2_p3", "ref_transpose", "t_k4_s2", "t_rect_dil"])
def test_reference_shaped_fp16_dtype_forward(name, oracle):
    """`dtype=Float16` tensors (the reference's run_conv2d<half> / run_conv_transpose2d<half>,
    nectarml/csrc/ops/tensor/conv/conv2d.cpp:71-211): NCHW fp16 in, NCHW fp16 out, no half_precision flag."""
    case = cases.CONV_CASES[name]
    x, w, b, dy = cases.draw_conv(name, case)
    r = oracle.round_f16
    y_o = oracle_all(oracle, case, r(x), r(w), r(b) if b is not None else None, dy)[0]
    h = torch.float16
    y = shim_forward(case, dev(x, h), dev(w, h), dev(b, h) if b is not None else None, F16, False)
    ops.device_status()
    assert y.dtype == np.float16
    assert_f16(y.astype(np.float32), y_o, f"{name} fp16-dtype y")


def test_matmul_2d_right_operand_is_shared_over_the_batch(oracle):
    """[B, T, d] @ [d, 4d]: the projection of an attention block.  The reference advances the 2-D right
    operand per batch entry and reads past its end (nectarml/csrc/ops/tensor/matmul.cpp:27,39); here it is
    shared, which is what `np.matmul` (the reference's CPU backend, nectarml/cpu/math.py:80-81) computes."""
    rng = np.random.default_rng(6)
    for a_shape, b_shape in (((3, 50, 64), (64, 256)), ((2, 4, 17, 40), (40, 24))):
        a = rng.standard_normal(a_shape, dtype=np.float32)
        b = rng.standard_normal(b_shape, dtype=np.float32)
        a32, b32 = dev(a), dev(b)
        ptr = _nectarml.tensor.matmul(a32.data_ptr(), b32.data_ptr(), list(a_shape), list(b_shape), F32)
        got = fetch(ptr, a_shape[:-1] + (b_shape[-1],))
        assert_f32(got, oracle.matmul(a, b), f"matmul {a_shape}x{b_shape}")
        a16, b16 = dev(a, torch.float16), dev(b, torch.float16)
        ptr = _nectarml.tensor.matmul(a16.data_ptr(), b16.data_ptr(), list(a_shape), list(b_shape), F16)
        got = fetch(ptr, a_shape[:-1] + (b_shape[-1],), np.float16)
        assert_f16(got, oracle.matmul(oracle.round_f16(a), oracle.round_f16(b)), f"matmul fp16 {a_shape}")
    ops.device_status()


def test_sm_limit_changes_the_plan_not_the_result(oracle):
    """nml_set_sm_limit (used while a collective shares the GPU): the kernels run on fewer SMs, tile and split-K
    plans are made for that count, results stay within tolerance of the oracle."""
    name = "w_3x3_64_64"
    case = WGRAD_PATCH_SHAPES[name]
    g = geometry(case)
    x, w, b, dy = cases.draw_conv(name, case)
    r = oracle.round_f16
    y_o, dx_o, dw_o, db_o = oracle_all(oracle, case, r(x), r(w), r(b), r(dy))
    h = torch.float16
    xd, dyd, wd, bd = dev(x, h, nhwc=True), dev(dy, h, nhwc=True), dev(w, h), dev(b, h)
    gen = torch.Generator(device=DEV).manual_seed(8)
    lx = torch.randn(4096, 512, device=DEV, generator=gen).half()
    ldy = torch.randn(4096, 2048, device=DEV, generator=gen).half()
    try:
        for limit in (140, 37, 1):
            ops.set_sm_limit(limit)
            assert_f16(host(ops.conv_forward(g, xd, wd, bd, layout="nhwc"), nhwc=True), y_o, f"y @ {limit} SMs")
            assert_f16(host(ops.conv_backward_data(g, dyd, wd, layout="nhwc"), nhwc=True), dx_o, f"dx @ {limit} SMs")
            dw, db = ops.conv_backward_weight(g, xd, dyd, layout="nhwc")
            assert_f32(host(dw), dw_o, f"dw @ {limit} SMs", tol=2e-5)
            assert_f32(host(db), db_o, f"db @ {limit} SMs", tol=2e-5)
            if limit > 1:
                ldw, ldb = ops.linear_backward_weight(lx, ldy)
                ref = ldy[:, :64].double().t() @ lx.double()
                assert torch.allclose(ldw[:64].double(), ref, rtol=1e-4, atol=2e-5 * float(ref.abs().max()))
            ops.device_status()
    finally:
        ops.set_sm_limit(0)


def test_weight_gradient_call_keeps_stream_order_and_records_into_a_graph():
    """A consumer queued on the caller's stream right after a weight-gradient call (no host synchronisation)
    sees the finished db, the call can be recorded into a CUDA graph, and repeated calls give the same bits."""
    gen = torch.Generator(device=DEV).manual_seed(21)
    x = torch.randn(4096, 512, device=DEV, generator=gen).half()
    dy = torch.randn(4096, 2048, device=DEV, generator=gen).half()
    want = dy.double().sum(0)
    dw = torch.empty(2048, 512, device=DEV)
    db = torch.empty(2048, device=DEV)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        copies = []
        for _ in range(3):
            db.fill_(float("nan"))
            ops.linear_backward_weight(x, dy, dw=dw, db=db)
            copies.append(db.clone())          # queued behind the call on the same stream
        stream.synchronize()
    for c in copies:
        assert torch.allclose(c.double(), want, rtol=1e-5, atol=1e-3)
        assert torch.equal(c, copies[0])
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    db.fill_(float("nan"))
    from nectarml_b200.train import capture_into
    with capture_into(graph):
        ops.linear_backward_weight(x, dy, dw=dw, db=db)
    db.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(db, copies[0])
    ops.device_status()


def test_workspace_too_small_is_reported():
    import ctypes as C
    from nectarml_b200 import _lib
    g = geometry(cases.CONV_CASES["c72"])
    x, w, b, dy = cases.draw_conv("c72", cases.CONV_CASES["c72"])
    xd, wd = dev(x), dev(w)
    y = torch.empty(g.act_shape("out", "nchw"), device=DEV)
    d = g.desc(_lib.NML_F32, "nchw", _lib.NML_F32, "nchw", _lib.NML_F32, "3xtf32", False)
    small = torch.empty(1024, dtype=torch.uint8, device=DEV)
    st = _lib.load().nml_conv_forward(C.byref(d), xd.data_ptr(), wd.data_ptr(), None, y.data_ptr(),
                                      small.data_ptr(), small.numel(), None)
    assert st == 2
    st = _lib.load().nml_conv_forward(C.byref(d), None, wd.data_ptr(), None, y.data_ptr(), None, 0, None)
    assert st == 1
