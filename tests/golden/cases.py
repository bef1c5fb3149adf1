"""Shared list of golden cases: geometry + how inputs are drawn.  Used by make_golden.py (which
runs the reference's own NumPy functions on them) and by the tests (which regenerate the same
inputs).  Geometry tuples: (B, C_in, H, W, C_out, KH, KW, stride, padding, dilation, output_padding).
"""
import numpy as np

# name -> (transposed, geometry, bias?, input distribution)
CONV_CASES = {
    # the shapes the reference's own tests use (tests/automatic/test_nn.py:459-548), inputs U(0.1, 0.9)
    "ref_basic":      (False, (2, 3, 16, 16, 8, 3, 3, (1, 1), (1, 1), (1, 1), (0, 0)), True, "uniform"),
    "ref_stride":     (False, (2, 3, 16, 16, 8, 3, 3, (2, 2), (1, 1), (1, 1), (0, 0)), True, "uniform"),
    "ref_no_bias":    (False, (2, 3, 8, 8, 8, 3, 3, (1, 1), (1, 1), (1, 1), (0, 0)), False, "uniform"),
    "ref_backward":   (False, (2, 3, 8, 8, 4, 3, 3, (1, 1), (1, 1), (1, 1), (0, 0)), True, "uniform"),
    "ref_transpose":  (True,  (2, 8, 8, 8, 4, 3, 3, (2, 2), (1, 1), (1, 1), (1, 1)), True, "uniform"),
    # edge cases the reference's tests do not reach
    "k1":             (False, (3, 20, 7, 9, 12, 1, 1, (1, 1), (0, 0), (1, 1), (0, 0)), True, "normal"),
    "k1_s2":          (False, (2, 16, 14, 14, 24, 1, 1, (2, 2), (0, 0), (1, 1), (0, 0)), False, "normal"),
    "k4_s2":          (False, (2, 6, 16, 16, 10, 4, 4, (2, 2), (1, 1), (1, 1), (0, 0)), True, "normal"),
    "k7_s2_p3":       (False, (1, 3, 20, 20, 8, 7, 7, (2, 2), (3, 3), (1, 1), (0, 0)), True, "normal"),
    "dilated":        (False, (2, 5, 13, 11, 7, 3, 3, (1, 1), (2, 2), (2, 2), (0, 0)), True, "normal"),
    "rect":           (False, (2, 4, 9, 12, 6, 3, 2, (2, 1), (1, 0), (1, 2), (0, 0)), True, "normal"),
    "pad_gt_kernel":  (False, (1, 2, 5, 5, 3, 3, 3, (1, 1), (3, 3), (1, 1), (0, 0)), True, "normal"),
    "single_pixel":   (False, (1, 9, 3, 3, 5, 3, 3, (1, 1), (0, 0), (1, 1), (0, 0)), True, "normal"),
    "c72":            (False, (2, 72, 8, 8, 40, 3, 3, (1, 1), (1, 1), (1, 1), (0, 0)), True, "normal"),
    "t_k4_s2":        (True,  (2, 6, 5, 5, 4, 4, 4, (2, 2), (1, 1), (1, 1), (0, 0)), True, "normal"),
    "t_s1":           (True,  (2, 5, 6, 7, 3, 3, 3, (1, 1), (1, 1), (1, 1), (0, 0)), False, "normal"),
    "t_rect_dil":     (True,  (1, 4, 5, 4, 6, 3, 2, (2, 3), (1, 1), (2, 1), (1, 1)), True, "normal"),
    "t_k2_s2":        (True,  (2, 7, 4, 4, 5, 2, 2, (2, 2), (0, 0), (1, 1), (0, 0)), True, "normal"),
}

# benchmark configuration 1: Conv2d fp32, N=8, 64->64, 56x56, 3x3 s1 p1; sampled (the full tensors are 6 MB each).
CONFIG1 = (False, (8, 64, 56, 56, 64, 3, 3, (1, 1), (1, 1), (1, 1), (0, 0)), True, "config1")
CONFIG1_SEED = 1235
CONFIG1_SAMPLES = 4096

# 1-D convolutions: name -> (transposed, (B, C_in, L, C_out, K, stride, padding, dilation, output_padding), bias?)
CONV1D_CASES = {
    "c1_basic":   (False, (2, 3, 24, 8, 3, 1, 1, 1, 0), True),
    "c1_stride":  (False, (2, 6, 31, 10, 5, 2, 2, 1, 0), True),
    "c1_dilated": (False, (1, 5, 40, 7, 3, 1, 3, 3, 0), False),
    "c1_wide":    (False, (2, 72, 50, 40, 4, 3, 0, 1, 0), True),
    "c1_t_s2":    (True,  (2, 8, 13, 4, 4, 2, 1, 1, 1), True),
    "c1_t_s1":    (True,  (1, 5, 17, 6, 3, 1, 1, 2, 0), False),
}


def conv1d_as_2d(case):
    """The same layer as a CONV_CASES-style tuple over an image of height 1."""
    transposed, (B, Ci, L, Co, K, s, p, d, op), has_bias = case
    return (transposed, (B, Ci, 1, L, Co, 1, K, (1, s), (0, p), (1, d), (0, op)), has_bias, "normal")


def draw_conv1d(name, case):
    """x [B, C_in, L], w [C_out, C_in, K] ([C_in, C_out, K] transposed), bias or None, dy [B, C_out, L_out]."""
    x, w, b, dy = draw_conv(name, conv1d_as_2d(case))
    return x[:, :, 0, :].copy(), w[:, :, 0, :].copy(), b, dy[:, :, 0, :].copy()


LINEAR_CASES = {  # rows, in_features, out_features
    "lin_small": (4, 8, 4),
    "lin_odd": (37, 24, 19),
    "lin_mid": (128, 96, 160),
}


def out_hw(transposed, geom):
    B, Ci, H, W, Co, KH, KW, s, p, d, op = geom
    if transposed:
        return ((H - 1) * s[0] - 2 * p[0] + d[0] * (KH - 1) + 1 + op[0],
                (W - 1) * s[1] - 2 * p[1] + d[1] * (KW - 1) + 1 + op[1])
    return ((H + 2 * p[0] - d[0] * (KH - 1) - 1) // s[0] + 1, (W + 2 * p[1] - d[1] * (KW - 1) - 1) // s[1] + 1)


def draw_conv(name, case, seed=None):
    """x, w, bias (or None), dy -- float32, deterministic per case name."""
    transposed, geom, has_bias, dist = case
    B, Ci, H, W, Co, KH, KW, s, p, d, op = geom
    if seed is None:
        seed = 7000 + sum(ord(c) * (i + 1) for i, c in enumerate(name))
    rng = np.random.default_rng(seed)
    Ho, Wo = out_hw(transposed, geom)
    wshape = (Ci, Co, KH, KW) if transposed else (Co, Ci, KH, KW)
    if dist == "uniform":
        x = rng.uniform(0.1, 0.9, (B, Ci, H, W)).astype(np.float32)
        w = rng.uniform(-0.5, 0.5, wshape).astype(np.float32)
        b = rng.uniform(-0.5, 0.5, Co).astype(np.float32)
        dy = rng.uniform(0.1, 0.9, (B, Co, Ho, Wo)).astype(np.float32)
    elif dist == "config1":
        # X, dY ~ N(0,1); W and b Kaiming-uniform U(+-1/sqrt(C_in*KH*KW)) as nn.Conv2d initialises
        bound = 1.0 / np.sqrt(Ci * KH * KW)
        x = rng.standard_normal((B, Ci, H, W), dtype=np.float32)
        w = rng.uniform(-bound, bound, wshape).astype(np.float32)
        b = rng.uniform(-bound, bound, Co).astype(np.float32)
        dy = rng.standard_normal((B, Co, Ho, Wo), dtype=np.float32)
    else:
        x = rng.standard_normal((B, Ci, H, W), dtype=np.float32)
        w = (rng.standard_normal(wshape, dtype=np.float32) * 0.2).astype(np.float32)
        b = rng.standard_normal(Co, dtype=np.float32)
        dy = rng.standard_normal((B, Co, Ho, Wo), dtype=np.float32)
    return x, w, (b if has_bias else None), dy


def draw_linear(name, shape):
    rows, fin, fout = shape
    rng = np.random.default_rng(9000 + sum(ord(c) for c in name))
    x = rng.standard_normal((rows, fin), dtype=np.float32)
    bound = np.sqrt(6.0 / (fin + fout))  # Xavier-uniform
    w = rng.uniform(-bound, bound, (fout, fin)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, fout).astype(np.float32)
    dy = rng.standard_normal((rows, fout), dtype=np.float32)
    return x, w, b, dy


def sample_indices(n, count, seed):
    rng = np.random.default_rng(seed)
    return np.sort(rng.choice(n, size=min(count, n), replace=False))
