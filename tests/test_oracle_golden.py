"""The CPU oracle against fixtures produced by the reference's own NumPy functions
(tests/golden/make_golden.py).  Forward values follow the reference's loop order exactly, so
they must match bit for bit; where the reference sums through np.einsum / matmul (unspecified
order) a few fp32 ulps of the accumulated magnitude are allowed."""
import numpy as np
import pytest

import cases


def _geom(case):
    transposed, geom, has_bias, _ = case
    B, Ci, H, W, Co, KH, KW, s, p, d, op = geom
    return transposed, (B, Ci, H, W), Co, (KH, KW), s, p, d, op


def _close(a, b, scale_tol=2e-6):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert a.shape == b.shape
    return np.abs(a - b).max() <= scale_tol * max(np.abs(b).max(), 1e-30)


@pytest.mark.parametrize("name", sorted(cases.CONV_CASES))
def test_inputs_reproduce(name, golden_small):
    x, w, b, dy = cases.draw_conv(name, cases.CONV_CASES[name])
    got = np.array([x.sum(dtype=np.float64), w.sum(dtype=np.float64), dy.sum(dtype=np.float64)])
    assert np.array_equal(got, golden_small[f"{name}__insum"]), "seeded inputs differ from those the fixtures saw"


@pytest.mark.parametrize("name", sorted(cases.CONV_CASES))
def test_conv_oracle_matches_reference(name, golden_small, oracle):
    case = cases.CONV_CASES[name]
    transposed, xs, Co, k, s, p, d, op = _geom(case)
    x, w, b, dy = cases.draw_conv(name, case)
    if not transposed:
        y = oracle.conv2d(x, w, b, s, p, d)
        dx = oracle.conv2d_backward_input(dy, w, x.shape, s, p, d)
        dw = oracle.conv2d_backward_weight(dy, x, w.shape, s, p, d)
        # same loop order and fp32 arithmetic as the reference's _conv2d: bit-exact
        assert np.array_equal(y, golden_small[f"{name}__y"])
    else:
        y = oracle.conv_transpose2d(x, w, b, s, p, d, op)
        dx = oracle.conv_transpose2d_backward_input(dy, w, x.shape, s, p, d)
        dw = oracle.conv_transpose2d_backward_weight(dy, x, w.shape, s, p, d)
        assert _close(y, golden_small[f"{name}__y"])
        # the reference computes this gradient with its _conv2d loop: bit-exact again
        assert np.array_equal(dx, golden_small[f"{name}__dx"])
    assert _close(dx, golden_small[f"{name}__dx"])
    assert _close(dw, golden_small[f"{name}__dw"])
    assert _close(oracle.bias_grad(dy), golden_small[f"{name}__db"])


def _oracle_conv1d(oracle, case, x, w, b, dy):
    transposed, (B, Ci, L, Co, K, s, p, d, op), _ = case
    if not transposed:
        return (oracle.conv1d(x, w, b, s, p, d), oracle.conv1d_backward_input(dy, w, x.shape, s, p, d),
                oracle.conv1d_backward_weight(dy, x, w.shape, s, p, d))
    return (oracle.conv_transpose1d(x, w, b, s, p, d, op), oracle.conv_transpose1d_backward_input(dy, w, x.shape, s, p, d),
            oracle.conv_transpose1d_backward_weight(dy, x, w.shape, s, p, d))


@pytest.mark.parametrize("name", sorted(cases.CONV1D_CASES))
def test_conv1d_oracle_matches_reference(name, golden_conv1d, oracle):
    """The 1-D wrappers of the oracle against the reference's own 1-D functions (nectarml/cpu/conv/conv1d.py)."""
    case = cases.CONV1D_CASES[name]
    x, w, b, dy = cases.draw_conv1d(name, case)
    got = np.array([x.sum(dtype=np.float64), w.sum(dtype=np.float64), dy.sum(dtype=np.float64)])
    assert np.array_equal(got, golden_conv1d[f"{name}__insum"]), "seeded inputs differ from those the fixtures saw"
    y, dx, dw = _oracle_conv1d(oracle, case, x, w, b, dy)
    if not case[0]:
        # same accumulation order as the reference's scalar loop (bias, input channel, kernel position): bit-exact
        assert np.array_equal(y, golden_conv1d[f"{name}__y"])
    assert _close(y, golden_conv1d[f"{name}__y"])
    assert _close(dx, golden_conv1d[f"{name}__dx"])
    assert _close(dw, golden_conv1d[f"{name}__dw"])
    assert _close(dy.sum(axis=(0, 2)), golden_conv1d[f"{name}__db"])


@pytest.mark.parametrize("name", sorted(cases.LINEAR_CASES))
def test_linear_oracle_matches_reference(name, golden_small, oracle):
    x, w, b, dy = cases.draw_linear(name, cases.LINEAR_CASES[name])
    y = oracle.linear_forward(x, w, b)
    dx, dw, db = oracle.linear_backward(x, w, dy)
    assert np.array_equal(y, golden_small[f"{name}__y"])
    assert np.array_equal(dx, golden_small[f"{name}__dx"])
    assert np.array_equal(dw, golden_small[f"{name}__dw"])
    assert _close(db, golden_small[f"{name}__db"])


def test_config1_oracle_matches_reference(golden_config1, oracle):
    """benchmark configuration 1 at full size (Conv2d fp32, N=8, 64->64, 56x56, 3x3 s1 p1) against samples
    of the reference's own outputs."""
    case = cases.CONFIG1
    x, w, b, dy = cases.draw_conv("config1", case, cases.CONFIG1_SEED)
    g = golden_config1
    got = np.array([x.sum(dtype=np.float64), w.sum(dtype=np.float64), dy.sum(dtype=np.float64)])
    assert np.array_equal(got, g["insum"])
    y = oracle.conv2d(x, w, b, (1, 1), (1, 1), (1, 1)).reshape(-1)
    assert np.array_equal(y[g["y_idx"]], g["y_val"])
    assert y.sum(dtype=np.float64) == g["y_sum"][0]
    dx = oracle.conv2d_backward_input(dy, w, x.shape, (1, 1), (1, 1), (1, 1)).reshape(-1)
    assert _close(dx[g["dx_idx"]], g["dx_val"], 3e-6)
    dw = oracle.conv2d_backward_weight(dy, x, w.shape, (1, 1), (1, 1), (1, 1)).reshape(-1)
    assert _close(dw[g["dw_idx"]], g["dw_val"], 3e-5)  # 25088-term fp32 sums, order differs from einsum
    assert _close(oracle.bias_grad(dy), g["db"], 3e-6)


def test_output_size_formulas(oracle):
    # nectarml/nn/functional/conv.py:406-407 and :479-482
    assert oracle.conv_out_hw(224, 224, 7, 7, (2, 2), (3, 3), (1, 1)) == (112, 112)
    assert oracle.conv_out_hw(56, 56, 3, 3, (1, 1), (1, 1), (1, 1)) == (56, 56)
    assert oracle.conv_out_hw(14, 14, 1, 1, (2, 2), (0, 0), (1, 1)) == (7, 7)
    assert oracle.conv_transpose_out_hw(8, 8, 3, 3, (2, 2), (1, 1), (1, 1), (1, 1)) == (16, 16)
    assert oracle.conv_transpose_out_hw(128, 128, 4, 4, (2, 2), (1, 1), (1, 1), (0, 0)) == (256, 256)
