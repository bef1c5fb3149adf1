"""Full-size checks at the benchmark shapes (ResNet-style conv sweep at batch 256, Linear projections),
where running the CPU oracle on the whole tensor would take hours.  Two size-independent tools:

* sampled outputs: a few thousand output elements are recomputed in float64 on the host straight
  from the definition (nectarml/cpu/conv/conv2d.py:163-180, 260-271, 326-334) and compared;
* the adjoint identity  <dY, conv(X)> = <dX, X> = <dW, W>  (no bias), which ties forward,
  input-gradient and weight-gradient of one layer together like a checksum of checksums.
"""
import numpy as np
import pytest
import torch

from nectarml_b200 import ops
from nectarml_b200.ops import ConvGeometry

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# (c_in, hw, c_out, k, stride, pad) at batch 256 -- benchmark configuration 3
LAYERS = {
    "7x7s2_3_64_224": (3, 224, 64, 7, 2, 3),
    "3x3_64_64_56": (64, 56, 64, 3, 1, 1),
    "1x1_256_64_56": (256, 56, 64, 1, 1, 0),
    "3x3s2_128_128_28": (128, 28, 128, 3, 2, 1),
    "1x1s2_1024_2048_14": (1024, 14, 2048, 1, 2, 0),
}
BATCH = 256


def _sample_forward(x, w, s, p, idx, ho, wo):
    """x NHWC, w [co,ci,kh,kw] (float64 numpy); idx rows of (n, oh, ow, co)."""
    N, H, W, C = x.shape
    k = w.shape[2]
    out = np.zeros(len(idx))
    for j, (n, oh, ow, co) in enumerate(idx):
        acc = 0.0
        for kh in range(k):
            ih = oh * s - p + kh
            if ih < 0 or ih >= H:
                continue
            for kw in range(k):
                iw = ow * s - p + kw
                if 0 <= iw < W:
                    acc += float(np.dot(x[n, ih, iw, :], w[co, :, kh, kw]))
        out[j] = acc
    return out


def _sample_dgrad(dy, w, s, p, idx):
    """dy NHWC, idx rows of (n, h, w, ci)."""
    N, Ho, Wo, Co = dy.shape
    k = w.shape[2]
    out = np.zeros(len(idx))
    for j, (n, h, ww, ci) in enumerate(idx):
        acc = 0.0
        for kh in range(k):
            nh = h + p - kh
            if nh % s or not (0 <= nh // s < Ho):
                continue
            for kw in range(k):
                nw = ww + p - kw
                if nw % s or not (0 <= nw // s < Wo):
                    continue
                acc += float(np.dot(dy[n, nh // s, nw // s, :], w[:, ci, kh, kw]))
        out[j] = acc
    return out


def _sample_wgrad(x, dy, s, p, idx):
    """idx rows of (co, ci, kh, kw); full reduction over batch and pixels, vectorised."""
    N, H, W, C = x.shape
    _, Ho, Wo, Co = dy.shape
    out = np.zeros(len(idx))
    for j, (co, ci, kh, kw) in enumerate(idx):
        oh = np.arange(Ho)
        ow = np.arange(Wo)
        ih = oh * s - p + kh
        iw = ow * s - p + kw
        vh = (ih >= 0) & (ih < H)
        vw = (iw >= 0) & (iw < W)
        xs = x[:, ih[vh]][:, :, iw[vw], ci].astype(np.float64)
        ds = dy[:, oh[vh]][:, :, ow[vw], co].astype(np.float64)
        out[j] = float((xs * ds).sum())
    return out


@pytest.mark.parametrize("name", sorted(LAYERS))
def test_resnet_shape_full_batch(name):
    ci, hw, co, k, s, p = LAYERS[name]
    g = ConvGeometry(BATCH, ci, hw, hw, co, k, k, (s, s), (p, p))
    ho, wo = g.out_hw()
    gen = torch.Generator(device=DEV).manual_seed(1237)
    x = torch.randn(BATCH, hw, hw, ci, device=DEV, generator=gen).half()
    dy = torch.randn(BATCH, ho, wo, co, device=DEV, generator=gen).half()
    w = (torch.randn(co, ci, k, k, device=DEV, generator=gen) * float(np.sqrt(2.0 / (ci * k * k)))).half()
    y = ops.conv_forward(g, x, w, None, layout="nhwc")
    dx = ops.conv_backward_data(g, dy, w, layout="nhwc")
    dw, db = ops.conv_backward_weight(g, x, dy, layout="nhwc")
    ops.device_status()

    # adjoint identity (sums in float64 on the device; fp16 rounding of y and dx averages out)
    a = float((dy.double() * y.double()).sum())
    b = float((dx.double() * x.double()).sum())
    c = float((dw.double() * w.double()).sum())
    scale = float(np.sqrt(float((dy.double() ** 2).sum()) * float((y.double() ** 2).sum())))
    assert abs(a - b) <= 2e-4 * scale and abs(a - c) <= 2e-4 * scale, (a, b, c, scale)
    assert torch.allclose(db.double(), dy.double().sum(dim=(0, 1, 2)), rtol=1e-4, atol=1e-2 * float(np.sqrt(BATCH * ho * wo)))

    # sampled elements against the definition in float64
    rng = np.random.default_rng(7)
    xh, dyh, wh = x.cpu().numpy().astype(np.float64), dy.cpu().numpy().astype(np.float64), w.cpu().numpy().astype(np.float64)
    ns = 600
    idx = np.stack([rng.integers(0, BATCH, ns), rng.integers(0, ho, ns), rng.integers(0, wo, ns), rng.integers(0, co, ns)], 1)
    idx[:8, 1:3] = [[0, 0], [0, wo - 1], [ho - 1, 0], [ho - 1, wo - 1], [0, 1], [1, 0], [ho - 1, wo - 2], [ho - 2, wo - 1]]
    ref = _sample_forward(xh, wh, s, p, idx, ho, wo)
    got = y.cpu().numpy().astype(np.float64)[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]]
    assert np.all(np.abs(got - ref) <= 1e-3 + 1e-2 * np.abs(ref)), np.abs(got - ref).max()

    idx = np.stack([rng.integers(0, BATCH, ns), rng.integers(0, hw, ns), rng.integers(0, hw, ns), rng.integers(0, ci, ns)], 1)
    idx[:4, 1:3] = [[0, 0], [0, hw - 1], [hw - 1, 0], [hw - 1, hw - 1]]
    ref = _sample_dgrad(dyh, wh, s, p, idx)
    got = dx.cpu().numpy().astype(np.float64)[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]]
    assert np.all(np.abs(got - ref) <= 1e-3 + 1e-2 * np.abs(ref)), np.abs(got - ref).max()

    nw = 24
    idx = np.stack([rng.integers(0, co, nw), rng.integers(0, ci, nw), rng.integers(0, k, nw), rng.integers(0, k, nw)], 1)
    ref = _sample_wgrad(xh, dyh, s, p, idx)
    got = dw.cpu().numpy().astype(np.float64)[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]]
    # fp32 accumulation of up to 3.2 million fp16 products per element (tensor-core accumulation
    # truncates, split-K slices are added with fp32 atomics): 1e-3 of the largest gradient entry
    assert np.all(np.abs(got - ref) <= 1e-3 * np.abs(dw.cpu().numpy()).max()), np.abs(got - ref).max()


@pytest.mark.parametrize("rows,d", [(16384, 1024), (16384, 2048)])
def test_linear_projection_full_size(rows, d):
    """benchmark configuration 2 at its large shapes: sampled rows against float64 and the adjoint identity."""
    gen = torch.Generator(device=DEV).manual_seed(1236)
    x = torch.randn(rows, d, device=DEV, generator=gen).half()
    w = ((torch.rand(4 * d, d, device=DEV, generator=gen) * 2 - 1) * float(np.sqrt(6.0 / (5 * d)))).half()
    b = ((torch.rand(4 * d, device=DEV, generator=gen) * 2 - 1) * 0.1).half()
    dy = torch.randn(rows, 4 * d, device=DEV, generator=gen).half()
    y = ops.linear_forward(x, w, b)
    dx = ops.linear_backward_data(dy, w)
    dw, db = ops.linear_backward_weight(x, dy)
    ops.device_status()
    r = torch.randint(0, rows, (64,), device=DEV)
    ref = x[r].double() @ w.double().t() + b.double()
    assert torch.allclose(y[r].double(), ref, rtol=1e-2, atol=1e-3)
    ref = dy[r].double() @ w.double()
    assert torch.allclose(dx[r].double(), ref, rtol=1e-2, atol=1e-3)
    c = torch.randint(0, 4 * d, (32,), device=DEV)
    ref = dy[:, c].double().t() @ x.double()
    assert torch.allclose(dw[c].double(), ref, rtol=1e-4, atol=2e-5 * float(ref.abs().max()))
    assert torch.allclose(db.double(), dy.double().sum(0), rtol=1e-4, atol=1e-2 * float(np.sqrt(rows)))
    a = float((dy.double() * (y.double() - b.double())).sum())
    bb = float((dx.double() * x.double()).sum())
    cc = float((dw.double() * w.double()).sum())
    scale = float(np.sqrt(float((dy.double() ** 2).sum()) * float((y.double() ** 2).sum())))
    assert abs(a - bb) <= 2e-4 * scale and abs(a - cc) <= 2e-4 * scale, (a, bb, cc, scale)
