"""Full-size checks at the benchmark shapes (ResNet-style conv sweep and ResNet-50 layers at batch 256,
Pix2Pix U-Net generator layers at batch 64 incl. the transposed ones, Linear projections),
where running the CPU oracle on the whole tensor would take hours.  Two size-independent tools:

* sampled outputs: a few thousand output elements are recomputed in float64 on the host straight
  from the definition (nectarml/cpu/conv/conv2d.py:163-180, 260-271, 326-334) and compared;
* the adjoint identity  <dY, conv(X)> = <dX, X> = <dW, W>  (no bias), which ties forward,
  input-gradient and weight-gradient of one layer together like a checksum of checksums.
The transposed layers follow nectarml/cpu/conv/conv2d.py:196-230 (forward), 280-300, 349-376.
"""
import numpy as np
import pytest
import torch

from nectarml_b200 import ops
from nectarml_b200.ops import ConvGeometry

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# name -> (c_in, input h = w, c_out, k, stride, pad, transposed, batch, weight std)
def _kaiming(ci, k):
    return float(np.sqrt(2.0 / (ci * k * k)))


LAYERS = {
    # benchmark configuration 3: ResNet-style shapes at batch 256, Kaiming-normal weights
    "7x7s2_3_64_224": (3, 224, 64, 7, 2, 3, False, 256, _kaiming(3, 7)),
    "3x3_64_64_56": (64, 56, 64, 3, 1, 1, False, 256, _kaiming(64, 3)),
    "1x1_256_64_56": (256, 56, 64, 1, 1, 0, False, 256, _kaiming(256, 1)),
    "3x3s2_128_128_28": (128, 28, 128, 3, 2, 1, False, 256, _kaiming(128, 3)),
    "1x1s2_1024_2048_14": (1024, 14, 2048, 1, 2, 0, False, 256, _kaiming(1024, 1)),
    # benchmark configuration 5: the other distinct ResNet-50 layer shapes at batch 256
    "r50_1x1_64_256_56": (64, 56, 256, 1, 1, 0, False, 256, _kaiming(64, 1)),
    "r50_3x3s2_256_256_28": (256, 28, 256, 3, 2, 1, False, 256, _kaiming(256, 3)),
    "r50_1x1_512_2048_7": (512, 7, 2048, 1, 1, 0, False, 256, _kaiming(512, 1)),
    # benchmark configuration 4: Pix2Pix U-Net generator layers at batch 64, 4x4 s2 p1, weights N(0, 0.02)
    "p2p_conv_3_64_256": (3, 256, 64, 4, 2, 1, False, 64, 0.02),
    "p2p_conv_64_128_128": (64, 128, 128, 4, 2, 1, False, 64, 0.02),
    "p2p_conv_512_512_16": (512, 16, 512, 4, 2, 1, False, 64, 0.02),
    "p2p_conv_512_512_4": (512, 4, 512, 4, 2, 1, False, 64, 0.02),
    "p2p_conv_512_512_2": (512, 2, 512, 4, 2, 1, False, 64, 0.02),
    "p2p_convT_512_512_1": (512, 1, 512, 4, 2, 1, True, 64, 0.02),
    "p2p_convT_1024_512_4": (1024, 4, 512, 4, 2, 1, True, 64, 0.02),
    "p2p_convT_1024_256_16": (1024, 16, 256, 4, 2, 1, True, 64, 0.02),
    "p2p_convT_256_64_64": (256, 64, 64, 4, 2, 1, True, 64, 0.02),
    "p2p_convT_128_3_128": (128, 128, 3, 4, 2, 1, True, 64, 0.02),
}


def _sample_forward(x, w, s, p, idx):
    """Strided read: out[n, oh, ow, co] = sum x[n, oh*s-p+kh, ow*s-p+kw, :] . w[co, :, kh, kw].
    x NHWC, w [co, ci, kh, kw]; idx rows of (n, oh, ow, co).  Conv2d forward, ConvTranspose2d input-gradient."""
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
                    acc += float(np.dot(x[n, ih, iw, :].astype(np.float64), w[co, :, kh, kw].astype(np.float64)))
        out[j] = acc
    return out


def _sample_gather(dy, w, s, p, idx):
    """Gather: out[n, h, w, ci] = sum over taps with (h+p-kh) % s == 0 of dy[n, (h+p-kh)/s, (w+p-kw)/s, :] . w[:, ci, kh, kw].
    dy NHWC, idx rows of (n, h, w, ci).  Conv2d input-gradient, ConvTranspose2d forward."""
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
                acc += float(np.dot(dy[n, nh // s, nw // s, :].astype(np.float64), w[:, ci, kh, kw].astype(np.float64)))
        out[j] = acc
    return out


def _sample_wgrad(big, small, s, p, idx):
    """out[a, b, kh, kw] = sum over n, oh, ow of small[n, oh, ow, a] * big[n, oh*s-p+kh, ow*s-p+kw, b]
    (Conv2d: big = x, small = dy, a = c_out, b = c_in; ConvTranspose2d: big = dy, small = x, a = c_in, b = c_out)."""
    N, H, W, _ = big.shape
    _, Ho, Wo, _ = small.shape
    out = np.zeros(len(idx))
    for j, (a, b, kh, kw) in enumerate(idx):
        oh = np.arange(Ho)
        ow = np.arange(Wo)
        ih = oh * s - p + kh
        iw = ow * s - p + kw
        vh = (ih >= 0) & (ih < H)
        vw = (iw >= 0) & (iw < W)
        xs = big[:, ih[vh]][:, :, iw[vw], b].astype(np.float64)
        ds = small[:, oh[vh]][:, :, ow[vw], a].astype(np.float64)
        out[j] = float((xs * ds).sum())
    return out


@pytest.mark.parametrize("name", sorted(LAYERS))
def test_benchmark_layer_at_full_size(name):
    ci, hw, co, k, s, p, tr, batch, std = LAYERS[name]
    g = ConvGeometry(batch, ci, hw, hw, co, k, k, (s, s), (p, p), transposed=tr)
    ho, wo = g.out_hw()
    gen = torch.Generator(device=DEV).manual_seed(1237)
    x = torch.randn(batch, hw, hw, ci, device=DEV, generator=gen).half()
    dy = torch.randn(batch, ho, wo, co, device=DEV, generator=gen).half()
    w = (torch.randn(*g.weight_shape(), device=DEV, generator=gen) * std).half()
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
    assert torch.allclose(db.double(), dy.double().sum(dim=(0, 1, 2)), rtol=1e-4, atol=1e-2 * float(np.sqrt(batch * ho * wo)))

    # sampled elements against the definition in float64
    rng = np.random.default_rng(7)
    xh, dyh, wh = x.cpu().numpy(), dy.cpu().numpy(), w.cpu().numpy()
    yh, dxh, dwh = y.cpu().numpy(), dx.cpu().numpy(), dw.cpu().numpy()
    ns = 400

    def positions(n_, h_, w_, c_):
        idx = np.stack([rng.integers(0, n_, ns), rng.integers(0, h_, ns), rng.integers(0, w_, ns), rng.integers(0, c_, ns)], 1)
        corners = [[0, 0], [0, w_ - 1], [h_ - 1, 0], [h_ - 1, w_ - 1], [0, min(1, w_ - 1)], [min(1, h_ - 1), 0],
                   [h_ - 1, max(w_ - 2, 0)], [max(h_ - 2, 0), w_ - 1]]
        idx[:8, 1:3] = corners
        return idx

    idx = positions(batch, ho, wo, co)
    ref = (_sample_gather if tr else _sample_forward)(xh, wh, s, p, idx)
    got = yh[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]].astype(np.float64)
    assert np.all(np.abs(got - ref) <= 1e-3 + 1e-2 * np.abs(ref)), ("y", np.abs(got - ref).max())

    idx = positions(batch, hw, hw, ci)
    ref = (_sample_forward if tr else _sample_gather)(dyh, wh, s, p, idx)
    got = dxh[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]].astype(np.float64)
    assert np.all(np.abs(got - ref) <= 1e-3 + 1e-2 * np.abs(ref)), ("dx", np.abs(got - ref).max())

    nw = 24
    d0, d1 = g.weight_shape()[:2]
    idx = np.stack([rng.integers(0, d0, nw), rng.integers(0, d1, nw), rng.integers(0, k, nw), rng.integers(0, k, nw)], 1)
    ref = _sample_wgrad(dyh, xh, s, p, idx) if tr else _sample_wgrad(xh, dyh, s, p, idx)
    got = dwh[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]].astype(np.float64)
    # fp32 accumulation of up to 3.2 million fp16 products per element (the tensor core's accumulation
    # truncates): 1e-3 of the largest gradient entry
    assert np.all(np.abs(got - ref) <= 1e-3 * np.abs(dwh).max()), ("dw", np.abs(got - ref).max())


def test_resnet50_classifier_head_full_size():
    """benchmark configuration 5: Linear 2048 -> 1000 at batch 256 (out_features not a multiple of 64)."""
    gen = torch.Generator(device=DEV).manual_seed(1238)
    rows, fin, fout = 256, 2048, 1000
    x = torch.randn(rows, fin, device=DEV, generator=gen).half()
    w = ((torch.rand(fout, fin, device=DEV, generator=gen) * 2 - 1) * float(1 / np.sqrt(fin))).half()
    b = ((torch.rand(fout, device=DEV, generator=gen) * 2 - 1) * float(1 / np.sqrt(fin))).half()
    dy = torch.randn(rows, fout, device=DEV, generator=gen).half()
    y = ops.linear_forward(x, w, b)
    dx = ops.linear_backward_data(dy, w)
    dw, db = ops.linear_backward_weight(x, dy)
    ops.device_status()
    assert torch.allclose(y.double(), x.double() @ w.double().t() + b.double(), rtol=1e-2, atol=1e-3)
    assert torch.allclose(dx.double(), dy.double() @ w.double(), rtol=1e-2, atol=1e-3)
    ref = dy.double().t() @ x.double()
    assert torch.allclose(dw.double(), ref, rtol=1e-4, atol=2e-5 * float(ref.abs().max()))
    assert torch.allclose(db.double(), dy.double().sum(0), rtol=1e-5, atol=1e-3)


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
