"""Pins the TMA behaviour the implicit-GEMM address math relies on: a box may start at a
negative or out-of-range coordinate and reads zeros there, and with an element stride s the
i-th element of a box dimension is taken at coordinate start + i*s."""
import numpy as np
import pytest
import torch

from nectarml_b200 import ops

pytestmark = pytest.mark.gpu
N, H, W, C = 2, 6, 10, 16


def expected(tn, box, es, co):
    cnt = [(b + s - 1) // s for b, s in zip(box, es)]
    o = np.zeros((cnt[3], cnt[2], cnt[1], cnt[0]), dtype=tn.dtype)
    for n in range(cnt[3]):
        for h in range(cnt[2]):
            for w in range(cnt[1]):
                for c in range(cnt[0]):
                    nn, hh, ww, cc = co[3] + n * es[3], co[2] + h * es[2], co[1] + w * es[1], co[0] + c * es[0]
                    if 0 <= nn < N and 0 <= hh < H and 0 <= ww < W and 0 <= cc < C:
                        o[n, h, w, c] = tn[nn, hh, ww, cc]
    return o.reshape(-1)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("box,es,co", [
    ((16, 4, 2, 1), (1, 1, 1, 1), (0, 1, 1, 0)),
    ((16, 4, 2, 1), (1, 1, 1, 1), (0, -1, -1, 0)),
    ((16, 4, 4, 2), (1, 1, 1, 1), (0, 8, 4, 1)),
    ((16, 8, 4, 1), (1, 2, 2, 1), (0, 0, 0, 0)),
    ((16, 8, 4, 1), (1, 2, 2, 1), (0, 1, 1, 0)),
    ((16, 8, 4, 1), (1, 2, 2, 1), (0, -1, -1, 0)),
    ((16, 8, 4, 1), (1, 2, 2, 1), (0, -2, -3, 0)),
    ((32, 16, 8, 1), (1, 1, 1, 1), (0, 0, 0, 0)),
])
def test_tma_box_semantics(dtype, box, es, co):
    t = (torch.arange(N * H * W * C, device="cuda:0") % 2048).to(dtype).reshape(N, H, W, C).contiguous()
    got = ops.tma_box(t, box, es, co).cpu().numpy()
    ops.device_status()
    assert np.array_equal(got, expected(t.cpu().numpy(), box, es, co))
