"""One training step of the two conv nets against the same step composed from plain fp32 torch ops.

The nets are shrunk (narrow ResNet with one block per stage on 32x32 images; a 5-level U-Net on 32x32 images)
so that the fp32 reference runs in moments; every layer type, the residual / skip plumbing, the fused
batch-norm + activation kernels, the flat gradient buffer, micro-batch accumulation and the fused
SGD-momentum update are the ones the full-size steps use.  The reference keeps fp16 storage between layers
like the step does (values rounded through fp16, gradients straight through) and takes the derivative
pattern of every ReLU / LeakyReLU / max-pool / |.| from the step's own forward pass (see `gate`).
Tolerances: loss 1e-2 relative; every gradient tensor 2e-2 relative in the Frobenius norm (the gradients
themselves are still rounded to fp16 layer by layer).
"""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from nectarml_b200 import ops, train
from nectarml_b200.train import ACT_LEAKY, ACT_NONE, ACT_RELU, BatchNormAct, Conv, Linear

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def q(t):
    """fp16 storage between layers, as the step under test keeps it: the value is rounded through fp16, the
    gradient passes straight through."""
    return t + (t.half().float() - t).detach()


def gate(t, seen, act):
    """The activation with its derivative pattern taken from the output `seen` of the step under test (NHWC).
    Rounding makes ~0.05 % of a deep fp16 net's pre-activations change sign against any other evaluation; each
    such flip is a jump in the gradient, and together they are ~3 % of noise per ReLU layer (10 % over the depth
    of these nets) that says nothing about the wiring.  With the pattern fixed, what is compared is the chain of
    linear maps the backward pass has to implement."""
    if act == ACT_NONE:
        return t
    pos = (seen.permute(0, 3, 1, 2) > 0).float()
    return t * pos if act == ACT_RELU else t * (pos + 0.2 * (1.0 - pos))


class RefParams:
    """fp32 leaf copies of the (fp16-rounded) parameters, indexed like the store."""

    def __init__(self, store):
        self.store = store
        self.t = [store.w16(i).float().clone().requires_grad_(True)
                  for i in range(len(store.shapes))]
        for i in range(len(store.shapes)):  # BN affine parameters are read in fp32 by the kernels
            if len(store.shapes[i]) == 1:
                self.t[i] = store.w32(i).clone().requires_grad_(True)

    def conv(self, l: Conv, x):
        w = self.t[l.ia]
        b = self.t[l.ib].half().float() if l.ib is not None else None
        if l.transposed:
            return q(F.conv_transpose2d(x, w, b, stride=l.stride, padding=l.pad))
        return q(F.conv2d(x, w, b, stride=l.stride, padding=l.pad))

    def bn(self, l: BatchNormAct, x, act, seen, residual=None):
        y = F.batch_norm(x, None, None, self.t[l.ia], self.t[l.ib], training=True, eps=l.eps)
        if residual is not None:
            y = y + residual
        return q(gate(y, seen, act))


def _compare(store, ref, scale, what, tol):
    errs = []
    for i in range(len(store.shapes)):
        g = ref.t[i].grad
        if g is None:
            continue
        got = store.g32(i).double() / scale
        errs.append((float((got - g.double()).norm() / max(float(g.double().norm()), 1e-12)), i, store.shapes[i]))
    errs.sort(reverse=True)
    print(what, "gradient errors, worst first:", [(f"{e:.2e}", i, sh) for e, i, sh in errs[:6]], "median", f"{errs[len(errs) // 2][0]:.2e}")
    assert errs[0][0] <= tol, f"{what}: gradients off, worst first: {[(f'{e:.2e}', i, sh) for e, i, sh in errs[:8]]}"
    return errs[0][0]


def _resnet_ref(net, p, x, trace):
    seen = iter(trace)
    stem_out = next(seen)
    x = p.bn(net.stem_bn, p.conv(net.stem, x), ACT_RELU, stem_out)
    # max-pool with the window winners of the step under test
    _, idx = F.max_pool2d(stem_out.permute(0, 3, 1, 2).float(), 3, 2, 1, return_indices=True)
    next(seen)
    x = x.flatten(2).gather(2, idx.flatten(2)).view(idx.shape)
    for blk in net.blocks:
        idn = x
        y = p.bn(blk["b1"], p.conv(blk["c1"], x), ACT_RELU, next(seen))
        y = p.bn(blk["b2"], p.conv(blk["c2"], y), ACT_RELU, next(seen))
        if "cd" in blk:
            idn = p.bn(blk["bd"], p.conv(blk["cd"], x), ACT_NONE, next(seen))
        x = p.bn(blk["b3"], p.conv(blk["c3"], y), ACT_RELU, next(seen), residual=idn)
    pooled = q(x.mean(dim=(2, 3)))
    return q(F.linear(pooled, p.t[net.fc.ia], p.t[net.fc.ib].half().float()))


def test_resnet_step_matches_the_fp32_composition():
    torch.manual_seed(0)
    net = train.ResNet50(DEV, num_classes=24, blocks=(1, 1, 1, 1), width=16)
    net.init(seed=3)
    n = 16
    x = torch.randn(n, 64, 64, 3, device=DEV).half()
    labels = torch.randint(0, 24, (n,), device=DEV)
    step = train.TrainStep(net, "cross_entropy", lr=0.05, momentum=0.9, weight_decay=1e-4, loss_scale=8192.0)
    ref = RefParams(net.store)
    before = net.store.p32.clone()

    # two micro-batches of 8 against one reference pass per micro-batch (BN statistics are per micro-batch)
    net.store.trace = []
    loss = step([(x[:8].contiguous(), labels[:8]), (x[8:].contiguous(), labels[8:])], global_count=n, optimize=False)
    ops.device_status()
    trace, net.store.trace = net.store.trace, None
    per_pass = len(trace) // 2
    ref_loss = 0.0
    for k, lo in enumerate((0, 8)):
        out = _resnet_ref(net, ref, x[lo:lo + 8].float().permute(0, 3, 1, 2), trace[k * per_pass:(k + 1) * per_pass])
        l = F.cross_entropy(out, labels[lo:lo + 8], reduction="sum") / n
        l.backward()
        ref_loss += float(l.detach())
    assert abs(float(loss) - ref_loss) <= 1e-2 * abs(ref_loss), (float(loss), ref_loss)
    worst = _compare(net.store, ref, step.loss_scale, "resnet", 2e-2)

    # the fused update: g = grad / scale + wd * p; v = 0.9 * 0 + g; p -= lr * v; fp16 copy refreshed
    grads = net.store.grad.clone()
    net.store.sgd_step(step.lr, step.momentum, step.wd, 1.0 / step.loss_scale)
    want = before - step.lr * (grads / step.loss_scale + step.wd * before)
    assert torch.allclose(net.store.p32, want, rtol=1e-6, atol=1e-7)
    assert torch.equal(net.store.p16, net.store.p32.half())
    assert int(net.store.found_inf) == 0
    # an overflowed gradient leaves every parameter alone
    snap = net.store.p32.clone()
    net.store.grad[5] = float("inf")
    net.store.sgd_step(step.lr, step.momentum, step.wd, 1.0 / step.loss_scale)
    assert int(net.store.found_inf) == 1 and torch.equal(net.store.p32, snap)
    print(f"worst gradient error {worst:.3e}")


def _unet_ref(net, p, x, trace):
    seen = iter(trace)
    skips = []
    for i, (conv, bn) in enumerate(net.down):
        y = p.conv(conv, x)
        x = p.bn(bn, y, ACT_LEAKY, next(seen)) if bn is not None else q(gate(y, next(seen), ACT_LEAKY if i == 0 else ACT_RELU))
        skips.append(x)
    skips.pop()
    for i, (conv, bn) in enumerate(net.up):
        if i > 0:
            x = torch.cat((x, skips.pop()), dim=1)
        x = p.bn(bn, p.conv(conv, x), ACT_RELU, next(seen))
    x = torch.cat((x, skips.pop()), dim=1)
    return q(torch.tanh(p.conv(net.final, x)))


def test_unet_step_matches_the_fp32_composition():
    torch.manual_seed(1)
    net = train.Pix2PixGenerator(DEV, in_channels=3, features=8)
    # five levels instead of eight, so that a 32x32 image reaches 1x1 at the bottleneck
    net.down = net.down[:4] + [net.down[-1]]
    net.up = [net.up[0]] + net.up[4:]
    net.init(seed=5)
    for i, shape in enumerate(net.store.shapes):  # larger weights than N(0, 0.02): the tiny net would output ~0
        if len(shape) == 4:
            net.store.w32(i).mul_(8.0)
    net.store.sync_half()
    n = 6
    x = (torch.rand(n, 32, 32, 3, device=DEV) * 2 - 1).half()
    target = (torch.rand(n, 32, 32, 3, device=DEV) * 2 - 1).half()
    step = train.TrainStep(net, "l1", loss_scale=8192.0)
    ref = RefParams(net.store)
    net.store.trace = []
    loss = step([(x, target)], global_count=target.numel(), optimize=False)
    ops.device_status()
    trace, net.store.trace = net.store.trace, None
    out = _unet_ref(net, ref, x.float().permute(0, 3, 1, 2), trace)
    tgt = target.float().permute(0, 3, 1, 2)
    ref_loss = (out - tgt).abs().sum() / target.numel()
    # the L1 loss with the signs the step under test saw (its own output is the last entry of the trace)
    sign = torch.sign(trace[-1].float().permute(0, 3, 1, 2) - tgt)
    ((out - tgt) * sign).sum().div(target.numel()).backward()
    assert abs(float(loss) - float(ref_loss)) <= 1e-2 * abs(float(ref_loss)), (float(loss), float(ref_loss))
    worst = _compare(net.store, ref, step.loss_scale, "unet", 2e-2)
    print(f"worst gradient error {worst:.3e}")


def test_max_pool_matches_torch():
    gen = torch.Generator(device=DEV).manual_seed(4)
    for (n, h, w, c, k, s_, p) in ((2, 13, 10, 16, 3, 2, 1), (1, 8, 8, 64, 2, 2, 0), (3, 7, 9, 8, 3, 1, 1), (2, 12, 12, 24, 5, 3, 2)):
        x = torch.randn(n, h, w, c, device=DEV, generator=gen).half().requires_grad_(True)
        y = train.max_pool(x, k, s_, p)
        dy = torch.randn_like(y)
        y.backward(dy)
        xr = x.detach().float().permute(0, 3, 1, 2).requires_grad_(True)
        yr = F.max_pool2d(xr, k, s_, p)
        yr.backward(dy.float().permute(0, 3, 1, 2))
        assert torch.equal(y.float(), yr.permute(0, 2, 3, 1))
        # (random fp16 inputs: ties inside a window are rare but exist; both sides then pick the first tap)
        assert torch.allclose(x.grad.float(), xr.grad.permute(0, 2, 3, 1), rtol=1e-3, atol=1e-3)
    ops.device_status()


def test_bn_act_kernels_match_torch_and_repeat_bitwise():
    """nml_bn_forward / nml_bn_backward on their own: all three activations, with and without a residual."""
    import ctypes as C
    from nectarml_b200 import _lib
    gen = torch.Generator(device=DEV).manual_seed(2)
    for (rows_shape, c) in (((3, 9, 7), 64), ((2, 5, 5), 2048), ((4, 6, 6), 24)):
        for act in (ACT_NONE, ACT_RELU, ACT_LEAKY):
            for with_res in (False, True):
                x = (torch.randn(*rows_shape, c, device=DEV, generator=gen) * 2 + 0.5).half()
                res = torch.randn(*rows_shape, c, device=DEV, generator=gen).half() if with_res else None
                dy = torch.randn(*rows_shape, c, device=DEV, generator=gen).half()
                store = train.ParamStore(DEV)
                layer = BatchNormAct(store, c)
                store.finalize(1)
                layer.gamma.copy_(torch.rand(c, device=DEV, generator=gen) + 0.5)
                layer.beta.copy_(torch.randn(c, device=DEV, generator=gen))
                token = torch.zeros((), device=DEV, requires_grad=True)
                outs = []
                for _ in range(2):
                    store.begin_backward(False)
                    xr = x.clone().requires_grad_(True)
                    rr = res.clone().requires_grad_(True) if with_res else None
                    y = layer(xr, token, act, residual=rr)
                    y.backward(dy)
                    outs.append((y.detach().clone(), xr.grad.clone(), rr.grad.clone() if with_res else None,
                                 store.grad.clone()))
                for a, b in zip(outs[0], outs[1]):
                    assert a is None or torch.equal(a, b), "not bitwise repeatable"
                xf = x.float().requires_grad_(True)
                rf = res.float().requires_grad_(True) if with_res else None
                gm = layer.gamma.clone().requires_grad_(True)
                bt = layer.beta.clone().requires_grad_(True)
                t = F.batch_norm(xf.permute(0, 3, 1, 2), None, None, gm, bt, training=True, eps=layer.eps).permute(0, 2, 3, 1)
                if with_res:
                    t = t + rf
                t = t if act == ACT_NONE else F.relu(t) if act == ACT_RELU else F.leaky_relu(t, 0.2)
                t.backward(dy.float())
                y, dx, dres, grads = outs[0]
                assert torch.allclose(y.float(), t, rtol=1e-2, atol=1e-2)
                assert float((dx.float() - xf.grad).norm() / xf.grad.norm()) < 1e-2
                if with_res:
                    assert float((dres.float() - rf.grad).norm() / rf.grad.norm()) < 1e-2
                assert float((store.g32(layer.ia) - gm.grad).norm() / gm.grad.norm()) < 1e-2
                assert float((store.g32(layer.ib) - bt.grad).norm() / bt.grad.norm()) < 1e-2
    ops.device_status()


def test_graph_captures_replay_the_eager_step_bit_for_bit():
    """CUDA-graph capture of forward + backward (one graph, and the U-Net's decoder | encoder split used to
    overlap the gradient exchange) against the eager micro-batch: every kernel is deterministic, so the flat
    gradient buffer must come out bit-identical."""
    torch.manual_seed(2)
    net = train.Pix2PixGenerator(DEV, in_channels=3, features=8)
    net.init(seed=7)
    for i, shape in enumerate(net.store.shapes):
        if len(shape) == 4:
            net.store.w32(i).mul_(8.0)
    net.store.sync_half()
    x = (torch.rand(2, 256, 256, 3, device=DEV) * 2 - 1).half()
    target = (torch.rand(2, 256, 256, 3, device=DEV) * 2 - 1).half()
    step = train.TrainStep(net, "l1", loss_scale=8192.0)
    count = target.numel()
    loss = step.micro_batch(x, target, count, first=True, last=False)
    ops.device_status()
    want, want_loss = net.store.grad.clone(), float(loss)
    assert float(want.abs().max()) > 0

    graph, gloss = step.capture(x, target, count)[False]
    net.store.grad.zero_()
    graph.replay()
    ops.device_status()
    assert torch.equal(net.store.grad, want) and float(gloss) == want_loss

    split = step.capture_split(x, target, count)
    net.store.grad.zero_()
    step.replay_split(split)
    ops.device_status()
    assert torch.equal(net.store.grad, want) and float(split[2]) == want_loss
    cut = net.frontier_first_param
    assert 0 < cut < net.store.n and cut == net.store.offsets[net.up[0][0].ia]
