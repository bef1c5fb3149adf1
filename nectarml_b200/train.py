"""Training steps of the two conv nets the benchmark configurations name, built on the contraction path.

* ``ResNet50``  -- bottleneck blocks [3, 4, 6, 3], widths 64-2048, BatchNorm + ReLU, 1000-way Linear head
  (the reference's example: examples/resnet/model.py:4-97; step: examples/resnet/train.py:57-77 --
  autocast forward, scaled backward, unscale, SGD-momentum step).
* ``Pix2PixGenerator`` -- 8 Conv2d 4x4 s2 p1 down, 8 ConvTranspose2d 4x4 s2 p1 up with skip concatenation,
  BatchNorm + LeakyReLU(0.2) / ReLU, tanh output (examples/pix2pix/generator.py:54-170; weights N(0, 0.02)).

What runs where: every Conv2d / ConvTranspose2d / Linear, forward, input-gradient and weight-gradient, is the
C ABI's descriptor API on fp16 NHWC tensors that stay in that layout between layers; BatchNorm with the
activation and residual add that follow it, the finiteness check and the SGD-momentum update are the
library's own kernels (``nml_bn_*``, ``nml_grads_check``, ``nml_sgd_momentum_step``).  torch supplies device
memory, the autograd tape that orders the calls, and the few remaining small ops (pooling, concatenation,
tanh, the loss).  Parameters live in ONE flat fp32 buffer with an fp16 copy for the kernels; their gradients
are written by the weight-gradient kernels straight into ONE flat fp32 buffer, whose buckets are
all-reduced over NCCL as the backward pass completes them (weight gradient before input gradient in every
layer, so the exchange starts as early as it can).
"""
from __future__ import annotations

import contextlib
import ctypes as C
import gc
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _lib, ops
from .ops import ConvGeometry

ACT_NONE, ACT_RELU, ACT_LEAKY = 0, 1, 2

# Stream captures here are checked per thread: the capturing thread issues only capture-safe calls, while the
# NCCL watchdog thread of torch.distributed polls the events of earlier collectives whenever it likes, which a
# capture in "global" mode takes for an error (the capture is then invalidated, every so many runs).
CAPTURE_MODE = "thread_local"


@contextlib.contextmanager
def capture_into(graph, pool=None):
    """torch.cuda.graph with the garbage collector held off: a dead reference cycle that owns an older
    CUDAGraph would otherwise be collected at some allocation inside the capture, and destroying a graph
    while a stream is capturing invalidates the capture."""
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        kw = {"pool": pool} if pool is not None else {}
        with torch.cuda.graph(graph, capture_error_mode=CAPTURE_MODE, **kw):
            yield
    finally:
        if was_enabled:
            gc.enable()


# ------------------------------------------------------------------ parameters --
class ParamStore:
    """Flat fp32 parameters + fp16 copy + flat fp32 gradients + momentum, all with the same offsets."""

    def __init__(self, device) -> None:
        self.device = torch.device(device)
        self.shapes: List[Tuple[int, ...]] = []
        self.offsets: List[int] = []
        self.n = 0
        self.p32 = self.p16 = self.grad = self.vel = None
        self.accumulate = False          # True from the second micro-batch of a step on
        self.scratch: Optional[torch.Tensor] = None
        self.layer_ranges: List[Tuple[int, int]] = []   # (first element, end) of every layer, forward order
        self.bucket_bounds: List[int] = []
        self.world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        self.pending: List = []
        self.found_inf = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.communicate = True
        self.flops = 0.0                 # algorithmic FLOPs of the contraction passes since it was last zeroed
        self.trace: Optional[list] = None  # when a list: every nonlinearity's output is appended (test support)

    def record(self, t):
        if self.trace is not None:
            self.trace.append(t.detach())
        return t

    def add(self, shape: Sequence[int]) -> int:
        assert self.p32 is None, "parameters are registered before finalize()"
        self.shapes.append(tuple(shape))
        self.offsets.append(self.n)
        cnt = 1
        for d in shape:
            cnt *= d
        self.n += (cnt + 63) // 64 * 64   # keep every view 256-byte aligned
        return len(self.shapes) - 1

    def finalize(self, n_buckets: int = 4) -> None:
        mk = lambda dt: torch.zeros(self.n, dtype=dt, device=self.device)
        self.p32, self.p16, self.grad, self.vel = mk(torch.float32), mk(torch.float16), mk(torch.float32), mk(torch.float32)
        biggest = max(int(torch.tensor(s).prod()) for s in self.shapes)
        self.scratch = torch.empty(biggest, dtype=torch.float32, device=self.device)
        # buckets: contiguous ranges of the flat gradient, cut at layer boundaries into n_buckets of similar size
        starts = sorted(a for a, _ in self.layer_ranges)
        self.bucket_bounds = [0]
        for k in range(1, n_buckets):
            target = self.n * k // n_buckets
            cut = min(starts, key=lambda e: abs(e - target))
            if self.bucket_bounds[-1] < cut < self.n:
                self.bucket_bounds.append(cut)
        self.bucket_bounds.append(self.n)
        self._bucket_left = []
        self._exchange = False
        # SMs left to NCCL while an all-reduce may be in flight (the contraction kernels are persistent, one CTA
        # per SM; see nml_set_sm_limit)
        self.sm_reserve = 16
        self.sms = torch.cuda.get_device_properties(self.device).multi_processor_count if self.device.type == "cuda" else 0

    def _view(self, buf, i):
        cnt = 1
        for d in self.shapes[i]:
            cnt *= d
        return buf[self.offsets[i]:self.offsets[i] + cnt].view(self.shapes[i])

    def w32(self, i): return self._view(self.p32, i)
    def w16(self, i): return self._view(self.p16, i)
    def g32(self, i): return self._view(self.grad, i)

    def sync_half(self) -> None:
        self.p16.copy_(self.p32)

    # ---- step bookkeeping
    def begin_backward(self, last_micro_batch: bool) -> None:
        nb = len(self.bucket_bounds) - 1
        self._bucket_left = [0] * nb
        for (a, e) in self.layer_ranges:
            self._bucket_left[self._bucket_of(a)] += 1
        self._exchange = last_micro_batch and self.world > 1 and self.communicate

    def _bucket_of(self, elem: int) -> int:
        for b in range(len(self.bucket_bounds) - 1):
            if self.bucket_bounds[b] <= elem < self.bucket_bounds[b + 1]:
                return b
        return len(self.bucket_bounds) - 2

    def layer_done(self, first_elem: int) -> None:
        """Called when a layer has written its gradients; all-reduces the layer's bucket once it is complete."""
        b = self._bucket_of(first_elem)
        self._bucket_left[b] -= 1
        if self._bucket_left[b] == 0 and self._exchange:
            lo, hi = self.bucket_bounds[b], self.bucket_bounds[b + 1]
            self.pending.append(dist.all_reduce(self.grad[lo:hi], async_op=True))
            if self.sm_reserve and self.sms:
                ops.set_sm_limit(self.sms - self.sm_reserve)

    def wait_exchange(self) -> None:
        for p in self.pending:
            p.wait()
        if self.pending and self.sm_reserve and self.sms:
            ops.set_sm_limit(0)
        self.pending = []

    def sgd_step(self, lr: float, momentum: float, weight_decay: float, inv_scale: float) -> None:
        """Finiteness check + SGD-momentum update of every parameter (and of the fp16 copy): two launches."""
        lib = _lib.load()
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.nml_grads_check(self.grad.data_ptr(), self.n, inv_scale, self.found_inf.data_ptr(), st))
        _lib.check(lib.nml_sgd_momentum_step(self.p32.data_ptr(), self.grad.data_ptr(), self.vel.data_ptr(),
                                             self.p16.data_ptr(), self.n, lr, momentum, 0.0, weight_decay, inv_scale,
                                             self.found_inf.data_ptr(), st))


_bn_ws = ops.Workspace()


def _bn_workspace(rows: int, c: int, device):
    need = C.c_size_t()
    _lib.check(_lib.load().nml_bn_workspace_size(rows, c, C.byref(need)))
    return _bn_ws.get(need.value, device)


# ------------------------------------------------------------------ autograd nodes --
class _ConvFn(torch.autograd.Function):
    """Conv2d / ConvTranspose2d on fp16 NHWC through the descriptor API; the weight gradient goes straight
    into the flat gradient buffer (before the input gradient, so that its bucket can leave early)."""

    @staticmethod
    def forward(ctx, x, token, layer):
        g = layer.geometry(x)
        y = ops.conv_forward(g, x, layer.w16, layer.b16, layout="nhwc")
        pix = x.shape[1] * x.shape[2] if layer.transposed else y.shape[1] * y.shape[2]  # a transposed layer multiplies per input pixel
        layer.store.flops += (3 if layer.needs_dx else 2) * 2.0 * x.shape[0] * pix * g.c_out * g.c_in * g.kh * g.kw
        ctx.layer, ctx.g = layer, g
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        layer, g = ctx.layer, ctx.g
        (x,) = ctx.saved_tensors
        dy = dy.contiguous()
        layer.weight_gradient(lambda dw, db: ops.conv_backward_weight(g, x, dy, layout="nhwc", dw=dw, db=db,
                                                                        want_bias_grad=db is not None))
        dx = ops.conv_backward_data(g, dy, layer.w16, layout="nhwc") if layer.needs_dx else None
        return dx, None, None


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, token, layer):
        y = ops.linear_forward(x, layer.w16, layer.b16)
        layer.store.flops += 3 * 2.0 * x.shape[0] * x.shape[1] * y.shape[1]
        ctx.layer = layer
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        layer = ctx.layer
        (x,) = ctx.saved_tensors
        dy = dy.contiguous()
        layer.weight_gradient(lambda dw, db: ops.linear_backward_weight(x, dy, dw=dw, db=db, want_bias_grad=db is not None))
        return ops.linear_backward_data(dy, layer.w16), None, None


class _BnActFn(torch.autograd.Function):
    """y = act(batchnorm(x) [+ residual]) over the rows of an NHWC tensor (training statistics)."""

    @staticmethod
    def forward(ctx, x, residual, token, layer, act):
        rows, c = x.numel() // x.shape[-1], x.shape[-1]
        y = torch.empty_like(x)
        mean = torch.empty(c, dtype=torch.float32, device=x.device)
        rstd = torch.empty(c, dtype=torch.float32, device=x.device)
        wp, wb = _bn_workspace(rows, c, x.device)
        _lib.check(_lib.load().nml_bn_forward(x.data_ptr(), rows, c, layer.gamma.data_ptr(), layer.beta.data_ptr(),
                                              residual.data_ptr() if residual is not None else None, act, 0.2, layer.eps,
                                              y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), wp, wb,
                                              torch.cuda.current_stream().cuda_stream))
        ctx.layer, ctx.act, ctx.has_res = layer, act, residual is not None
        ctx.save_for_backward(x, y, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        layer = ctx.layer
        x, y, mean, rstd = ctx.saved_tensors
        dy = dy.contiguous()
        rows, c = x.numel() // x.shape[-1], x.shape[-1]
        dx = torch.empty_like(x)
        dres = torch.empty_like(x) if ctx.has_res else None
        wp, wb = _bn_workspace(rows, c, x.device)

        def run(dgamma, dbeta):
            _lib.check(_lib.load().nml_bn_backward(dy.data_ptr(), y.data_ptr(), x.data_ptr(), rows, c, layer.gamma.data_ptr(),
                                                   mean.data_ptr(), rstd.data_ptr(), ctx.act, 0.2, dx.data_ptr(),
                                                   dres.data_ptr() if dres is not None else None, dgamma.data_ptr(),
                                                   dbeta.data_ptr(), wp, wb, torch.cuda.current_stream().cuda_stream))
        layer.weight_gradient(run)
        return dx, dres, None, None, None


class _MaxPoolFn(torch.autograd.Function):
    """Max pooling on NHWC fp16 (window winners recorded in the forward, gathered in the backward)."""

    @staticmethod
    def forward(ctx, x, k, stride, pad):
        n, h, w, c = x.shape
        ho, wo = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        y = torch.empty(n, ho, wo, c, dtype=x.dtype, device=x.device)
        index = torch.empty(n, ho, wo, c, dtype=torch.uint8, device=x.device)
        _lib.check(_lib.load().nml_maxpool_forward(x.data_ptr(), n, h, w, c, k, stride, pad, y.data_ptr(), index.data_ptr(),
                                                   torch.cuda.current_stream().cuda_stream))
        ctx.geom = (n, h, w, c, k, stride, pad)
        ctx.save_for_backward(index)
        return y

    @staticmethod
    def backward(ctx, dy):
        (index,) = ctx.saved_tensors
        n, h, w, c, k, stride, pad = ctx.geom
        dy = dy.contiguous()
        dx = torch.empty(n, h, w, c, dtype=dy.dtype, device=dy.device)
        _lib.check(_lib.load().nml_maxpool_backward(dy.data_ptr(), index.data_ptr(), n, h, w, c, k, stride, pad, dx.data_ptr(),
                                                    torch.cuda.current_stream().cuda_stream))
        return dx, None, None, None


def max_pool(x, k, stride, pad):
    return _MaxPoolFn.apply(x, k, stride, pad)


# ------------------------------------------------------------------ layers --
class _Layer:
    """A parameterised layer: two parameter slots (weight-like, bias-like) in the ParamStore."""

    def __init__(self, store: ParamStore, shape_a, shape_b) -> None:
        self.store = store
        self.ia = store.add(shape_a)
        self.ib = store.add(shape_b) if shape_b is not None else None
        first = store.offsets[self.ia]
        last = self.ib if self.ib is not None else self.ia
        store.layer_ranges.append((first, store.offsets[last]))
        self.first = first

    def weight_gradient(self, run) -> None:
        """run(dw, db) writes fresh gradients; they replace or (later micro-batches) add to the flat buffer."""
        s = self.store
        ga = s.g32(self.ia)
        gb = s.g32(self.ib) if self.ib is not None else None
        if not s.accumulate:
            run(ga, gb)
        else:
            ta = s.scratch[:ga.numel()].view(ga.shape)
            tb = torch.empty_like(gb) if gb is not None else None
            run(ta, tb)
            ga.add_(ta)
            if gb is not None:
                gb.add_(tb)
        s.layer_done(self.first)


class Conv(_Layer):
    def __init__(self, store, c_in, c_out, k, stride, pad, bias=False, transposed=False, needs_dx=True):
        wshape = (c_in, c_out, k, k) if transposed else (c_out, c_in, k, k)
        super().__init__(store, wshape, (c_out,) if bias else None)
        self.c_in, self.c_out, self.k, self.stride, self.pad, self.transposed = c_in, c_out, k, stride, pad, transposed
        self.needs_dx = needs_dx

    @property
    def w16(self): return self.store.w16(self.ia)
    @property
    def b16(self): return self.store.w16(self.ib) if self.ib is not None else None

    def geometry(self, x) -> ConvGeometry:
        n, h, w, c = x.shape
        assert c == self.c_in, (c, self.c_in)
        return ConvGeometry(n, c, h, w, self.c_out, self.k, self.k, (self.stride, self.stride), (self.pad, self.pad),
                            transposed=self.transposed)

    def __call__(self, x, token):
        return _ConvFn.apply(x, token, self)


class Linear(_Layer):
    def __init__(self, store, fin, fout):
        super().__init__(store, (fout, fin), (fout,))

    @property
    def w16(self): return self.store.w16(self.ia)
    @property
    def b16(self): return self.store.w16(self.ib)

    def __call__(self, x, token):
        return _LinearFn.apply(x, token, self)


class BatchNormAct(_Layer):
    def __init__(self, store, c, eps=1e-5):
        super().__init__(store, (c,), (c,))
        self.eps = eps

    @property
    def gamma(self): return self.store.w32(self.ia)
    @property
    def beta(self): return self.store.w32(self.ib)

    def __call__(self, x, token, act=ACT_RELU, residual=None):
        return self.store.record(_BnActFn.apply(x, residual, token, self, act))


# ------------------------------------------------------------------ models --
class _Net:
    split_backward = False   # True for nets whose forward() sets `frontier` (see TrainStep.capture_split)

    def __init__(self, device):
        self.device = torch.device(device)
        self.store = ParamStore(device)
        # an input that requires grad, so that autograd runs the backward of layers whose data input does not
        self.token = torch.zeros((), device=device, requires_grad=True)
        # Activations at which a split backward pass stops (set by forward() of nets that support it).  Never
        # kept across steps: tensors of an earlier, uncaptured pass that die INSIDE a later stream capture
        # invalidate the capture (their allocator bookkeeping records events on the streams they crossed).
        self.frontier = None

    def _finish(self, n_buckets):
        self.store.finalize(n_buckets)

    def parameters_init(self, gen: torch.Generator):
        raise NotImplementedError


class ResNet50(_Net):
    """Bottleneck ResNet [3, 4, 6, 3]: 7x7 s2 p3 stem + BN + ReLU + 3x3 s2 p1 max-pool, stride on the 3x3
    convolution of a block (as examples/resnet/model.py:22-26), global average pool, Linear 2048 -> classes."""

    def __init__(self, device, num_classes=1000, blocks=(3, 4, 6, 3), width=64, image_channels=3):
        super().__init__(device)
        s = self.store
        self.stem = Conv(s, image_channels, width, 7, 2, 3, needs_dx=False)
        self.stem_bn = BatchNormAct(s, width)
        self.blocks = []
        c_in = width
        for stage, n in enumerate(blocks):
            c_mid = width * 2 ** stage
            for b in range(n):
                stride = 2 if (b == 0 and stage > 0) else 1
                blk = {"c1": Conv(s, c_in, c_mid, 1, 1, 0), "b1": BatchNormAct(s, c_mid),
                       "c2": Conv(s, c_mid, c_mid, 3, stride, 1), "b2": BatchNormAct(s, c_mid),
                       "c3": Conv(s, c_mid, c_mid * 4, 1, 1, 0), "b3": BatchNormAct(s, c_mid * 4)}
                if b == 0:
                    blk["cd"] = Conv(s, c_in, c_mid * 4, 1, stride, 0)
                    blk["bd"] = BatchNormAct(s, c_mid * 4)
                self.blocks.append(blk)
                c_in = c_mid * 4
        self.fc = Linear(s, c_in, num_classes)
        self.num_classes = num_classes
        self._finish(4)

    def init(self, seed=0):
        g = torch.Generator(device=self.device).manual_seed(seed)
        s = self.store
        for i, shape in enumerate(s.shapes):
            w = s.w32(i)
            if len(shape) == 4:    # Kaiming-normal, fan_in, relu (nectarml/nn/init.py:272-317)
                fan_in = shape[1] * shape[2] * shape[3]
                w.copy_(torch.randn(shape, device=self.device, generator=g) * (2.0 / fan_in) ** 0.5)
            elif len(shape) == 2:
                w.copy_(torch.randn(shape, device=self.device, generator=g) * (1.0 / shape[1]) ** 0.5)
        for blk in [{"b": self.stem_bn}] + self.blocks:
            for k, l in blk.items():
                if isinstance(l, BatchNormAct):
                    l.gamma.fill_(1.0)
        s.sync_half()

    def forward(self, x):
        """x: [N, H, W, 3] fp16 NHWC -> logits [N, classes] fp16."""
        t = self.token
        x = self.stem_bn(self.stem(x, t), t, ACT_RELU)
        x = self.store.record(max_pool(x, 3, 2, 1))
        for blk in self.blocks:
            idn = x
            y = blk["b1"](blk["c1"](x, t), t, ACT_RELU)
            y = blk["b2"](blk["c2"](y, t), t, ACT_RELU)
            if "cd" in blk:
                idn = blk["bd"](blk["cd"](x, t), t, ACT_NONE)
            x = blk["b3"](blk["c3"](y, t), t, ACT_RELU, residual=idn)
        pooled = x.float().mean(dim=(1, 2)).half()
        return self.fc(pooled, t)


class Pix2PixGenerator(_Net):
    """U-Net generator: 8 x (Conv2d 4x4 s2 p1) down to 1x1, 8 x (ConvTranspose2d 4x4 s2 p1) up with the encoder
    activations concatenated in (examples/pix2pix/generator.py:54-170); BatchNorm + LeakyReLU(0.2) down, BatchNorm +
    ReLU up, tanh on the 3-channel output."""

    split_backward = True

    def __init__(self, device, in_channels=3, features=64):
        super().__init__(device)
        s, f = self.store, features
        down = [f, f * 2, f * 4, f * 8, f * 8, f * 8, f * 8, f * 8]
        self.down, c = [], in_channels
        for i, co in enumerate(down):
            first, last = i == 0, i == len(down) - 1
            conv = Conv(s, c, co, 4, 2, 1, bias=first or last, needs_dx=not first)
            bn = None if (first or last) else BatchNormAct(s, co)
            self.down.append((conv, bn))
            c = co
        up = [f * 8, f * 8, f * 8, f * 8, f * 4, f * 2, f]
        self.up = []
        for i, co in enumerate(up):
            ci = c if i == 0 else c * 2
            self.up.append((Conv(s, ci, co, 4, 2, 1, transposed=True), BatchNormAct(s, co)))
            c = co
        self.final = Conv(s, c * 2, in_channels, 4, 2, 1, bias=True, transposed=True)
        self._finish(3)

    def init(self, seed=0):
        g = torch.Generator(device=self.device).manual_seed(seed)
        s = self.store
        for i, shape in enumerate(s.shapes):
            if len(shape) == 4:
                s.w32(i).copy_(torch.randn(shape, device=self.device, generator=g) * 0.02)
        for _, bn in self.down + self.up:
            if bn is not None:
                bn.gamma.fill_(1.0)
        s.sync_half()

    def forward(self, x):
        """x: [N, H, W, 3] fp16 NHWC in [-1, 1] -> generated image, same shape."""
        t = self.token
        skips = []
        for i, (conv, bn) in enumerate(self.down):
            y = conv(x, t)
            if bn is not None:
                x = bn(y, t, ACT_LEAKY)
            elif i == 0:
                x = self.store.record(torch.nn.functional.leaky_relu(y, 0.2))
            else:
                x = self.store.record(torch.relu(y))       # bottleneck
            skips.append(x)
        skips.pop()
        # The frontier between decoder and encoder in the backward pass: the bottleneck's output as the decoder
        # reads it and the encoder activations as the concatenations read them (views, so that each is its own
        # autograd node).  A split backward (TrainStep.capture_split) stops here, sends the decoder's gradients
        # off, and then continues into the encoder.
        x = x.view_as(x)
        skips = [d.view_as(d) for d in skips]
        self.frontier = [x] + list(skips)   # (dropped again by whoever ran the backward pass: see TrainStep)
        self.frontier_first_param = self.up[0][0].first   # decoder (and final layer) parameters start here
        for i, (conv, bn) in enumerate(self.up):
            if i > 0:
                x = torch.cat((x, skips.pop()), dim=3)
            x = bn(conv(x, t), t, ACT_RELU)
        x = torch.cat((x, skips.pop()), dim=3)
        return self.store.record(torch.tanh(self.final(x, t)))


# ------------------------------------------------------------------ steps --
class TrainStep:
    """One optimisation step = micro-batches of forward + backward (gradients accumulate in the flat buffer),
    the bucketed all-reduce of the last micro-batch's backward, the finiteness check and the SGD-momentum update."""

    def __init__(self, net: _Net, loss: str, lr=0.1, momentum=0.9, weight_decay=1e-4, loss_scale=16384.0):
        self.net, self.loss_kind = net, loss
        self.lr, self.momentum, self.wd, self.loss_scale = lr, momentum, weight_decay, loss_scale

    def _loss(self, out, target, denom):
        if self.loss_kind == "cross_entropy":
            return torch.nn.functional.cross_entropy(out.float(), target, reduction="sum") / denom
        return (out.float() - target.float()).abs().sum() / denom     # L1 against the target image

    def micro_batch(self, x, target, global_count, first: bool, last: bool) -> torch.Tensor:
        """Forward + backward of one micro-batch; gradients replace (first) or add to the flat buffer."""
        store = self.net.store
        store.accumulate = not first
        store.begin_backward(last_micro_batch=last)
        out = self.net.forward(x)
        loss = self._loss(out, target, global_count)
        (loss * self.loss_scale).backward()
        store.accumulate = False
        self.net.frontier = None
        return loss.detach()

    def capture(self, x, target, global_count: int, accumulate_variants=(False,)):
        """Captures forward + backward of one micro-batch on STATIC input tensors into CUDA graphs (one per
        requested accumulate mode), after a warm-up on a side stream.  The ~500 kernel launches of a micro-batch
        then cost one graph launch; the gradient exchange and the optimizer update stay outside the graphs.
        Returns {accumulate: (graph, static loss tensor)}."""
        store = self.net.store
        saved = store.communicate
        store.communicate = False
        side = torch.cuda.Stream(device=self.net.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.micro_batch(x, target, global_count, first=True, last=False)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graphs = {}
        for acc in accumulate_variants:
            g = torch.cuda.CUDAGraph()
            with capture_into(g):
                loss = self.micro_batch(x, target, global_count, first=not acc, last=False)
            graphs[acc] = (g, loss)
        store.communicate = saved
        return graphs

    def capture_split(self, x, target, global_count: int):
        """For nets that expose a `frontier` (the U-Net: decoder | encoder): captures forward + the decoder's
        backward into one CUDA graph and the encoder's backward into a second one, so that the all-reduce of the
        decoder's gradients (two thirds of the parameters) runs while the encoder's backward does.  The second
        graph is planned under the SM reserve that leaves room for NCCL.  Returns (graph_a, graph_b, loss)."""
        store, net = self.net.store, self.net
        if not net.split_backward:
            raise ValueError("capture_split needs a net whose forward() marks a frontier (split_backward)")
        saved = store.communicate
        store.communicate = False

        def part_a():
            store.accumulate = False
            store.begin_backward(last_micro_batch=False)
            out = net.forward(x)
            loss = self._loss(out, target, global_count)
            grads = torch.autograd.grad(loss * self.loss_scale, net.frontier)
            return loss.detach(), grads

        def part_b(grads):
            torch.autograd.backward(net.frontier, grads)
            net.frontier = None

        side = torch.cuda.Stream(device=net.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                _, g = part_a()
                part_b(g)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        ga, gb = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with capture_into(ga):
            loss, grads = part_a()
        if store.world > 1 and store.sm_reserve and store.sms:
            ops.set_sm_limit(store.sms - store.sm_reserve)
        try:
            with capture_into(gb, pool=ga.pool()):
                part_b(grads)
        finally:
            ops.set_sm_limit(0)
        store.communicate = saved
        return ga, gb, loss

    def replay_split(self, graphs) -> None:
        """Replays a split capture with the decoder's gradient exchange overlapping the encoder's backward."""
        ga, gb, _ = graphs
        store, cut = self.net.store, self.net.frontier_first_param
        ga.replay()
        if store.world > 1:
            store.pending.append(dist.all_reduce(store.grad[cut:], async_op=True))
        gb.replay()
        if store.world > 1:
            store.pending.append(dist.all_reduce(store.grad[:cut], async_op=True))
            store.wait_exchange()

    def exchange_all(self) -> None:
        """All-reduces every bucket of the flat gradient (used after a graph-captured backward)."""
        store = self.net.store
        if store.world > 1:
            for b in range(len(store.bucket_bounds) - 1):
                lo, hi = store.bucket_bounds[b], store.bucket_bounds[b + 1]
                store.pending.append(dist.all_reduce(store.grad[lo:hi], async_op=True))
            store.wait_exchange()

    def optimizer_step(self) -> None:
        self.net.store.sgd_step(self.lr, self.momentum, self.wd, 1.0 / self.loss_scale)

    def __call__(self, micro_batches, global_count: int, optimize: bool = True) -> torch.Tensor:
        """micro_batches: list of (input NHWC fp16, target); global_count: samples (cross-entropy) or elements (L1)
        of the GLOBAL batch, the divisor of the summed loss.  Returns this rank's share of the mean loss."""
        store = self.net.store
        total = torch.zeros((), device=self.net.device)
        for i, (x, target) in enumerate(micro_batches):
            store.accumulate = i > 0
            store.begin_backward(last_micro_batch=(i == len(micro_batches) - 1))
            out = self.net.forward(x)
            loss = self._loss(out, target, global_count)
            (loss * self.loss_scale).backward()
            total += loss.detach()
        store.accumulate = False
        store.wait_exchange()
        if optimize:
            store.sgd_step(self.lr, self.momentum, self.wd, 1.0 / self.loss_scale)
        return total
