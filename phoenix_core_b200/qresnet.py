"""Quaternion ResNet-18 training step on the quaternion operators of this package, data-parallel with NCCL.

    python -m phoenix_core_b200.qresnet [--batch 128] [--steps 10] [--warmup 3]          (torchrun for N > 1)

Standard ResNet-18 topology with every real channel count divided by 4 (quaternion channels 16/32/64/128,
1000 classes = 250 quaternion outputs), every convolution and the classifier replaced by their quaternion
versions (`conv2DFwd/Bwd`, `denseFwd/Bwd` of this package). The UpStride engine itself contains no model code:
batch-norm, ReLU, pooling, loss and optimiser are plain torch ops and are harness glue, not part of the
drop-in path. Batch-norm normalises each quaternion channel with one mean / variance shared by its four
components (statistics over the stacked `[4N, C, H, W]` tensor); it runs on helper kernels of the library
(`pcb_aux_bn_*`: plain, with the residual add of a block's tail, and with the stem's max-pool fused in), because the
framework's own batch-norm kernels idle the GPU at 16 channels. On one GPU the whole step is captured once and
replayed as a CUDA graph (`QResNet18.capture` / `step`).

Precision: fp16 activations and filters (the reference's fp16 tensors; every kernel accumulates in fp32),
fp32 master weights, static loss scale. All filter gradients are written by the kernels straight into ONE
flat fp16 bucket, which is all-reduced in two parts (the tail beside the rest of the backward pass); the batch-norm
parameters and their gradients live in a second small flat fp32 buffer that the batch-norm kernels write.
"""
import argparse
import json
import math
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import phoenix_core_b200 as pcb  # noqa: E402
from phoenix_core_b200 import _lib  # noqa: E402
from phoenix_core_b200.ops import _raw_stream  # noqa: E402
from phoenix_core_b200.context import Context  # noqa: E402

LOSS_SCALE = 256.0
_DT = {torch.float16: _lib.PCB_F16, torch.bfloat16: _lib.PCB_BF16}


def reduce_and_apply(flat_w32, flat_mom, flat_grad, world, lr, momentum, loss_scale, split=0, pending=None):
    """The data-parallel exchange step and the SGD update on the flat buffers: sum the gradient bucket over
    the ranks, undo the loss scale, average over the ranks, momentum SGD on the fp32 masters. The bucket is reduced in two
    parts: elements from `split` on (the deep layers, whose gradients exist first) by an all-reduce that the backward pass
    started on a side stream (`pending`, its work handle) and that ran beside the rest of that pass; the head here."""
    if world > 1:
        if pending is not None:
            dist.all_reduce(flat_grad[:split])
            pending.wait()                      # the current stream waits for the side stream's all-reduce
        else:
            dist.all_reduce(flat_grad)
    inv = 1.0 / (loss_scale * world)
    flat_mom.mul_(momentum).add_(flat_grad.float(), alpha=inv)
    flat_w32.add_(flat_mom, alpha=-lr)


class _BNReLUFn(torch.autograd.Function):
    """Batch-norm over the stacked [4N, C, H, W] tensor (one mean / variance per quaternion channel, shared by its
    four components) with an optional fused ReLU. Harness glue, not part of the drop-in path: torch's own batch-norm
    kernels (native and cuDNN alike) launch one block per channel, which at 16 channels and a stacked batch of 512
    leaves the GPU idle, so 16-bit CUDA tensors go to the helper kernels of the library (statistics + apply:
    three passes over the data forward, five to seven backward); anything else takes plain torch reductions."""

    @staticmethod
    def forward(ctx, x, gamma, beta, eps, relu, grad_out=None):
        """`grad_out` = (dgamma, dbeta) buffers of the caller: the backward kernels write the parameter gradients there and
        autograd is given none for them (the model keeps all batch-norm parameters and gradients in flat buffers)."""
        ctx.relu = relu
        ctx.grad_out = grad_out
        if x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and x.is_contiguous():
            planes, c = x.shape[0], x.shape[1]
            hw = x.numel() // (planes * c)
            y = torch.empty_like(x)
            mean = torch.empty(c, dtype=torch.float32, device=x.device)
            invstd = torch.empty_like(mean)
            scratch = torch.empty(5 * c, dtype=torch.float32, device=x.device)
            _lib.check(_lib.lib().pcb_aux_bn_relu_fwd(_DT[x.dtype], x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(),
                                                      mean.data_ptr(), invstd.data_ptr(), scratch.data_ptr(), planes, c, hw, eps, int(relu),
                                                      _raw_stream()))
            ctx.fused = True
            # the backward kernels recompute the ReLU mask from x, so the output is not kept for them
            ctx.save_for_backward(x, None, mean, invstd, gamma, beta)
            return y
        var, mean = torch.var_mean(x.float(), dim=(0, 2, 3), unbiased=False)
        invstd = torch.rsqrt(var + eps)
        scale = (gamma * invstd)
        shift = beta - mean * scale
        y = torch.addcmul(shift.to(x.dtype).view(1, -1, 1, 1), x, scale.to(x.dtype).view(1, -1, 1, 1))
        if relu:
            y.clamp_min_(0)
        ctx.fused = False
        ctx.save_for_backward(x, y if relu else None, mean, invstd, gamma, beta)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, y, mean, invstd, gamma, beta = ctx.saved_tensors
        if ctx.fused:
            dy = dy.contiguous()
            planes, c = x.shape[0], x.shape[1]
            hw = x.numel() // (planes * c)
            dx = torch.empty_like(x)
            if ctx.grad_out is not None:
                dgamma, dbeta = ctx.grad_out
            else:
                dgamma = torch.empty(c, dtype=torch.float32, device=x.device)
                dbeta = torch.empty_like(dgamma)
            scratch = torch.empty(5 * c, dtype=torch.float32, device=x.device)
            if ctx.relu:
                _lib.check(_lib.lib().pcb_aux_bn_relu_bwd_from_input(_DT[x.dtype], x.data_ptr(), dy.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                                                     mean.data_ptr(), invstd.data_ptr(), dx.data_ptr(), dgamma.data_ptr(),
                                                                     dbeta.data_ptr(), scratch.data_ptr(), planes, c, hw,
                                                                     _raw_stream()))
                return (dx, None, None, None, None, None) if ctx.grad_out is not None else (dx, dgamma, dbeta, None, None, None)
            _lib.check(_lib.lib().pcb_aux_bn_relu_bwd(_DT[x.dtype], x.data_ptr(), y.data_ptr() if ctx.relu else None, dy.data_ptr(),
                                                      gamma.data_ptr(), mean.data_ptr(), invstd.data_ptr(), dx.data_ptr(), dgamma.data_ptr(),
                                                      dbeta.data_ptr(), scratch.data_ptr(), planes, c, hw, int(ctx.relu),
                                                      _raw_stream()))
            return (dx, None, None, None, None, None) if ctx.grad_out is not None else (dx, dgamma, dbeta, None, None, None)
        g = dy * (y > 0) if ctx.relu else dy
        m = x.numel() // x.shape[1]
        sum_g = g.sum(dim=(0, 2, 3), dtype=torch.float32)
        sum_gx = (g * x).sum(dim=(0, 2, 3), dtype=torch.float32)
        # xhat = (x - mean) * invstd;  dgamma = sum(g * xhat);  dbeta = sum(g)
        dgamma = (sum_gx - mean * sum_g) * invstd
        dbeta = sum_g
        # dx = gamma*invstd * (g - dbeta/m - xhat * dgamma/m)  =  a*g + b*x + c   per channel
        a = gamma * invstd
        b = -a * invstd * dgamma / m
        c = -a * dbeta / m - b * mean
        dx = g * a.to(g.dtype).view(1, -1, 1, 1)
        dx.addcmul_(x, b.to(g.dtype).view(1, -1, 1, 1))
        dx.add_(c.to(g.dtype).view(1, -1, 1, 1))
        if ctx.grad_out is not None:
            ctx.grad_out[0].copy_(dgamma)
            ctx.grad_out[1].copy_(dbeta)
            return dx, None, None, None, None, None
        return dx, dgamma, dbeta, None, None, None


class _BNAddReLUFn(torch.autograd.Function):
    """y = relu(batch_norm(x) + residual), the tail of a residual block, in the passes of the batch-norm itself (the
    add and the ReLU as separate framework operations cost five more passes over the tensor forward and three backward).
    16-bit contiguous CUDA tensors only; the caller falls back to the separate operations otherwise."""

    @staticmethod
    def forward(ctx, x, residual, gamma, beta, eps, grad_out=None):
        ctx.grad_out = grad_out
        planes, c = x.shape[0], x.shape[1]
        hw = x.numel() // (planes * c)
        y = torch.empty_like(x)
        mean = torch.empty(c, dtype=torch.float32, device=x.device)
        invstd = torch.empty_like(mean)
        scratch = torch.empty(5 * c, dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().pcb_aux_bn_add_relu_fwd(_DT[x.dtype], x.data_ptr(), residual.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                                      y.data_ptr(), mean.data_ptr(), invstd.data_ptr(), scratch.data_ptr(), planes, c, hw, eps,
                                                      _raw_stream()))
        ctx.save_for_backward(x, y, mean, invstd, gamma)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, y, mean, invstd, gamma = ctx.saved_tensors
        dy = dy.contiguous()
        planes, c = x.shape[0], x.shape[1]
        hw = x.numel() // (planes * c)
        dx, dres = torch.empty_like(x), torch.empty_like(x)
        if ctx.grad_out is not None:
            dgamma, dbeta = ctx.grad_out
        else:
            dgamma = torch.empty(c, dtype=torch.float32, device=x.device)
            dbeta = torch.empty_like(dgamma)
        scratch = torch.empty(5 * c, dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().pcb_aux_bn_add_relu_bwd(_DT[x.dtype], x.data_ptr(), y.data_ptr(), dy.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                                                      invstd.data_ptr(), dx.data_ptr(), dres.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(),
                                                      scratch.data_ptr(), planes, c, hw, _raw_stream()))
        return (dx, dres, None, None, None, None) if ctx.grad_out is not None else (dx, dres, dgamma, dbeta, None, None)


class _BNReLUPoolFn(torch.autograd.Function):
    """max_pool_3x3_s2(relu(batch_norm(x))) without the full-size normalised tensor: statistics, then normalise + ReLU + pool
    in one kernel; backward gathers the pooled gradient inside the batch-norm gradient's two passes (five passes over the
    large tensor instead of thirteen). 16-bit contiguous CUDA tensors with lines of a multiple of 8 pixels."""

    @staticmethod
    def forward(ctx, x, gamma, beta, eps, grad_out=None):
        ctx.grad_out = grad_out
        planes, c, h, w = x.shape
        y = torch.empty((planes, c, h // 2, w // 2), dtype=x.dtype, device=x.device)
        arg = torch.empty(y.shape, dtype=torch.uint8, device=x.device)
        mean = torch.empty(c, dtype=torch.float32, device=x.device)
        invstd = torch.empty_like(mean)
        scratch = torch.empty(5 * c, dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().pcb_aux_bn_relu_maxpool_fwd(_DT[x.dtype], x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(), arg.data_ptr(),
                                                          mean.data_ptr(), invstd.data_ptr(), scratch.data_ptr(), planes, c, h, w, eps,
                                                          _raw_stream()))
        ctx.save_for_backward(x, arg, mean, invstd, gamma, beta)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, arg, mean, invstd, gamma, beta = ctx.saved_tensors
        dy = dy.contiguous()
        planes, c, h, w = x.shape
        dx = torch.empty_like(x)
        if ctx.grad_out is not None:
            dgamma, dbeta = ctx.grad_out
        else:
            dgamma = torch.empty(c, dtype=torch.float32, device=x.device)
            dbeta = torch.empty_like(dgamma)
        scratch = torch.empty(5 * c, dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().pcb_aux_bn_relu_maxpool_bwd(_DT[x.dtype], x.data_ptr(), dy.data_ptr(), arg.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                                          mean.data_ptr(), invstd.data_ptr(), dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(),
                                                          scratch.data_ptr(), planes, c, h, w, _raw_stream()))
        return (dx, None, None, None, None) if ctx.grad_out is not None else (dx, dgamma, dbeta, None, None)


class _MaxPoolFn(torch.autograd.Function):
    """3x3 stride-2 pad-1 max pooling on the library's helper kernels (the framework's backward kernel scatters with atomics and
    takes three times as long as the forward pass). Harness glue."""

    @staticmethod
    def forward(ctx, x):
        rows, h, w = x.shape[0] * x.shape[1], x.shape[2], x.shape[3]
        y = torch.empty((x.shape[0], x.shape[1], (h - 1) // 2 + 1, (w - 1) // 2 + 1), dtype=x.dtype, device=x.device)
        arg = torch.empty(y.shape, dtype=torch.uint8, device=x.device)
        _lib.check(_lib.lib().pcb_aux_maxpool3x3s2_fwd(_DT[x.dtype], x.data_ptr(), y.data_ptr(), arg.data_ptr(), rows, h, w,
                                                       _raw_stream()))
        ctx.save_for_backward(arg)
        ctx.shape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        (arg,) = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty(ctx.shape, dtype=dy.dtype, device=dy.device)
        _lib.check(_lib.lib().pcb_aux_maxpool3x3s2_bwd(_DT[dy.dtype], dy.data_ptr(), arg.data_ptr(), dx.data_ptr(), ctx.shape[0] * ctx.shape[1],
                                                       ctx.shape[2], ctx.shape[3], _raw_stream()))
        return dx


def max_pool_3x3_s2(x):
    if x.is_cuda and x.dtype in _DT and x.is_contiguous():
        return _MaxPoolFn.apply(x)
    return F.max_pool2d(x, 3, 2, 1)


class BNReLU:
    """Batch-norm (+ ReLU) layer. Standalone (`flat` = None) it owns its parameters as autograd leaves; inside the model
    its parameters and their gradients are slices of the model's flat fp32 buffers (`flat` = (weights, gradients, offset)),
    the backward kernels write the gradients straight into their slices, and autograd sees no parameter at all."""

    def __init__(self, c, device, relu, flat=None):
        self.relu = relu
        self.grad_out = None
        if flat is None:
            self.weight = torch.ones(c, dtype=torch.float32, device=device, requires_grad=True)
            self.bias = torch.zeros(c, dtype=torch.float32, device=device, requires_grad=True)
        else:
            w, g, off = flat
            self.weight, self.bias = w[off:off + c], w[off + c:off + 2 * c]
            self.weight.fill_(1.0)
            self.bias.zero_()
            self.grad_out = (g[off:off + c], g[off + c:off + 2 * c])

    def __call__(self, x, relu=None):
        return _BNReLUFn.apply(x, self.weight, self.bias, 1e-5, self.relu if relu is None else relu, self.grad_out)

    def relu_pool(self, x):
        """max_pool_3x3_s2(relu(batch_norm(x)))."""
        if x.is_cuda and x.dtype in _DT and x.is_contiguous() and x.shape[2] % 2 == 0 and x.shape[3] % 8 == 0:
            return _BNReLUPoolFn.apply(x, self.weight, self.bias, 1e-5, self.grad_out)
        return max_pool_3x3_s2(self(x, relu=True))

    def add_relu(self, x, residual):
        """relu(batch_norm(x) + residual)."""
        if x.is_cuda and x.dtype in _DT and x.is_contiguous() and residual.is_contiguous() and residual.shape == x.shape and residual.dtype == x.dtype:
            return _BNAddReLUFn.apply(x, residual, self.weight, self.bias, 1e-5, self.grad_out)
        return F.relu_(self(x, relu=False) + residual)


class _QConvFn(torch.autograd.Function):
    """y = conv(x, w); the filter gradient is written into `grad_view` (a slice of the flat bucket)."""

    @staticmethod
    def forward(ctx, x, w, layer):
        y = torch.empty(layer.fwd.getOutputShape(), dtype=x.dtype, device=x.device)
        pcb.conv2DFwd(x, w, None, y, layer.fwd, layer.context, keep=layer.kept)
        ctx.layer = layer
        ctx.save_for_backward(x, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        layer = ctx.layer
        if layer.before_backward is not None:
            layer.before_backward()
        dy = dy.contiguous()
        need_dx = ctx.needs_input_grad[0]
        dx = torch.empty_like(x) if need_dx else None
        pcb.conv2DBwd(x, w, dy, layer.grad_view, dx, layer.bwd_dx if need_dx else layer.bwd_nodx, layer.context, kept=layer.kept)
        return dx, None, None


class QConv:
    """One quaternion convolution layer: descriptors built once per input shape, weights and their gradient are
    views into the model's flat buffers."""

    def __init__(self, model, ci, co, k, stride, real_input=False):
        self.ci, self.co, self.k, self.stride, self.real_input = ci, co, k, stride, real_input
        self.shape = (4, co, ci, k, k)
        self.offset = model.reserve(self.shape)
        self.model = model
        self.context = model.context
        self.fwd = None
        self.before_backward = None      # optional callable run when this layer's backward pass begins
        self.kept = pcb.KeptInput() if model.keep_staged_inputs else None   # the forward call's staged x, read again by the filter gradient

    def bind(self):
        n = math.prod(self.shape)
        self.weight = self.model.flat_w16[self.offset:self.offset + n].view(self.shape)
        self.grad_view = self.model.flat_g16[self.offset:self.offset + n].view(self.shape)
        std = math.sqrt(2.0 / (4 * self.ci * self.k * self.k))          # He-normal over the 4*Ci*k*k real inputs
        self.model.flat_w32[self.offset:self.offset + n].normal_(0.0, std, generator=self.model.gen)

    def __call__(self, x):
        if self.fwd is None or self.fwd.getInputShape() != tuple(x.shape):
            args = (tuple(x.shape), self.shape, self.stride, 1, pcb.Padding.SAME, (), 1, pcb.Algebra.QUATERNION,
                    pcb.DataFormat.NCHW, pcb.FilterLayout.OIHW)
            self.fwd = pcb.Conv2DFwdDescriptor(*args, False, self.real_input)
            self.bwd_dx = None if self.real_input else pcb.Conv2DBwdDescriptor(*args, True)
            self.bwd_nodx = pcb.Conv2DBwdDescriptor(*args, False, self.real_input)
        w = self.weight.detach().requires_grad_(True)       # a leaf so that backward runs even for the image input
        return _QConvFn.apply(x, w, self)


class _QDenseFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, layer):
        y = torch.empty(layer.fwd.getOutputShape(), dtype=x.dtype, device=x.device)
        pcb.denseFwd(x, w, b, y, layer.fwd, layer.context)
        ctx.layer = layer
        ctx.save_for_backward(x, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        layer = ctx.layer
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        pcb.denseBwd(x, w, dy, layer.grad_view, dx, layer.bwd, layer.context)
        # the engine's dense backward has no bias gradient (the framework side owns it): sum over the batch per component
        layer.bias_grad_view.copy_(dy.view(4, -1, dy.shape[1]).sum(1))
        return dx, None, None, None


class QDense:
    def __init__(self, model, i, o):
        self.i, self.o = i, o
        self.shape = (4, i, o)
        self.offset = model.reserve(self.shape)
        self.bias_offset = model.reserve((4, o))
        self.model, self.context, self.fwd = model, model.context, None

    def bind(self):
        n = math.prod(self.shape)
        m = self.model
        self.weight = m.flat_w16[self.offset:self.offset + n].view(self.shape)
        self.grad_view = m.flat_g16[self.offset:self.offset + n].view(self.shape)
        self.bias = m.flat_w16[self.bias_offset:self.bias_offset + 4 * self.o].view(4, self.o)
        self.bias_grad_view = m.flat_g16[self.bias_offset:self.bias_offset + 4 * self.o].view(4, self.o)
        m.flat_w32[self.offset:self.offset + n].normal_(0.0, math.sqrt(2.0 / (4 * self.i)), generator=m.gen)
        m.flat_w32[self.bias_offset:self.bias_offset + 4 * self.o].zero_()

    def __call__(self, x):
        if self.fwd is None or self.fwd.getInputShape() != tuple(x.shape):
            self.fwd = pcb.DenseFwdDescriptor(tuple(x.shape), self.shape, pcb.Algebra.QUATERNION, pcb.FilterLayout.IO, True)
            self.bwd = pcb.DenseBwdDescriptor(tuple(x.shape), self.shape, pcb.Algebra.QUATERNION, pcb.FilterLayout.IO, True)
        w = self.weight.detach().requires_grad_(True)
        return _QDenseFn.apply(x, w, self.bias, self)


class QResNet18:
    """Quaternion ResNet-18 (quaternion channels 16 / 32 / 64 / 128, 250 quaternion classes)."""

    def __init__(self, device, seed=0, num_classes=1000, keep_staged_inputs=True):
        self.device = device
        self.keep_staged_inputs = keep_staged_inputs
        self.context = Context({"UPSTRIDE_MEMORY_OPTIMIZED": "1", "UPSTRIDE_CONV_FP16_POLICY": "backward32"})
        self.gen = torch.Generator(device=device).manual_seed(seed)
        self._numel = 0
        self.convs, self.bns = [], []
        # batch-norm parameters, their gradients and momenta: flat fp32 buffers (gamma and beta of a layer side by side)
        self._bn_numel = 0
        self.bn_w = torch.empty(8192, dtype=torch.float32, device=device)
        self.bn_g = torch.zeros(8192, dtype=torch.float32, device=device)
        # the stem takes the RGB image as a real-valued (type-0) input: only the real component exists, which is the
        # engine's own way of entering the quaternion domain (reference src/conv2d.hpp:122-164) and a quarter of the work
        self.conv1 = self._conv(3, 16, 7, 2, real_input=True)
        self.bn1 = self._bn(16)
        self.stages = []
        cin = 16
        for si, cout in enumerate((16, 32, 64, 128)):
            blocks = []
            for bi in range(2):
                stride = 2 if (si > 0 and bi == 0) else 1
                blk = {"c1": self._conv(cin, cout, 3, stride), "b1": self._bn(cout), "c2": self._conv(cout, cout, 3, 1),
                       "b2": self._bn(cout), "ds": None}
                if stride != 1 or cin != cout:
                    blk["ds"] = (self._conv(cin, cout, 1, stride), self._bn(cout))
                blocks.append(blk)
                cin = cout
            self.stages.append(blocks)
        self.fc = QDense(self, 128, num_classes // 4)
        # flat parameter / gradient storage: fp32 masters, fp16 working copy, fp16 gradient bucket
        self.flat_w32 = torch.zeros(self._numel, dtype=torch.float32, device=device)
        self.flat_w16 = torch.zeros(self._numel, dtype=torch.float16, device=device)
        self.flat_g16 = torch.zeros(self._numel, dtype=torch.float16, device=device)
        self.flat_mom = torch.zeros(self._numel, dtype=torch.float32, device=device)
        for c in self.convs:
            c.bind()
        self.fc.bind()
        self.bn_w, self.bn_g = self.bn_w[:self._bn_numel], self.bn_g[:self._bn_numel]
        self.bn_m = torch.zeros_like(self.bn_w)
        # Data-parallel exchange in two parts. The flat bucket is laid out in forward order, so the last stage and the
        # classifier (72 % of the parameters) are its tail, and their gradients are complete when the backward pass
        # reaches the last convolution of stage 3: that layer's backward hook starts the tail's all-reduce on a side
        # stream, where it overlaps the backward pass of stages 3 .. 1; the head is reduced at the end of the pass.
        self.split = self.stages[3][0]["c1"].offset
        self.world = 1
        self.comm_stream = None
        self.pending = None
        self.stages[2][1]["c2"].before_backward = self._start_tail_reduce

    def _start_tail_reduce(self):
        if self.world > 1:
            if self.comm_stream is None:
                self.comm_stream = torch.cuda.Stream(priority=-1)
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                self.pending = dist.all_reduce(self.flat_g16[self.split:], async_op=True)

    def reserve(self, shape):
        off = self._numel
        self._numel += (math.prod(shape) + 7) // 8 * 8        # 16-byte aligned slices
        return off

    def _conv(self, ci, co, k, stride, real_input=False):
        c = QConv(self, ci, co, k, stride, real_input)
        self.convs.append(c)
        return c

    def _bn(self, c, relu=True):
        bn = BNReLU(c, self.device, relu, flat=(self.bn_w, self.bn_g, self._bn_numel))
        self._bn_numel += 2 * c
        self.bns.append(bn)
        return bn

    def num_parameters(self):
        return sum(math.prod(c.shape) for c in self.convs) + math.prod(self.fc.shape) + 4 * self.fc.o

    def forward(self, images):
        """images: [N, 3, H, W] real RGB (the quaternion with zero imaginary parts) -> logits [N, classes]."""
        n = images.shape[0]
        x = self.bn1.relu_pool(self.conv1(images.contiguous()))
        for blocks in self.stages:
            for blk in blocks:
                idt = x
                out = blk["b1"](blk["c1"](x))
                if blk["ds"] is not None:
                    idt = blk["ds"][1](blk["ds"][0](x), relu=False)
                x = blk["b2"].add_relu(blk["c2"](out), idt)
        x = x.mean(dim=(2, 3))                                   # [4N, 128]
        y = self.fc(x.contiguous())                              # [4N, 250]
        return y.view(4, n, -1).permute(1, 0, 2).reshape(n, -1)  # class index = component * 250 + unit

    def capture(self, images, labels, lr=0.1, momentum=0.9):
        """Captures one single-GPU training step (forward, loss, backward, update) as a CUDA graph over static copies of
        the batch; `step` then replays it. The step is ~400 launches behind ~4.7 ms of Python per step against ~6.5 ms
        of kernels, so an eager loop turns host-bound as soon as the host is slower than usual; the replay is one launch.
        Returns False (and stays eager) if the capture fails."""
        self.graph = None
        try:
            # the caller has run a few eager steps (workspaces grown, kernels loaded); every parameter gradient is written by
            # the kernels into flat buffers, so autograd holds no accumulation node tied to another stream
            self.static_images, self.static_labels = images.clone(), labels.clone()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.static_loss = self.train_step(self.static_images, self.static_labels, 1, lr, momentum)
            self.graph = graph
        except Exception as err:                                # noqa: BLE001 -- any capture problem: run eagerly
            sys.stderr.write("qresnet: CUDA graph capture failed (%s); running eagerly\n" % (err,))
            self.graph = None
            torch.cuda.synchronize()
        return self.graph is not None

    def step(self, images, labels, world=1, lr=0.1, momentum=0.9):
        """One training step: the captured graph if there is one (single GPU), the eager step otherwise."""
        if world == 1 and getattr(self, "graph", None) is not None:
            if images.data_ptr() != self.static_images.data_ptr():
                self.static_images.copy_(images, non_blocking=True)
                self.static_labels.copy_(labels, non_blocking=True)
            self.graph.replay()
            return self.static_loss
        return self.train_step(images, labels, world, lr, momentum)

    def train_step(self, images, labels, world=1, lr=0.1, momentum=0.9):
        self.flat_w16.copy_(self.flat_w32)
        self.world, self.pending = world, None
        logits = self.forward(images)
        loss = F.cross_entropy(logits.float(), labels)
        (loss * LOSS_SCALE).backward()
        reduce_and_apply(self.flat_w32, self.flat_mom, self.flat_g16, world, lr, momentum, LOSS_SCALE, self.split, self.pending)
        self.pending = None
        # the batch-norm parameters: one flat gradient buffer (written by the backward kernels), one all-reduce, one update
        if world > 1:
            dist.all_reduce(self.bn_g)
        self.bn_m.mul_(momentum).add_(self.bn_g, alpha=1.0 / (LOSS_SCALE * world))
        self.bn_w.add_(self.bn_m, alpha=-lr)
        return loss


FWD_GFLOP_PER_IMAGE = 4.336      # quaternion conv + fc layers, 16-product count, 224x224

# The distinct convolution layers of the network: name, input channels, output channels, input size, kernel, stride,
# real-valued input, how many times the layer occurs.
LAYERS = [("conv1 7x7/2 (real input)", 3, 16, 224, 7, 2, True, 1), ("stage1 3x3 16", 16, 16, 56, 3, 1, False, 4),
          ("stage2 3x3/2 16-32", 16, 32, 56, 3, 2, False, 1), ("stage2 3x3 32", 32, 32, 28, 3, 1, False, 3),
          ("stage3 3x3/2 32-64", 32, 64, 28, 3, 2, False, 1), ("stage3 3x3 64", 64, 64, 14, 3, 1, False, 3),
          ("stage4 3x3/2 64-128", 64, 128, 14, 3, 2, False, 1), ("stage4 3x3 128", 128, 128, 7, 3, 1, False, 3),
          ("downsample 1x1/2 16-32", 16, 32, 56, 1, 2, False, 1), ("downsample 1x1/2 32-64", 32, 64, 28, 1, 2, False, 1),
          ("downsample 1x1/2 64-128", 64, 128, 14, 1, 2, False, 1)]


def layer_table(batch=128, reps=10, peak_tflops=None):
    """Times every distinct convolution layer of the network on its own (fp16, SAME padding, the three passes through the
    operator API, CUDA events, 3 warm-up + `reps` launches) and returns one row per layer: milliseconds, TFLOP/s
    (F = 32*N*Ho*Wo*Co*Ci*k*k, a quarter of it for the real-valued stem) and, if a peak is given, the fraction of it."""
    dev = torch.device("cuda", torch.cuda.current_device())
    ctx = Context({"UPSTRIDE_MEMORY_OPTIMIZED": "1", "UPSTRIDE_CONV_FP16_POLICY": "backward32"})

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    rows, per_step = [], 0.0
    for name, ci, co, h, k, s_, real, count in LAYERS:
        xshape = ((1 if real else 4) * batch, ci, h, h)
        args = (xshape, (4, co, ci, k, k), s_, 1, pcb.Padding.SAME, (), 1, pcb.Algebra.QUATERNION, pcb.DataFormat.NCHW, pcb.FilterLayout.OIHW)
        fwd = pcb.Conv2DFwdDescriptor(*args, False, real)
        bwd = pcb.Conv2DBwdDescriptor(*args, not real, real)
        x = torch.randn(xshape, device=dev, dtype=torch.float16)
        w = torch.randn((4, co, ci, k, k), device=dev, dtype=torch.float16) * 0.05
        y = torch.empty(fwd.getOutputShape(), device=dev, dtype=torch.float16)
        dy, dw = torch.randn_like(y), torch.empty_like(w)
        dx = None if real else torch.empty_like(x)
        t_f = timed(lambda: pcb.conv2DFwd(x, w, None, y, fwd, ctx))
        t_b = timed(lambda: pcb.conv2DBwd(x, w, dy, dw, dx, bwd, ctx))
        ho = y.shape[2]
        gflop = 32.0 * batch * ho * ho * co * ci * k * k * (0.25 if real else 1.0) / 1e9
        passes = 2 if real else 3
        row = {"layer": name, "count": count, "fwd_ms": round(t_f, 4), "bwd_ms": round(t_b, 4),
               "tflops": round(passes * gflop / (t_f + t_b), 1)}
        if peak_tflops:
            row["frac_of_peak"] = round(row["tflops"] / peak_tflops, 3)
        rows.append(row)
        per_step += count * (t_f + t_b)
    return {"batch": batch, "rows": rows, "conv_ms_per_step": round(per_step, 3)}


def run(batch, steps, warmup, image=224, quiet=False):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    own_pg = False
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=device)
        own_pg = True
    torch.backends.cudnn.enabled = False                         # nothing here may fall into cuDNN
    model = QResNet18(device, seed=0)
    if world > 1:                                                # identical replicas
        dist.broadcast(model.flat_w32, 0)
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    host_images = torch.randn((batch, 3, image, image), generator=g).to(torch.float16).pin_memory()
    host_labels = torch.randint(0, 1000, (batch,), generator=g).pin_memory()
    images, labels = host_images.to(device), host_labels.to(device)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(5, warmup)):                              # the first steps grow the device workspace
        loss = model.train_step(images, labels, world)
    sync()
    graphed = False
    if world == 1 and os.environ.get("PCB_QRESNET_GRAPH", "1") not in ("", "0"):
        graphed = model.capture(images, labels)
        for _ in range(2):
            loss = model.step(images, labels, world)
        sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = model.step(images, labels, world)
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    # end to end: host images -> device every step, loss read back
    sync()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = min(steps, 8)
    # the next batch is copied in on a side stream while this one trains; every step's loss goes back to pinned host memory
    copy_stream = torch.cuda.Stream()
    bufs = [(images, labels), (torch.empty_like(images), torch.empty_like(labels))]
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    used = [torch.cuda.Event(), torch.cuda.Event()]
    losses_host = torch.zeros(e2e_steps, dtype=torch.float32).pin_memory()

    def prefetch(i):
        with torch.cuda.stream(copy_stream):
            if i >= 2:
                copy_stream.wait_event(used[i & 1])
            bufs[i & 1][0].copy_(host_images, non_blocking=True)
            bufs[i & 1][1].copy_(host_labels, non_blocking=True)
            ready[i & 1].record(copy_stream)

    a.record()
    prefetch(0)
    for i in range(e2e_steps):
        torch.cuda.current_stream().wait_event(ready[i & 1])
        if i + 1 < e2e_steps:
            prefetch(i + 1)
        loss = model.step(bufs[i & 1][0], bufs[i & 1][1], world)
        used[i & 1].record()
        losses_host[i].copy_(loss.detach(), non_blocking=True)
    b.record()
    sync()
    loss_host = float(losses_host[-1])
    e2e_ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    result = None
    if rank == 0:
        ips = batch * world * steps / (ms * 1e-3)
        result = {"metric": "QResNet-18 train images/s", "value": ips, "unit": "images/s", "n_gpus": world, "steps": steps,
                  "ms_per_step": ms / steps, "batch_per_gpu": batch, "image": image, "dtype": "f16",
                  "tflops_conv": 3 * FWD_GFLOP_PER_IMAGE * (image / 224.0) ** 2 * ips / 1e3, "loss": loss_host,
                  "parameters": model.num_parameters(), "cuda_graph": graphed,
                  "e2e": {"value": batch * world * e2e_steps / (e2e_ms * 1e-3), "unit": "images/s",
                          "h2d_bytes_per_step": host_images.numel() * 2 + host_labels.numel() * 8, "d2h_bytes_per_step": 4},
                  "glue": "convolutions and dense: this package only; batch-norm (+ residual add) + ReLU and max-pool: helper kernels of the library; loss / SGD: torch ops (none of these is in the reference)"}
        if not quiet:
            print(json.dumps(result), flush=True)
    if own_pg:
        dist.barrier()
        dist.destroy_process_group()
    return result


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--image", type=int, default=224)
    a = ap.parse_args()
    run(a.batch, a.steps, a.warmup, a.image)


if __name__ == "__main__":
    main()
