"""PyTorch autograd front end of the engine: ``QConv2dFunction`` / ``QDenseFunction`` and two small modules.

The reference is driven from a framework plugin (its TensorFlow ops call ``upstride::conv2DFwd`` / ``conv2DBwd`` /
``denseFwd`` / ``denseBwd`` of ``src/upstride.hpp:18-86`` from the op's compute callback). This module is the same
thing for PyTorch: each function's ``forward`` calls the forward entry point, its ``backward`` the backward entry
point, on the caller's tensors and the current CUDA stream. Tensors use the engine's layouts: activations
``[D*N, C, H, W]`` (or ``[D*N, H, W, C]``) with the multivector components stacked on the batch axis, filters
``[D, Co, Ci, kh, kw]`` (OIHW) and friends, dense filters ``[D, I, O]`` / ``[D, O, I]``, bias ``[D, C]``.

The engine's backward pass has no bias gradient (the framework side owns the bias in the reference too): it is the
sum of the output gradient over batch and pixels per component and channel, computed here with one torch reduction.
"""
import torch

from . import _lib
from .descriptors import (Algebra, Conv2DBwdDescriptor, Conv2DFwdDescriptor, DataFormat, DenseBwdDescriptor, DenseFwdDescriptor,
                          FilterLayout, MULTIVECTOR_DIM, Padding)
from .ops import conv2DBwd, conv2DFwd, denseBwd, denseFwd


class QConv2dFunction(torch.autograd.Function):
    """``y = QConv2dFunction.apply(x, w, bias, stride, dilation, padding, explicit_pad, groups, algebra, data_format,
    filter_layout, real_valued_input, context)``.

    padding: a ``Padding`` value; ``explicit_pad`` = (top, left, bottom, right) when it is ``Padding.EXPLICIT``.
    ``real_valued_input``: x is a real ``[N, C, H, W]`` tensor entering a hyper-complex layer (no input gradient
    exists then, reference ``src/conv2d.hpp:384-396``)."""

    @staticmethod
    def forward(ctx, x, w, bias, stride=1, dilation=1, padding=Padding.VALID, explicit_pad=(), groups=1,
                algebra=Algebra.QUATERNION, data_format=DataFormat.NCHW, filter_layout=FilterLayout.OIHW,
                real_valued_input=False, context=None):
        x, w = x.contiguous(), w.contiguous()
        args = (tuple(x.shape), tuple(w.shape), stride, dilation, padding, tuple(explicit_pad), groups, algebra, data_format, filter_layout)
        fwd = Conv2DFwdDescriptor(*args, bias is not None, real_valued_input)
        y = torch.empty(fwd.getOutputShape(), dtype=x.dtype, device=x.device)
        conv2DFwd(x, w, None if bias is None else bias.contiguous(), y, fwd, context)
        ctx.save_for_backward(x, w)
        ctx.args, ctx.real, ctx.context, ctx.has_bias = args, real_valued_input, context, bias is not None
        ctx.channel_axis = 1 if data_format == DataFormat.NCHW else 3
        ctx.dim = MULTIVECTOR_DIM[algebra]
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        need_dx = ctx.needs_input_grad[0] and not ctx.real
        bwd = Conv2DBwdDescriptor(*ctx.args, need_dx, ctx.real)
        dw = torch.empty_like(w)
        dx = torch.empty_like(x) if need_dx else None
        conv2DBwd(x, w, dy, dw, dx, bwd, ctx.context)
        db = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            g = dy.view(ctx.dim, -1, *dy.shape[1:])
            axes = [a for a in range(g.dim()) if a not in (0, ctx.channel_axis + 1)]
            db = g.float().sum(dim=axes).to(dy.dtype)
        return (dx, dw, db) + (None,) * 10


class QDenseFunction(torch.autograd.Function):
    """``y = QDenseFunction.apply(x, w, bias, algebra, filter_layout, context)`` with x ``[D*B, I]`` and w ``[D, I, O]``
    (``FilterLayout.IO``) or ``[D, O, I]`` (``FilterLayout.OI``). The engine always emits the filter gradient as
    ``[D, I, O]`` (reference ``src/backend/cudnn/dense.hpp:187-195``); it is transposed back here for OI filters so
    that the gradient has the shape of the parameter."""

    @staticmethod
    def forward(ctx, x, w, bias, algebra=Algebra.QUATERNION, filter_layout=FilterLayout.IO, context=None):
        x, w = x.contiguous(), w.contiguous()
        fwd = DenseFwdDescriptor(tuple(x.shape), tuple(w.shape), algebra, filter_layout, bias is not None)
        y = torch.empty(fwd.getOutputShape(), dtype=x.dtype, device=x.device)
        denseFwd(x, w, None if bias is None else bias.contiguous(), y, fwd, context)
        ctx.save_for_backward(x, w)
        ctx.algebra, ctx.layout, ctx.context, ctx.has_bias = algebra, filter_layout, context, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        need_dx = ctx.needs_input_grad[0]
        bwd = DenseBwdDescriptor(tuple(x.shape), tuple(w.shape), ctx.algebra, ctx.layout, need_dx)
        i, o = bwd.getInputChannels(), bwd.getOutputChannels()
        dw_io = torch.empty(w.shape[:-2] + (i, o), dtype=w.dtype, device=w.device)
        dx = torch.empty_like(x) if need_dx else None
        denseBwd(x, w, dy, dw_io, dx, bwd, ctx.context)
        dw = dw_io if ctx.layout == FilterLayout.IO else dw_io.transpose(-1, -2).contiguous()
        db = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            dim = MULTIVECTOR_DIM[ctx.algebra]
            db = dy.view(dim, -1, dy.shape[1]).float().sum(1).to(dy.dtype)
        return dx, dw, db, None, None, None


class QConv2d(torch.nn.Module):
    """Quaternion (or other algebra) convolution layer with He-normal filters over the D*Ci*kh*kw real inputs."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=Padding.SAME, dilation=1, groups=1, bias=True,
                 algebra=Algebra.QUATERNION, dtype=torch.float16, device="cuda", context=None):
        super().__init__()
        d = MULTIVECTOR_DIM[algebra]
        kh, kw = (kernel_size, kernel_size) if isinstance(kernel_size, int) else kernel_size
        std = (2.0 / (d * (in_channels // groups) * kh * kw)) ** 0.5
        self.weight = torch.nn.Parameter(torch.randn((d, out_channels, in_channels // groups, kh, kw), device=device) .mul_(std).to(dtype))
        self.bias = torch.nn.Parameter(torch.zeros((d, out_channels), dtype=dtype, device=device)) if bias else None
        self.stride, self.padding, self.dilation, self.groups, self.algebra, self.context = stride, padding, dilation, groups, algebra, context

    def forward(self, x):
        return QConv2dFunction.apply(x, self.weight, self.bias, self.stride, self.dilation, self.padding, (), self.groups, self.algebra,
                                     DataFormat.NCHW, FilterLayout.OIHW, False, self.context)


class QDense(torch.nn.Module):
    def __init__(self, in_features, out_features, bias=True, algebra=Algebra.QUATERNION, dtype=torch.float16, device="cuda", context=None):
        super().__init__()
        d = MULTIVECTOR_DIM[algebra]
        self.weight = torch.nn.Parameter(torch.randn((d, in_features, out_features), device=device).mul_((2.0 / (d * in_features)) ** 0.5).to(dtype))
        self.bias = torch.nn.Parameter(torch.zeros((d, out_features), dtype=dtype, device=device)) if bias else None
        self.algebra, self.context = algebra, context

    def forward(self, x):
        return QDenseFunction.apply(x, self.weight, self.bias, self.algebra, FilterLayout.IO, self.context)


__all__ = ["QConv2dFunction", "QDenseFunction", "QConv2d", "QDense"]
