"""The four entry points of the engine on torch CUDA tensors: ``conv2DFwd``, ``conv2DBwd``, ``denseFwd``,
``denseBwd`` (reference ``src/upstride.hpp:18-86``).

torch is used only to own device memory and streams; the arithmetic happens in the CUDA backend behind the
C ABI (``include/phoenix_core_b200.h``). Tensors are caller-owned and must be contiguous; work is enqueued
on the current torch stream and the calls return without synchronising, like the reference's GPU backend.
Only quaternion NCHW / OIHW (conv) and IO / OI (dense) problems are accepted; anything else raises (there
is no CPU fallback).
"""
import ctypes
import os
import threading

import torch

from . import _lib
from .context import Context
from .descriptors import MULTIVECTOR_DIM, Algebra, DataFormat, FilterLayout, _dims, _filter_dims

_DTYPES = {torch.float32: _lib.PCB_F32, torch.float16: _lib.PCB_F16, torch.bfloat16: _lib.PCB_BF16}


class Device:
    """Per-CUDA-device state: an access mutex and grow-only workspaces, as the reference's
    ``upstride::Device`` (``src/backend/device.hpp:12-110``: ``accessControl``, ``requestWorkspace``).

    The reference keeps one device object, and so one workspace, per CUDA stream
    (``src/backend/cudnn/cudnn.cc:5-14``). Here the workspace is keyed by the torch stream that is current at the
    call, for the same reason: it holds the split-K / staging scratch and the device status word, so operations
    issued on different streams must not share it. ``checkStatus`` reads the status word of the current stream's
    workspace back (it synchronises that stream); with ``PCB_CHECK_DEVICE_STATUS=1`` in the environment every
    operation does so before it returns."""
    _devices = {}
    _registry_lock = threading.Lock()

    def __init__(self, index):
        self.index = index
        self.accessControl = threading.Lock()
        self.workspaces = {}
        self.context = Context()
        self.check_after_each_op = os.environ.get("PCB_CHECK_DEVICE_STATUS", "0") not in ("", "0")

    @classmethod
    def get(cls, torch_device):
        idx = torch_device.index if torch_device.index is not None else torch.cuda.current_device()
        with cls._registry_lock:
            dev = cls._devices.get(idx)
            if dev is None:
                dev = cls._devices[idx] = Device(idx)
            return dev

    def requestWorkspace(self, nbytes):
        key = _raw_stream(self.index)
        ws = self.workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            with torch.cuda.device(self.index):
                ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=torch.device("cuda", self.index))
            self.workspaces[key] = ws      # allocated and used on this stream only, so torch's stream-ordered reuse holds
        return ws

    @property
    def workspace(self):
        return self.workspaces.get(_raw_stream(self.index))

    def checkStatus(self):
        """Raises BackendError(PCB_ERR_DEVICE_TIMEOUT) if a bounded device-side wait expired in the last operation
        issued on the current stream; synchronises that stream."""
        ws = self.workspace
        if ws is not None:
            with torch.cuda.device(self.index):
                _lib.check(_lib.lib().pcb_check_device_status(_ptr(ws), ws.numel(), _stream()))

    def _after_op(self):
        if self.check_after_each_op:
            self.checkStatus()

    def getContext(self):
        return self.context


class KeptInput:
    """Holds the workspace of one layer's forward call between that call and the layer's backward call, so that the
    filter gradient reads the staged copy of x the forward kernel made instead of staging x again (not in the
    reference). Pass one object per layer as ``keep=`` to ``conv2DFwd`` and as ``kept=`` to ``conv2DBwd``; for layers
    whose kernels share no staged layout it stays empty and both calls behave as without it."""

    def __init__(self):
        self.workspace = None


def setSmMargin(sms):
    """Leaves `sms` SMs free of the persistent tensor-core kernels from the next call on (process-wide), so that a kernel on
    another stream -- the all-reduce of a filter gradient beside backward-data -- finds SMs to run on. 0 restores the default."""
    _lib.check(_lib.lib().pcb_set_sm_margin(int(sms)))


def getSmMargin():
    return int(_lib.lib().pcb_get_sm_margin())


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _check_tensor(t, name, dtype=None, shape=None):
    if not t.is_cuda:
        raise ValueError("%s must be a CUDA tensor (no CPU fallback exists)" % name)
    if not t.is_contiguous():
        raise ValueError("%s must be contiguous" % name)
    if dtype is not None and t.dtype != dtype:
        raise ValueError("%s dtype mismatch: %s vs %s" % (name, t.dtype, dtype))
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError("%s shape mismatch: %s vs expected %s" % (name, tuple(t.shape), tuple(shape)))


def _raw_stream(index=None):
    """The current CUDA stream of a device as an integer handle (the fast path of ``torch.cuda.current_stream``, which
    builds a Python stream object on every call)."""
    if index is None:
        index = torch.cuda.current_device()
    getter = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if getter is not None:
        return getter(index)
    return torch.cuda.current_stream(index).cuda_stream


def _stream(index=None):
    return ctypes.c_void_p(_raw_stream(index))


class _OnDevice:
    """``torch.cuda.device(index)`` that does nothing when the device already is the current one (the usual case)."""

    __slots__ = ("index", "guard")

    def __init__(self, index):
        self.index, self.guard = index, None

    def __enter__(self):
        if torch.cuda.current_device() != self.index:
            self.guard = torch.cuda.device(self.index)
            self.guard.__enter__()
        return self

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)
            self.guard = None
        return False


# upstride::Algebra -> pcb_algebra (the C ABI keeps quaternion at zero)
_ALGEBRAS = {Algebra.QUATERNION: 0, Algebra.REAL: 1, Algebra.COMPLEX: 2, Algebra.GA_300: 3}


_DATA_FORMATS = {DataFormat.NCHW: 0, DataFormat.NHWC: 1}
_FILTER_LAYOUTS = {FilterLayout.OIHW: 0, FilterLayout.OHWI: 1, FilterLayout.HWIO: 2}


def _conv_desc(descriptor, dtype, context, engine, has_bias=False, require_input_grad=False):
    """The C descriptor of a call; built once per (descriptor object, dtype, context settings, engine, flags) and kept on
    the descriptor object (descriptors do not change after construction)."""
    key = (dtype, context.variant(), int(context.conv_fp16_policy), engine, bool(has_bias), bool(require_input_grad))
    cache = descriptor.__dict__.setdefault("_pcb_conv_desc", {})
    d = cache.get(key)
    if d is None:
        d = cache[key] = _build_conv_desc(descriptor, dtype, context, engine, has_bias, require_input_grad)
    return d


def _build_conv_desc(descriptor, dtype, context, engine, has_bias, require_input_grad):
    algebra = descriptor.getAlgebra()
    dim = MULTIVECTOR_DIM[algebra]
    data_format, filter_layout = descriptor.getDataFormat(), descriptor.getFilterLayout()
    if data_format not in _DATA_FORMATS or filter_layout not in _FILTER_LAYOUTS:
        raise _lib.BackendError(_lib.PCB_ERR_UNSUPPORTED, "unsupported tensor layout for a convolution")
    cd, hd, wd = _dims(data_format)                 # real filters carry no leading component axis: _filter_dims accounts for it
    fo, fi, fh, fw = _filter_dims(filter_layout, algebra)
    ishape, fshape = descriptor.getInputShape(), descriptor.getFilterShape()
    real = descriptor.isRealValuedInput() and algebra != Algebra.REAL
    if not real and ishape[0] % dim != 0:
        raise ValueError("leading input dimension must be a multiple of %d (components stacked on the batch axis)" % dim)
    if ishape[cd] != fshape[fi] * descriptor.getGroups():
        raise ValueError("input channels mismatch: %d vs %d" % (ishape[cd], fshape[fi]))
    d = _lib.ConvDesc()
    d.dtype = _DTYPES[dtype]
    d.algebra = _ALGEBRAS[algebra]
    d.data_format = _DATA_FORMATS[data_format]
    d.filter_layout = _FILTER_LAYOUTS[filter_layout]
    d.n = ishape[0] if real else ishape[0] // dim
    d.ci, d.co = fshape[fi], fshape[fo]
    d.h, d.w = ishape[hd], ishape[wd]
    d.kh, d.kw = fshape[fh], fshape[fw]
    d.stride_h, d.stride_w = descriptor.getStride()
    d.dilation_h, d.dilation_w = descriptor.getDilation()
    d.pad_top, d.pad_left = descriptor.getPaddingBefore()
    d.pad_bottom, d.pad_right = descriptor.getPaddingAfter()
    d.groups = descriptor.getGroups()
    d.has_bias = int(has_bias)
    d.require_input_grad = int(require_input_grad)
    d.real_valued_input = int(real)
    d.variant = context.variant()
    d.fp16_policy = int(context.conv_fp16_policy)
    d.engine = engine
    return d


def conv2DFwd(inputTensor, filterTensor, biasTensor, outputTensor, descriptor, context=None, engine=_lib.ENGINE_AUTO, keep=None):
    """y = x (*) w [+ bias]; mirrors ``upstride::conv2DFwd`` (reference ``src/upstride.hpp:18-33``).

    ``keep`` (not in the reference): a ``KeptInput``; see there."""
    dev = Device.get(inputTensor.device)
    context = context or dev.getContext()
    _check_tensor(inputTensor, "input", shape=descriptor.getInputShape())
    _check_tensor(filterTensor, "filter", inputTensor.dtype, descriptor.getFilterShape())
    _check_tensor(outputTensor, "output", inputTensor.dtype, descriptor.getOutputShape())
    if biasTensor is not None:
        if not descriptor.isBiasUsed():
            raise ValueError("Bias application is not configured for this operation")
        _check_tensor(biasTensor, "bias", inputTensor.dtype, descriptor.getBiasShape())
    if inputTensor.numel() == 0:
        return      # empty input: silent no-op (reference src/conv2d.hpp:81-82)
    d = _conv_desc(descriptor, inputTensor.dtype, context, engine, has_bias=biasTensor is not None)
    L = _lib.lib()
    with dev.accessControl, _OnDevice(dev.index):
        need = getattr(d, "_fwd_need", None)           # both queries depend on the descriptor alone: asked once
        if need is None:
            need = d._fwd_need = L.pcb_qconv2d_fwd_workspace_size(ctypes.byref(d))
            d._keeps = bool(L.pcb_qconv2d_fwd_keeps_input(ctypes.byref(d)))
        if keep is not None and d._keeps:
            if keep.workspace is None or keep.workspace.numel() < need or keep.workspace.device != inputTensor.device:
                keep.workspace = torch.empty(need, dtype=torch.uint8, device=inputTensor.device)
            ws = keep.workspace
        else:
            ws = dev.requestWorkspace(need)
        _lib.check(L.pcb_qconv2d_fwd(ctypes.byref(d), _ptr(inputTensor), _ptr(filterTensor), _ptr(biasTensor),
                                     _ptr(outputTensor), _ptr(ws), ws.numel(), _stream()))
        dev._after_op()


def conv2DBwd(inputTensor, filterTensor, gradTensor, filterGradTensor, inputGradTensor, descriptor, context=None,
              engine=_lib.ENGINE_AUTO, on_filter_grad=None, kept=None):
    """dW (always) and dX (when the descriptor requires it); mirrors ``upstride::conv2DBwd``
    (reference ``src/upstride.hpp:35-51``).

    ``on_filter_grad`` (not in the reference): a callable invoked after the filter gradient has been enqueued and
    before backward-data is, e.g. to start its all-reduce on another stream so that it overlaps backward-data.
    ``kept`` (not in the reference): the ``KeptInput`` given to this layer's forward call."""
    dev = Device.get(filterTensor.device)
    context = context or dev.getContext()
    _check_tensor(inputTensor, "input", shape=descriptor.getInputShape())
    _check_tensor(filterTensor, "filter", inputTensor.dtype, descriptor.getFilterShape())
    _check_tensor(gradTensor, "grad", inputTensor.dtype, descriptor.getOutputShape())
    _check_tensor(filterGradTensor, "filterGrad", inputTensor.dtype, descriptor.getFilterShape())
    need_dx = descriptor.isInputGradientRequired()
    if need_dx:
        if descriptor.isRealValuedInput():
            raise RuntimeError("Input gradient required for type0 input tensor")   # std::logic_error in the reference
        _check_tensor(inputGradTensor, "inputGrad", inputTensor.dtype, descriptor.getInputShape())
    if inputTensor.numel() == 0:
        filterGradTensor.zero_()     # reference src/conv2d.hpp:341-344
        return
    d = _conv_desc(descriptor, inputTensor.dtype, context, engine, require_input_grad=need_dx)
    L = _lib.lib()
    with dev.accessControl, _OnDevice(dev.index):
        need = getattr(d, "_bwd_need", None)
        if need is None:
            need = d._bwd_need = L.pcb_qconv2d_bwd_workspace_size(ctypes.byref(d))
        ws = dev.requestWorkspace(need)
        if kept is not None and kept.workspace is not None and on_filter_grad is None:
            _lib.check(L.pcb_qconv2d_bwd_kept(ctypes.byref(d), _ptr(inputTensor), _ptr(filterTensor), _ptr(gradTensor),
                                              _ptr(filterGradTensor), _ptr(inputGradTensor) if need_dx else None,
                                              _ptr(kept.workspace), kept.workspace.numel(), _ptr(ws), ws.numel(), _stream()))
        elif on_filter_grad is None:
            _lib.check(L.pcb_qconv2d_bwd(ctypes.byref(d), _ptr(inputTensor), _ptr(filterTensor), _ptr(gradTensor),
                                         _ptr(filterGradTensor), _ptr(inputGradTensor) if need_dx else None,
                                         _ptr(ws), ws.numel(), _stream()))
        else:
            _lib.check(L.pcb_qconv2d_bwd_filter(ctypes.byref(d), _ptr(inputTensor), _ptr(gradTensor), _ptr(filterGradTensor),
                                                _ptr(ws), ws.numel(), _stream()))
            on_filter_grad(filterGradTensor)
            if need_dx:
                _lib.check(L.pcb_qconv2d_bwd_data(ctypes.byref(d), _ptr(filterTensor), _ptr(gradTensor), _ptr(inputGradTensor),
                                                  _ptr(ws), ws.numel(), _stream()))
        dev._after_op()


def _dense_desc(descriptor, dtype, context, engine, has_bias=False, require_input_grad=False):
    algebra = descriptor.getAlgebra()
    dim = MULTIVECTOR_DIM[algebra]
    ishape = descriptor.getInputShape()
    if ishape[0] % dim != 0:
        raise ValueError("leading input dimension must be a multiple of %d (components stacked on the batch axis)" % dim)
    if ishape[1] != descriptor.getInputChannels():
        raise ValueError("input features mismatch: %d vs %d" % (ishape[1], descriptor.getInputChannels()))
    d = _lib.DenseDesc()
    d.dtype = _DTYPES[dtype]
    d.algebra = _ALGEBRAS[algebra]
    d.batch = ishape[0] // dim
    d.in_features = ishape[1]
    d.out_features = descriptor.getOutputChannels()
    d.filter_oi = int(descriptor.getFilterLayout() == FilterLayout.OI)
    d.has_bias = int(has_bias)
    d.require_input_grad = int(require_input_grad)
    d.variant = context.variant()
    d.engine = engine
    return d


def denseFwd(inputTensor, filterTensor, biasTensor, outputTensor, descriptor, context=None, engine=_lib.ENGINE_AUTO):
    """Mirrors ``upstride::denseFwd`` (reference ``src/upstride.hpp:53-68``)."""
    dev = Device.get(inputTensor.device)
    context = context or dev.getContext()
    _check_tensor(inputTensor, "input", shape=descriptor.getInputShape())
    _check_tensor(filterTensor, "filter", inputTensor.dtype, descriptor.getFilterShape())
    _check_tensor(outputTensor, "output", inputTensor.dtype, descriptor.getOutputShape())
    if biasTensor is not None:
        if not descriptor.isBiasUsed():
            raise ValueError("Bias application is not configured for this scalar Dense operation")
        _check_tensor(biasTensor, "bias", inputTensor.dtype, descriptor.getBiasShape())
    if inputTensor.numel() == 0:
        return
    d = _dense_desc(descriptor, inputTensor.dtype, context, engine, has_bias=biasTensor is not None)
    L = _lib.lib()
    with dev.accessControl, _OnDevice(dev.index):
        need = L.pcb_qdense_fwd_workspace_size(ctypes.byref(d))
        ws = dev.requestWorkspace(need)
        _lib.check(L.pcb_qdense_fwd(ctypes.byref(d), _ptr(inputTensor), _ptr(filterTensor), _ptr(biasTensor),
                                    _ptr(outputTensor), _ptr(ws), ws.numel(), _stream()))
        dev._after_op()


def denseBwd(inputTensor, filterTensor, gradTensor, filterGradTensor, inputGradTensor, descriptor, context=None,
             engine=_lib.ENGINE_AUTO):
    """Mirrors ``upstride::denseBwd`` (reference ``src/upstride.hpp:70-86``). The filter gradient is written
    input-major, ``[4, I, O]``, whatever the filter layout, as both reference backends do."""
    dev = Device.get(inputTensor.device)
    context = context or dev.getContext()
    _check_tensor(inputTensor, "input", shape=descriptor.getInputShape())
    _check_tensor(filterTensor, "filter", inputTensor.dtype, descriptor.getFilterShape())
    _check_tensor(gradTensor, "grad", inputTensor.dtype, descriptor.getOutputShape())
    if filterGradTensor.numel() != filterTensor.numel():
        raise ValueError("filterGrad size mismatch")
    _check_tensor(filterGradTensor, "filterGrad", inputTensor.dtype)
    need_dx = descriptor.isInputGradientRequired()
    if need_dx:
        _check_tensor(inputGradTensor, "inputGrad", inputTensor.dtype, descriptor.getInputShape())
    if inputTensor.numel() == 0:
        filterGradTensor.zero_()
        return
    d = _dense_desc(descriptor, inputTensor.dtype, context, engine, require_input_grad=need_dx)
    L = _lib.lib()
    with dev.accessControl, _OnDevice(dev.index):
        need = L.pcb_qdense_bwd_workspace_size(ctypes.byref(d))
        ws = dev.requestWorkspace(need)
        _lib.check(L.pcb_qdense_bwd(ctypes.byref(d), _ptr(inputTensor), _ptr(filterTensor), _ptr(gradTensor),
                                    _ptr(filterGradTensor), _ptr(inputGradTensor) if need_dx else None,
                                    _ptr(ws), ws.numel(), _stream()))
        dev._after_op()
