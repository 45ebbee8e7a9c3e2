"""ctypes binding of ``_ref/libupstride_ref.so``: the REFERENCE's own four operations on its CPU device, compiled
from the reference's sources by ``make ref`` (see the Makefile next to this file) with ``dnnl_stub/dnnl.hpp`` standing
in for oneDNN. TEST INFRASTRUCTURE ONLY: it exists where a reference checkout is present, it validates the oracle
and generates the golden vectors under ``tests/golden/``; nothing in the product imports it.

Arrays are float32 numpy arrays in whatever layout the call names; shapes are the reference's
(``[D*N, C, H, W]`` or ``[D*N, H, W, C]`` activations, ``[D, O, I, kh, kw]`` / ``[D, O, kh, kw, I]`` /
``[D, kh, kw, I, O]`` filters, no leading D for the real algebra)."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_ref", "libupstride_ref.so")

REAL, COMPLEX, QUATERNION, GA_300 = 0, 1, 2, 3
DIMS = {REAL: 1, COMPLEX: 2, QUATERNION: 4, GA_300: 8}
SAME, VALID, EXPLICIT = 0, 1, 2
DATA_FORMATS = {"NCHW": 0, "NHWC": 1}
FILTER_LAYOUTS = {"OIHW": 0, "OHWI": 1, "HWIO": 2, "IO": 3, "OI": 4}

_lib = None


def available(reference=None):
    """True when the library is built or can be built (a reference checkout is present)."""
    return os.path.exists(_LIB_PATH) or os.path.isdir(os.path.join(reference or _default_reference(), "src"))


def _default_reference():
    return os.environ.get("UPSTRIDE_REFERENCE", os.path.normpath(os.path.join(_HERE, "..", "..", "reference")))


def build(reference=None):
    reference = reference or _default_reference()
    if os.path.isdir(os.path.join(reference, "src")):
        subprocess.check_call(["make", "-C", _HERE, "ref", "REFERENCE=" + reference], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _f(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _shape(a):
    arr = (ctypes.c_int * a.ndim)(*a.shape)
    return arr, a.ndim


def _c(a):
    return None if a is None else np.ascontiguousarray(a, np.float32)


def _out_hw(size, k, dilation, stride, before, after):
    return (size + before + after - (k - 1) * dilation - 1) // stride + 1


def same_padding(size, k, dilation, stride):
    """(before, after) of TensorFlow-style SAME padding, as the reference computes it (src/utils.cc:25-31)."""
    out = (size + stride - 1) // stride
    needed = max(0, (out - 1) * stride + (k - 1) * dilation + 1 - size)
    return needed // 2, needed - needed // 2


def padding_of(padding, h, w, kh, kw, stride, dilation):
    """(top, left, bottom, right) the reference derives for a preset. Its descriptor rejects EXPLICIT padding
    (src/utils.cc:33-34 is reached from src/backend/conv2d_descriptor.hpp:165-173), so only the presets can be run."""
    if padding == "VALID":
        return (0, 0, 0, 0)
    (pt, pb), (pl, pr) = same_padding(h, kh, dilation[0], stride[0]), same_padding(w, kw, dilation[1], stride[1])
    return (pt, pl, pb, pr)


def _conv_args(stride, dilation, padding, groups, algebra, data_format, filter_layout):
    padv = (ctypes.c_int * 4)(0, 0, 0, 0)
    return (stride[0], stride[1], dilation[0], dilation[1], {"SAME": SAME, "VALID": VALID}[padding], padv, 0, groups, algebra,
            DATA_FORMATS[data_format], FILTER_LAYOUTS[filter_layout])


def _filter_dims(w, filter_layout, algebra):
    s = w.shape if algebra == REAL else w.shape[1:]
    if filter_layout == "OIHW":
        return s[0], s[1], s[2], s[3]
    if filter_layout == "OHWI":
        return s[0], s[3], s[1], s[2]
    return s[3], s[2], s[0], s[1]          # HWIO


def conv2d_fwd(x, w, bias=None, stride=(1, 1), dilation=(1, 1), padding="VALID", algebra=QUATERNION, memory_optimized=False,
               real_input=False, data_format="NCHW", filter_layout="OIHW", groups=1):
    """``padding`` is "SAME" or "VALID"."""
    x, w, bias = _c(x), _c(w), _c(bias)
    d = DIMS[algebra]
    co, _, kh, kw = _filter_dims(w, filter_layout, algebra)
    h, wd = (x.shape[2], x.shape[3]) if data_format == "NCHW" else (x.shape[1], x.shape[2])
    pad = padding_of(padding, h, wd, kh, kw, stride, dilation)
    ho = _out_hw(h, kh, dilation[0], stride[0], pad[0], pad[2])
    wo = _out_hw(wd, kw, dilation[1], stride[1], pad[1], pad[3])
    n_out = x.shape[0] * d if real_input else x.shape[0]
    y = np.full((n_out, co, ho, wo) if data_format == "NCHW" else (n_out, ho, wo, co), np.nan, np.float32)
    xs, xr = _shape(x)
    ws, wr = _shape(w)
    ys, yr = _shape(y)
    bs, br = _shape(bias) if bias is not None else (None, 0)
    rc = lib().ref_conv2d_fwd(int(memory_optimized), _f(x), xs, xr, _f(w), ws, wr, _f(bias), bs, br, _f(y), ys, yr,
                              *_conv_args(stride, dilation, padding, groups, algebra, data_format, filter_layout), int(real_input))
    if rc != 0:
        raise ValueError("the reference raised an exception")
    return y


def conv2d_bwd(x, w, dy, stride=(1, 1), dilation=(1, 1), padding="VALID", algebra=QUATERNION, memory_optimized=False, need_dx=True,
               real_input=False, data_format="NCHW", filter_layout="OIHW", groups=1):
    x, w, dy = _c(x), _c(w), _c(dy)
    dw = np.full(w.shape, np.nan, np.float32)
    dx = np.full(x.shape, np.nan, np.float32)
    xs, xr = _shape(x)
    ws, wr = _shape(w)
    ys, yr = _shape(dy)
    rc = lib().ref_conv2d_bwd(int(memory_optimized), _f(x), xs, xr, _f(w), ws, wr, _f(dy), ys, yr, _f(dw), _f(dx),
                              *_conv_args(stride, dilation, padding, groups, algebra, data_format, filter_layout), int(need_dx), int(real_input))
    if rc != 0:
        raise ValueError("the reference raised an exception")
    return dw, (dx if need_dx else None)


def dense_fwd(x, w, bias=None, oi=False, algebra=QUATERNION, memory_optimized=False):
    x, w, bias = _c(x), _c(w), _c(bias)
    o = w.shape[-2] if oi else w.shape[-1]
    y = np.full((x.shape[0], o), np.nan, np.float32)
    xs, _ = _shape(x)
    ws, wr = _shape(w)
    ys, _ = _shape(y)
    bs, br = _shape(bias) if bias is not None else (None, 0)
    rc = lib().ref_dense_fwd(int(memory_optimized), _f(x), xs, _f(w), ws, wr, _f(bias), bs, br, _f(y), ys, algebra,
                             FILTER_LAYOUTS["OI" if oi else "IO"])
    if rc != 0:
        raise ValueError("the reference raised an exception")
    return y


def dense_bwd(x, w, dy, oi=False, algebra=QUATERNION, memory_optimized=False, need_dx=True):
    """Returns (dW as the reference writes it: the filter's element count, filled input-major ``[D, I, O]``
    whatever the filter layout; dX or None)."""
    x, w, dy = _c(x), _c(w), _c(dy)
    i = x.shape[1]
    o = dy.shape[1]
    dw = np.full(w.shape, np.nan, np.float32)
    dx = np.full(x.shape, np.nan, np.float32)
    xs, _ = _shape(x)
    ws, wr = _shape(w)
    ys, _ = _shape(dy)
    rc = lib().ref_dense_bwd(int(memory_optimized), _f(x), xs, _f(w), ws, wr, _f(dy), ys, _f(dw), _f(dx), algebra,
                             FILTER_LAYOUTS["OI" if oi else "IO"], int(need_dx))
    if rc != 0:
        raise ValueError("the reference raised an exception")
    lead = () if algebra == REAL else (DIMS[algebra],)
    return dw.reshape(lead + (i, o)), (dx if need_dx else None)
