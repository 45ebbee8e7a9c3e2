"""ctypes binding of the CPU oracle (``oracle.c``). TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may import this module;
the product package never does. Arrays are float32 numpy arrays in the reference's layouts:
activations ``[4*N, C, H, W]`` with component ``c`` of sample ``n`` at leading index ``c*N + n``
(reference ``src/backend/tensor.hpp:501-545``), conv weights ``[4, Co, Ci, kh, kw]``, conv bias ``[4, Co]``,
dense input ``[4*B, I]``, dense weights ``[4, I, O]`` (IO) or ``[4, O, I]`` (OI), dense bias ``[4, O]``.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

REAL, COMPLEX, QUATERNION, GA_300 = 0, 1, 2, 3
DIMS = {REAL: 1, COMPLEX: 2, QUATERNION: 4, GA_300: 8}
VARIANT_16P, VARIANT_8P = 0, 1
VALID, SAME = 0, 1


class Geom(ctypes.Structure):
    _fields_ = [(k, ctypes.c_int) for k in
                ("n", "ci", "co", "h", "w", "kh", "kw", "sh", "sw", "dh", "dw", "pt", "pl", "pb", "pr")]


def build(force=False):
    """Compiles ``oracle.c`` into ``liboracle.so`` with the Makefile next to it."""
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "oracle.c")):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        fp = ctypes.POINTER(ctypes.c_float)
        gp = ctypes.POINTER(Geom)
        _lib.orc_conv2d_fwd.argtypes = [fp, fp, fp, fp, gp, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        _lib.orc_conv2d_bwd.argtypes = [fp, fp, fp, fp, fp, gp, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        _lib.orc_dense_fwd.argtypes = [fp, fp, fp, fp] + [ctypes.c_int] * 6
        _lib.orc_dense_bwd.argtypes = [fp, fp, fp, fp, fp] + [ctypes.c_int] * 7
        _lib.orc_real_conv_fwd.argtypes = [fp, fp, fp, fp, gp]
        _lib.orc_windowed_output_size_and_padding.argtypes = [ctypes.c_int] * 5 + [ctypes.POINTER(ctypes.c_int)] * 2
        _lib.orc_windowed_output_size.argtypes = [ctypes.c_int] * 6
        _lib.orc_sign_table.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
    return _lib


def _p(a):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def same_or_valid_padding(size, k, dilation, stride, mode):
    """Returns (output size, pad before, pad after) under the TF rule (reference ``src/utils.cc:10-38``)."""
    b, a = ctypes.c_int(0), ctypes.c_int(0)
    out = lib().orc_windowed_output_size_and_padding(size, k, dilation, stride, mode, ctypes.byref(b), ctypes.byref(a))
    return out, b.value, a.value


def output_size(size, k, dilation, stride, before, after):
    return lib().orc_windowed_output_size(size, k, dilation, stride, before, after)


def sign_table(algebra):
    """The product table of an algebra: D*D triples (left, right, sign), rows of D per output component."""
    n = DIMS[algebra] ** 2
    out = (ctypes.c_int * (3 * n))()
    lib().orc_sign_table(algebra, out)
    return [(out[3 * i], out[3 * i + 1], out[3 * i + 2]) for i in range(n)]


def quaternion_sign_table():
    return sign_table(QUATERNION)


def _geom(xshape, wshape, stride, dilation, pad, dims, real_input):
    n = xshape[0] if real_input else xshape[0] // dims
    co, ci, kh, kw = wshape[-4:]
    assert xshape[1] == ci, "input channels mismatch"
    sh, sw = stride
    dh, dw = dilation
    pt, pl, pb, pr = pad
    g = Geom(n, ci, co, xshape[2], xshape[3], kh, kw, sh, sw, dh, dw, pt, pl, pb, pr)
    ho = output_size(g.h, kh, dh, sh, pt, pb)
    wo = output_size(g.w, kw, dw, sw, pl, pr)
    return g, ho, wo


def conv2d_fwd(x, w, bias=None, stride=(1, 1), dilation=(1, 1), pad=(0, 0, 0, 0), algebra=QUATERNION,
               variant=VARIANT_16P, real_input=False):
    """Hyper-complex conv forward; ``pad`` = (top, left, bottom, right)."""
    dims = DIMS[algebra]
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
    g, ho, wo = _geom(x.shape, w.shape, stride, dilation, pad, dims, real_input)
    y = np.zeros((dims * g.n, g.co, ho, wo), np.float32)
    rc = lib().orc_conv2d_fwd(_p(x), _p(w), _p(bias), _p(y), ctypes.byref(g), algebra, variant, int(real_input))
    if rc != 0:
        raise ValueError("oracle: unsupported combination")
    return y


def conv2d_bwd(x, w, dy, stride=(1, 1), dilation=(1, 1), pad=(0, 0, 0, 0), algebra=QUATERNION,
               variant=VARIANT_16P, need_dx=True):
    """Returns (dW, dX or None)."""
    dims = DIMS[algebra]
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    dy = np.ascontiguousarray(dy, np.float32)
    g, ho, wo = _geom(x.shape, w.shape, stride, dilation, pad, dims, False)
    assert dy.shape == (dims * g.n, g.co, ho, wo), (dy.shape, (dims * g.n, g.co, ho, wo))
    dw = np.zeros_like(w)
    dx = np.zeros_like(x)
    rc = lib().orc_conv2d_bwd(_p(x), _p(w), _p(dy), _p(dw), _p(dx), ctypes.byref(g), algebra, variant, int(need_dx))
    if rc != 0:
        raise ValueError("oracle: unsupported combination")
    return dw, (dx if need_dx else None)


def dense_fwd(x, w, bias=None, oi=False, algebra=QUATERNION, variant=VARIANT_16P):
    dims = DIMS[algebra]
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
    b, i = x.shape[0] // dims, x.shape[1]
    o = w.shape[-2] if oi else w.shape[-1]
    assert (w.shape[-1] if oi else w.shape[-2]) == i
    y = np.zeros((dims * b, o), np.float32)
    rc = lib().orc_dense_fwd(_p(x), _p(w), _p(bias), _p(y), b, i, o, int(oi), algebra, variant)
    if rc != 0:
        raise ValueError("oracle: unsupported combination")
    return y


def dense_bwd(x, w, dy, oi=False, algebra=QUATERNION, variant=VARIANT_16P, need_dx=True):
    """Returns (dW in [D, I, O] orientation -- as both reference backends emit it -- and dX or None)."""
    dims = DIMS[algebra]
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    dy = np.ascontiguousarray(dy, np.float32)
    b, i = x.shape[0] // dims, x.shape[1]
    o = dy.shape[1]
    dw = np.zeros((dims, i, o), np.float32)
    dx = np.zeros_like(x)
    rc = lib().orc_dense_bwd(_p(x), _p(w), _p(dy), _p(dw), _p(dx), b, i, o, int(oi), algebra, variant, int(need_dx))
    if rc != 0:
        raise ValueError("oracle: unsupported combination")
    return dw, (dx if need_dx else None)
