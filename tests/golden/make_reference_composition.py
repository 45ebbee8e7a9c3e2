"""Generates ``reference_composition.npz``: inputs and outputs of the REFERENCE's own four operations (forward and
backward, both quaternion formulations, the other algebras, layouts, groups, real-valued input, dense), run here
from the reference's sources through ``oracle/reference_lib.py`` (the reference's composition code over exact
scalar convolutions; see ``oracle/ref_driver.cc``).

Run where a reference checkout is present:  python tests/golden/make_reference_composition.py
The file travels with the repository; the tests read it and never need the reference.

Every input value is a multiple of 1/16 in [-1, 1] (of 1/32 for the filters), so it is exact in fp32, fp16 and bf16:
one set of vectors serves every storage type. Arrays are stored in the canonical layout (NCHW / OIHW, dense filter as
given); a case that ran in another layout names it, and its tensors were permuted on the way in and out.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

REAL, COMPLEX, QUATERNION, GA_300 = 0, 1, 2, 3
DIMS = {REAL: 1, COMPLEX: 2, QUATERNION: 4, GA_300: 8}

# name, algebra, batch, ci, co, h, w, kh, kw, stride, dilation, padding, bias, data_format, filter_layout, groups, real_input
CONV_CASES = [
    ("q_3x3_same_bias",   QUATERNION, 2, 3, 5, 7, 6, 3, 3, (1, 1), (1, 1), "SAME",  True,  "NCHW", "OIHW", 1, False),
    ("q_3x2_s2_same",     QUATERNION, 1, 4, 6, 9, 8, 3, 2, (2, 2), (1, 1), "SAME",  False, "NCHW", "OIHW", 1, False),
    ("q_dilated_valid",   QUATERNION, 1, 2, 3, 9, 9, 3, 3, (1, 2), (2, 1), "VALID", False, "NCHW", "OIHW", 1, False),
    ("q_pointwise",       QUATERNION, 2, 8, 8, 5, 5, 1, 1, (1, 1), (1, 1), "VALID", True,  "NCHW", "OIHW", 1, False),
    ("q_pointwise_s2",    QUATERNION, 1, 8, 16, 8, 8, 1, 1, (2, 2), (1, 1), "VALID", False, "NCHW", "OIHW", 1, False),
    ("q_nhwc_hwio",       QUATERNION, 2, 5, 6, 9, 7, 3, 2, (2, 1), (1, 1), "SAME",  True,  "NHWC", "HWIO", 1, False),
    ("q_nhwc_ohwi",       QUATERNION, 2, 5, 6, 9, 7, 3, 2, (2, 1), (1, 1), "SAME",  True,  "NHWC", "OHWI", 1, False),
    ("q_nchw_hwio",       QUATERNION, 1, 4, 4, 6, 6, 3, 3, (1, 1), (1, 1), "SAME",  False, "NCHW", "HWIO", 1, False),
    ("q_groups2",         QUATERNION, 2, 6, 4, 9, 7, 3, 3, (2, 1), (1, 1), "SAME",  True,  "NCHW", "OIHW", 2, False),
    ("q_depthwise",       QUATERNION, 1, 4, 4, 6, 6, 3, 3, (1, 1), (1, 1), "SAME",  False, "NCHW", "OIHW", 4, False),
    ("q_real_input_7x7",  QUATERNION, 2, 3, 4, 10, 10, 7, 7, (2, 2), (1, 1), "SAME", False, "NCHW", "OIHW", 1, True),
    ("q_channels16",      QUATERNION, 1, 16, 32, 6, 6, 3, 3, (1, 1), (1, 1), "SAME", True, "NCHW", "OIHW", 1, False),
    ("complex_3x3",       COMPLEX,    2, 3, 4, 7, 6, 3, 3, (1, 1), (1, 1), "SAME",  True,  "NCHW", "OIHW", 1, False),
    ("ga300_3x3",         GA_300,     1, 2, 3, 5, 5, 3, 3, (1, 1), (1, 1), "VALID", True,  "NCHW", "OIHW", 1, False),
    ("real_3x3_s2",       REAL,       2, 3, 4, 7, 6, 3, 3, (2, 2), (1, 1), "SAME",  True,  "NCHW", "OIHW", 1, False),
]

# name, algebra, batch, inputs, outputs, oi, bias. The OI cases are square: the reference's CPU backend describes an OI
# filter by its own dims (O, I) with the transposed tag (src/backend/onednn/dense.hpp:33), which a matrix product with
# K = I accepts only when O = I.
DENSE_CASES = [
    ("q_dense_io_bias", QUATERNION, 3, 5, 7, False, True),
    ("q_dense_oi",      QUATERNION, 4, 6, 6, True,  False),
    ("q_dense_32",      QUATERNION, 8, 32, 16, False, True),
    ("complex_dense",   COMPLEX,    3, 4, 5, False, True),
    ("ga300_dense_oi",  GA_300,     2, 4, 4, True,  True),
    ("real_dense",      REAL,       3, 5, 4, False, True),
]


def quantised(seed, shape, steps):
    return (np.random.default_rng(seed).integers(-steps, steps + 1, size=shape) / float(steps)).astype(np.float32)


def to_layout(a, layout, lead):
    """Canonical (NCHW / OIHW, with `lead` leading multivector axes) -> the named layout."""
    a = np.asarray(a)
    n = a.ndim
    perm = {"NCHW": None, "OIHW": None, "NHWC": (0, 2, 3, 1), "OHWI": (0, 2, 3, 1), "HWIO": (2, 3, 1, 0)}[layout]
    if perm is None:
        return a
    perm = tuple(range(lead)) + tuple(lead + p for p in perm)
    assert len(perm) == n
    return np.ascontiguousarray(a.transpose(perm))


def from_layout(a, layout, lead):
    perm = {"NCHW": None, "OIHW": None, "NHWC": (0, 3, 1, 2), "OHWI": (0, 3, 1, 2), "HWIO": (3, 2, 0, 1)}[layout]
    if perm is None:
        return np.asarray(a)
    perm = tuple(range(lead)) + tuple(lead + p for p in perm)
    return np.ascontiguousarray(np.asarray(a).transpose(perm))


def main():
    from oracle import reference_lib as ref
    out = {}
    for idx, (name, alg, n, ci, co, h, w_, kh, kw, stride, dil, padding, bias, df, fl, groups, real_in) in enumerate(CONV_CASES):
        d = DIMS[alg]
        lead = 0 if alg == REAL else 1
        x = quantised(1000 + 10 * idx, ((1 if real_in else d) * n, ci, h, w_), 16)
        wshape = (co, ci // groups, kh, kw) if alg == REAL else (d, co, ci // groups, kh, kw)
        w = quantised(1001 + 10 * idx, wshape, 32)
        b = quantised(1002 + 10 * idx, (co,) if alg == REAL else (d, co), 16) if bias else None
        xl, wl = to_layout(x, df, 0), to_layout(w, fl, lead)
        out[name + "/x"], out[name + "/w"] = x, w
        if b is not None:
            out[name + "/b"] = b
        for mo in (0, 1):
            y = ref.conv2d_fwd(xl, wl, b, stride, dil, padding, alg, bool(mo), real_in, df, fl, groups)
            yc = from_layout(y, df, 0)
            if mo == 0:
                dy = quantised(1003 + 10 * idx, yc.shape, 16)
                out[name + "/dy"] = dy
            dw, dx = ref.conv2d_bwd(xl, wl, to_layout(dy, df, 0), stride, dil, padding, alg, bool(mo), not real_in, real_in, df, fl, groups)
            tag = name + ("/16p" if mo else "/8p")
            out[tag + "/y"] = yc
            out[tag + "/dw"] = from_layout(dw, fl, lead)
            if dx is not None:
                out[tag + "/dx"] = from_layout(dx, df, 0)
            assert np.isfinite(yc).all() and np.isfinite(out[tag + "/dw"]).all()
    for idx, (name, alg, bsz, i, o, oi, bias) in enumerate(DENSE_CASES):
        d = DIMS[alg]
        x = quantised(5000 + 10 * idx, (d * bsz, i), 16)
        wshape = ((o, i) if oi else (i, o))
        w = quantised(5001 + 10 * idx, wshape if alg == REAL else (d,) + wshape, 32)
        b = quantised(5002 + 10 * idx, (o,) if alg == REAL else (d, o), 16) if bias else None
        out[name + "/x"], out[name + "/w"] = x, w
        if b is not None:
            out[name + "/b"] = b
        for mo in (0, 1):
            y = ref.dense_fwd(x, w, b, oi, alg, bool(mo))
            if mo == 0:
                dy = quantised(5003 + 10 * idx, y.shape, 16)
                out[name + "/dy"] = dy
            dw, dx = ref.dense_bwd(x, w, dy, oi, alg, bool(mo), True)
            tag = name + ("/16p" if mo else "/8p")
            out[tag + "/y"], out[tag + "/dw"], out[tag + "/dx"] = y, dw, dx
            assert np.isfinite(y).all() and np.isfinite(dw).all() and np.isfinite(dx).all()
    path = os.path.join(HERE, "reference_composition.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
