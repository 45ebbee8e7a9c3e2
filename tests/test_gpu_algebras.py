"""GPU parity for the other algebras of the reference's Algebra enum (real, complex, GA(3,0,0)): the same kernels
with a 1x1, 2x2 or 8x8 signed block (reference tables src/algebras.cc:5-145) against the CPU oracle, plus the
reference's own known-answer vectors for them (tests/tests.cpp:224-290, :371-423, :562-648), plus dilation.

Tolerances: 1e-5 (fp32), 2e-2 (fp16 / bf16), max|got-ref| / max|ref| per output tensor.
"""
import json
import os

import numpy as np
import pytest
import torch

import phoenix_core_b200 as pcb
from helpers import normal, rel_err, uniform

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")
# name -> (host-layer enum, oracle code, components)
ALGEBRAS = {"real": (pcb.Algebra.REAL, 0, 1), "complex": (pcb.Algebra.COMPLEX, 1, 2),
            "quaternion": (pcb.Algebra.QUATERNION, 2, 4), "ga_300": (pcb.Algebra.GA_300, 3, 8)}


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util
    return gpu_util


def _check(got, ref, dtype, gpu, what):
    assert np.all(np.isfinite(got)), what + ": output not fully written"
    err = rel_err(got, ref)
    assert err <= gpu.TOL[dtype], "%s: relative error %.3e > %.1e" % (what, err, gpu.TOL[dtype])


def _shapes(name, n, ci, co, h, w_, kh, kw):
    """Tensor shapes in the reference's conventions: real tensors carry no component axis."""
    D = ALGEBRAS[name][2]
    if name == "real":
        return (n, ci, h, w_), (co, ci, kh, kw), (co,)
    return (D * n, ci, h, w_), (D, co, ci, kh, kw), (D, co)


def _oracle_view(name, x, w, b=None):
    """The oracle takes a leading component axis for every algebra."""
    if name != "real":
        return x, w, b
    return x, w[None], (None if b is None else b[None])


@pytest.mark.parametrize("engine", ["simt", "auto"])
def test_reference_kats_other_algebras_on_gpu(gpu, engine):
    """Complex and GA(3,0,0) known-answer vectors of the reference, exact (integer-valued data)."""
    with open(GOLDEN) as f:
        cases = [c for c in json.load(f)["cases"] if c.get("algebra") in ("complex", "ga_300")]
    assert len(cases) == 4
    for case in cases:
        alg = ALGEBRAS[case["algebra"]][0]
        x = np.asarray(case["x"], np.float32).reshape(case["x_shape"])
        w = np.asarray(case["w"], np.float32).reshape(case["w_shape"])
        want = np.asarray(case["y"], np.float32).reshape(case["y_shape"])
        if case["op"] == "conv2d_fwd":
            got = gpu.run_conv_fwd(x, w, None, tuple(case["stride"]), (0, 0, 0, 0), "f32", "16p", engine, False, alg)
        else:
            got = gpu.run_dense_fwd(x, w, None, False, "f32", "16p", engine, alg)
        assert np.array_equal(got, want), (case["name"], engine)


# n, ci, co, h, w, kh, kw, stride, pad(t,l,b,r)
SHAPES = [
    (2, 3, 5, 7, 6, 3, 3, (1, 1), (1, 1, 1, 1)),
    (1, 4, 2, 9, 8, 3, 3, (2, 2), (0, 0, 1, 1)),
    (2, 16, 32, 14, 14, 3, 3, (1, 1), (1, 1, 1, 1)),
    (2, 40, 24, 6, 5, 1, 1, (1, 1), (0, 0, 0, 0)),
    (3, 32, 16, 12, 12, 3, 3, (2, 2), (0, 0, 1, 1)),
    (2, 64, 48, 8, 8, 1, 1, (1, 1), (0, 0, 0, 0)),
]


@pytest.mark.parametrize("name", ["real", "complex", "ga_300"])
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype,engine", [("f32", "simt"), ("f32", "auto"), ("f16", "simt"), ("f16", "auto"), ("bf16", "auto")])
def test_conv_other_algebras_vs_oracle(gpu, oracle, name, shape, dtype, engine):
    n, ci, co, h, w_, kh, kw, stride, pad = shape
    alg, code, D = ALGEBRAS[name]
    xs, ws, bs = _shapes(name, n, ci, co, h, w_, kh, kw)
    x = gpu.rounded(uniform(61, xs), dtype)
    w = gpu.rounded(normal(62, ws, std=(2.0 / (D * ci * kh * kw)) ** 0.5), dtype)
    b = gpu.rounded(uniform(63, bs), dtype)
    ox, ow, ob = _oracle_view(name, x, w, b)
    ref = oracle.conv2d_fwd(ox, ow, ob, stride, (1, 1), pad, code, 0)
    got = gpu.run_conv_fwd(x, w, b, stride, pad, dtype, "8p", engine, False, alg)     # the variant is ignored off quaternions
    _check(got, ref, dtype, gpu, "y")
    dy = gpu.rounded(normal(64, ref.shape), dtype)
    rdw, rdx = oracle.conv2d_bwd(ox, ow, dy, stride, (1, 1), pad, code, 0, True)
    dw, dx = gpu.run_conv_bwd(x, w, dy, stride, pad, dtype, "16p", engine, True, alg)
    _check(dx, rdx, dtype, gpu, "dx")
    _check(dw.reshape(rdw.shape), rdw, dtype, gpu, "dw")


@pytest.mark.parametrize("name", ["real", "complex", "ga_300"])
@pytest.mark.parametrize("shape", [(3, 5, 7), (32, 64, 48), (17, 130, 70)])
@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("oi", [False, True])
def test_dense_other_algebras_vs_oracle(gpu, oracle, name, shape, dtype, oi):
    b_, i_, o_ = shape
    alg, code, D = ALGEBRAS[name]
    real = name == "real"
    x = gpu.rounded(uniform(71, (D * b_, i_)), dtype)
    wshape = (o_, i_) if oi else (i_, o_)
    w = gpu.rounded(normal(72, wshape if real else (D,) + wshape, std=(2.0 / (D * i_)) ** 0.5), dtype)
    bias = gpu.rounded(uniform(73, (o_,) if real else (D, o_)), dtype)
    ow, ob = (w[None], bias[None]) if real else (w, bias)
    ref = oracle.dense_fwd(x, ow, ob, oi, code, 0)
    got = gpu.run_dense_fwd(x, w, bias, oi, dtype, "16p", "auto", alg)
    _check(got, ref, dtype, gpu, "y")
    dy = gpu.rounded(normal(74, ref.shape), dtype)
    rdw, rdx = oracle.dense_bwd(x, ow, dy, oi, code, 0, True)
    dw, dx = gpu.run_dense_bwd(x, w, dy, oi, dtype, "16p", "auto", True, alg)
    _check(dx, rdx, dtype, gpu, "dx")
    _check(dw.reshape(rdw.shape), rdw, dtype, gpu, "dw")


@pytest.mark.parametrize("name", ["complex", "quaternion", "ga_300"])
@pytest.mark.parametrize("dtype,engine", [("f32", "simt"), ("f32", "auto"), ("f16", "auto")])
def test_dilated_conv_vs_oracle(gpu, oracle, name, dtype, engine):
    """Dilation 2 (the reference passes it to its scalar convolutions, src/backend/onednn/conv2d.hpp:121)."""
    alg, code, D = ALGEBRAS[name]
    n, ci, co, h, w_, k = 2, 16, 16, 13, 12, 3
    stride, dil, pad = (1, 1), (2, 2), (2, 2, 2, 2)
    x = gpu.rounded(uniform(81, (D * n, ci, h, w_)), dtype)
    w = gpu.rounded(normal(82, (D, co, ci, k, k), std=(2.0 / (D * ci * k * k)) ** 0.5), dtype)
    ref = oracle.conv2d_fwd(x, w, None, stride, dil, pad, code, 0)
    got = gpu.run_conv_fwd(x, w, None, stride, pad, dtype, "16p", engine, False, alg, dil)
    _check(got, ref, dtype, gpu, "y")
    dy = gpu.rounded(normal(84, ref.shape), dtype)
    rdw, rdx = oracle.conv2d_bwd(x, w, dy, stride, dil, pad, code, 0, True)
    dw, dx = gpu.run_conv_bwd(x, w, dy, stride, pad, dtype, "16p", engine, True, alg, dil)
    _check(dx, rdx, dtype, gpu, "dx")
    _check(dw, rdw, dtype, gpu, "dw")


def test_engines_for_other_algebras(gpu):
    """fp32 and 16-bit layers of every algebra reach the tensor-core kernels when the geometry allows."""
    import ctypes
    from phoenix_core_b200 import _lib
    L = _lib.lib()
    for algebra in (0, 1, 2, 3):
        for dtype in (0, 1):
            d = _lib.ConvDesc(dtype=dtype, n=4, ci=32, co=32, h=14, w=14, kh=3, kw=3, stride_h=1, stride_w=1, dilation_h=1,
                              dilation_w=1, pad_top=1, pad_left=1, pad_bottom=1, pad_right=1, groups=1, algebra=algebra)
            for p in (0, 1, 2):
                assert L.pcb_qconv2d_engine_for(ctypes.byref(d), p) == _lib.ENGINE_TENSOR, (algebra, dtype, p)


# ---- tensor layouts (reference: DataFormat / FilterLayout, src/backend/types.hpp:85-97) -------------------------
def _to_layout(a, fmt):
    """NCHW / OIHW numpy array -> the named layout (the component axis, if any, stays leading)."""
    if fmt in ("NCHW", "OIHW"):
        return np.ascontiguousarray(a)
    lead = a.ndim - 4                       # 1 for filters with a component axis, 0 otherwise
    perm = {"NHWC": (0, 2, 3, 1), "OHWI": (0, 2, 3, 1), "HWIO": (2, 3, 1, 0)}[fmt]
    return np.ascontiguousarray(a.transpose(tuple(range(lead)) + tuple(lead + p for p in perm)))


def _from_layout(a, fmt):
    if fmt in ("NCHW", "OIHW"):
        return a
    lead = a.ndim - 4
    inv = {"NHWC": (0, 3, 1, 2), "OHWI": (0, 3, 1, 2), "HWIO": (3, 2, 0, 1)}[fmt]
    return np.ascontiguousarray(a.transpose(tuple(range(lead)) + tuple(lead + p for p in inv)))


def test_reference_layout_kats_on_gpu(gpu):
    """Real channels-last convolutions with OHWI and HWIO filters: the reference's known answers (tests/tests.cpp:438-547)."""
    with open(GOLDEN) as f:
        cases = [c for c in json.load(f)["cases"] if c["op"] == "conv2d_layout"]
    assert len(cases) == 2
    for case in cases:
        x = np.asarray(case["x"], np.float32).reshape(case["x_shape"])
        w = np.asarray(case["w"], np.float32).reshape(case["w_shape"])
        want = np.asarray(case["y"], np.float32).reshape(case["y_shape"])
        got = _run_layout_fwd(gpu, x, w, None, (1, 1), (0, 0, 0, 0), "f32", pcb.Algebra.REAL, case["data_format"], case["filter_layout"])
        assert np.array_equal(got, want), case["name"]


def _descs(xshape, wshape, stride, pad, algebra, data_format, filter_layout, use_bias, need_dx):
    args = (xshape, wshape, stride, (1, 1), pcb.Padding.EXPLICIT, pad, 1, algebra, getattr(pcb.DataFormat, data_format),
            getattr(pcb.FilterLayout, filter_layout))
    return pcb.Conv2DFwdDescriptor(*args, use_bias), pcb.Conv2DBwdDescriptor(*args, need_dx)


def _run_layout_fwd(gpu, x, w, b, stride, pad, dtype, algebra, data_format, filter_layout):
    fwd, _ = _descs(x.shape, w.shape, stride, pad, algebra, data_format, filter_layout, b is not None, False)
    y = torch.full(fwd.getOutputShape(), float("nan"), dtype=gpu.TORCH_DTYPES[dtype], device="cuda")
    pcb.conv2DFwd(gpu.dev(x, dtype), gpu.dev(w, dtype), None if b is None else gpu.dev(b, dtype), y, fwd, gpu.context("16p"))
    return gpu.host(y)


@pytest.mark.parametrize("data_format,filter_layout", [("NHWC", "OHWI"), ("NHWC", "HWIO"), ("NCHW", "HWIO"), ("NHWC", "OIHW")])
@pytest.mark.parametrize("name", ["quaternion", "complex"])
@pytest.mark.parametrize("dtype,variant,engine", [("f32", "16p", "auto"), ("f32", "8p", "auto"), ("f16", "16p", "simt"), ("f16", "16p", "tensor"),
                                                  ("bf16", "16p", "tensor")])
def test_conv_layouts_vs_oracle(gpu, oracle, data_format, filter_layout, name, dtype, variant, engine):
    """The other activation / filter layouts against the oracle (which computes in NCHW / OIHW on permuted copies), on the
    CUDA-core kernels and, for 16-bit tensors, on the tensor cores (every tensor addressed through element strides)."""
    alg, code, D = ALGEBRAS[name]
    n, ci, co, h, w_, kh, kw, stride, pad = 2, 5, 6, 9, 7, 3, 2, (2, 1), (1, 0, 1, 1)
    x = gpu.rounded(uniform(101, (D * n, ci, h, w_)), dtype)
    w = gpu.rounded(normal(102, (D, co, ci, kh, kw), std=0.2), dtype)
    b = gpu.rounded(uniform(103, (D, co)), dtype)
    ref = oracle.conv2d_fwd(x, w, b, stride, (1, 1), pad, code, 0)
    dy = gpu.rounded(normal(104, ref.shape), dtype)
    rdw, rdx = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad, code, 0, True)
    xl, wl, dyl = _to_layout(x, data_format), _to_layout(w, filter_layout), _to_layout(dy, data_format)
    fwd, bwd = _descs(xl.shape, wl.shape, stride, pad, alg, data_format, filter_layout, True, True)
    ctx = gpu.context(variant)
    td = gpu.TORCH_DTYPES[dtype]
    y = torch.full(fwd.getOutputShape(), float("nan"), dtype=td, device="cuda")
    pcb.conv2DFwd(gpu.dev(xl, dtype), gpu.dev(wl, dtype), gpu.dev(b, dtype), y, fwd, ctx, gpu.ENGINES[engine])
    _check(_from_layout(gpu.host(y), data_format), ref, dtype, gpu, "y")
    dw = torch.full(wl.shape, float("nan"), dtype=td, device="cuda")
    dx = torch.full(xl.shape, float("nan"), dtype=td, device="cuda")
    pcb.conv2DBwd(gpu.dev(xl, dtype), gpu.dev(wl, dtype), gpu.dev(dyl, dtype), dw, dx, bwd, ctx, gpu.ENGINES[engine])
    _check(_from_layout(gpu.host(dx), data_format), rdx, dtype, gpu, "dx")
    _check(_from_layout(gpu.host(dw), filter_layout), rdw, dtype, gpu, "dw")


@pytest.mark.parametrize("dtype,variant,engine", [("f32", "16p", "auto"), ("f32", "8p", "auto"), ("f16", "16p", "simt"), ("bf16", "8p", "simt"),
                                                  ("f16", "16p", "tensor"), ("bf16", "16p", "tensor")])
@pytest.mark.parametrize("groups,ci,co", [(2, 6, 4), (4, 4, 8), (8, 8, 8), (2, 64, 96)])      # (8, 8, 8) is depthwise
def test_grouped_conv_vs_oracle(gpu, oracle, dtype, variant, engine, groups, ci, co):
    """Grouped quaternion convolution (reference: the groups argument, src/conv2d.hpp:70-91, :329-353) against the oracle run
    group by group on channel slices: forward with bias, both gradients."""
    n, h, w_, k = 2, 9, 7, 3
    cig, cog = ci // groups, co // groups
    x = gpu.rounded(uniform(71, (4 * n, ci, h, w_)), dtype)
    w = gpu.rounded(uniform(72, (4, co, cig, k, k)), dtype)
    b = gpu.rounded(uniform(73, (4, co)), dtype)
    stride, pad = (2, 1), (1, 1, 1, 1)
    ov = oracle.VARIANT_16P if variant == "16p" else oracle.VARIANT_8P
    ys = [oracle.conv2d_fwd(np.ascontiguousarray(x[:, g * cig:(g + 1) * cig]), np.ascontiguousarray(w[:, g * cog:(g + 1) * cog]),
                            np.ascontiguousarray(b[:, g * cog:(g + 1) * cog]), stride, (1, 1), pad, oracle.QUATERNION, ov) for g in range(groups)]
    ref = np.concatenate(ys, axis=1)
    got = gpu.run_conv_fwd(x, w, b, stride, pad, dtype, variant, engine, groups=groups)
    assert got.shape == ref.shape
    _check(got, ref, dtype, gpu, "y")
    dy = gpu.rounded(normal(74, ref.shape), dtype)
    dws, dxs = [], []
    for g in range(groups):
        dwg, dxg = oracle.conv2d_bwd(np.ascontiguousarray(x[:, g * cig:(g + 1) * cig]), np.ascontiguousarray(w[:, g * cog:(g + 1) * cog]),
                                     np.ascontiguousarray(dy[:, g * cog:(g + 1) * cog]), stride, (1, 1), pad, oracle.QUATERNION, ov, True)
        dws.append(dwg); dxs.append(dxg)
    dw, dx = gpu.run_conv_bwd(x, w, dy, stride, pad, dtype, variant, engine, True, groups=groups)
    _check(dw, np.concatenate(dws, axis=1), dtype, gpu, "dw")
    _check(dx, np.concatenate(dxs, axis=1), dtype, gpu, "dx")


# n, ci, co, h, w, k, stride, pad: channels-last layers whose channel counts are multiples of 16, which the tensor-core kernels
# read in place (no staged copy; the padding is the zero fill of out-of-range TMA coordinates)
DIRECT_SHAPES = [
    (2, 32, 48, 12, 10, 3, (1, 1), (1, 1, 1, 1)),      # plain form, 32-channel slices
    (1, 64, 32, 30, 21, 3, (1, 1), (1, 1, 1, 1)),      # halo form: one tile per image column, negative start coordinates
    (2, 64, 64, 14, 14, 3, (2, 2), (0, 0, 1, 1)),      # stride 2 through the element stride of the tensor map; backward-data staged
    (3, 16, 16, 9, 9, 1, (1, 1), (0, 0, 0, 0)),        # pointwise: a plain GEMM over [pixel][channel] rows
    (2, 128, 64, 8, 8, 5, (1, 1), (2, 2, 2, 2)),       # 25 taps, 64-channel slices
    (2, 96, 96, 20, 12, 3, (1, 1), (1, 1, 1, 1)),      # 96 = 3 x 32 channels: the transposing channels-last epilogue over three row tiles
]


@pytest.mark.parametrize("shape", DIRECT_SHAPES)
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("filter_layout", ["OHWI", "HWIO"])
def test_channels_last_read_in_place_on_tensor_cores(gpu, oracle, shape, dtype, filter_layout):
    n, ci, co, h, w_, k, stride, pad = shape
    x = gpu.rounded(uniform(111, (4 * n, ci, h, w_)), dtype)
    w = gpu.rounded(normal(112, (4, co, ci, k, k), std=(2.0 / (4 * ci * k * k)) ** 0.5), dtype)
    b = gpu.rounded(uniform(113, (4, co)), dtype)
    ref = oracle.conv2d_fwd(x, w, b, stride, (1, 1), pad)
    dy = gpu.rounded(normal(114, ref.shape), dtype)
    rdw, rdx = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad)
    xl, wl, dyl = _to_layout(x, "NHWC"), _to_layout(w, filter_layout), _to_layout(dy, "NHWC")
    fwd, bwd = _descs(xl.shape, wl.shape, stride, pad, pcb.Algebra.QUATERNION, "NHWC", filter_layout, True, True)
    ctx, td = gpu.context("16p"), gpu.TORCH_DTYPES[dtype]
    y = torch.full(fwd.getOutputShape(), float("nan"), dtype=td, device="cuda")
    pcb.conv2DFwd(gpu.dev(xl, dtype), gpu.dev(wl, dtype), gpu.dev(b, dtype), y, fwd, ctx, gpu.ENGINES["tensor"])
    _check(_from_layout(gpu.host(y), "NHWC"), ref, dtype, gpu, "y")
    dw = torch.full(wl.shape, float("nan"), dtype=td, device="cuda")
    dx = torch.full(xl.shape, float("nan"), dtype=td, device="cuda")
    pcb.conv2DBwd(gpu.dev(xl, dtype), gpu.dev(wl, dtype), gpu.dev(dyl, dtype), dw, dx, bwd, ctx, gpu.ENGINES["tensor"])
    _check(_from_layout(gpu.host(dx), "NHWC"), rdx, dtype, gpu, "dx")
    _check(_from_layout(gpu.host(dw), filter_layout), rdw, dtype, gpu, "dw")
