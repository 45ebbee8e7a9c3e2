"""The reference's own composition code as the yardstick. ``golden/reference_composition.npz`` holds inputs and outputs
of the reference's four operations -- forward AND backward, both quaternion formulations, the other algebras, the
layouts, groups, real-valued input, dense -- produced by the reference's sources themselves (see
``golden/make_reference_composition.py``). Checked here:

* the CPU oracle reproduces every vector (not gpu);
* where a reference checkout is present, a fresh run of the reference reproduces the committed file (not gpu);
* the CUDA path, through the public operators, reproduces every vector in fp32, and in fp16 / bf16 on the tensor cores
  (inputs are exact in every storage type) (gpu).
"""
import importlib.util
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_reference_composition", os.path.join(HERE, "golden", "make_reference_composition.py"))
cases = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(cases)

CONV = {c[0]: c for c in cases.CONV_CASES}
DENSE = {c[0]: c for c in cases.DENSE_CASES}
FORMS = ["8p", "16p"]


@pytest.fixture(scope="module")
def golden():
    return np.load(os.path.join(HERE, "golden", "reference_composition.npz"))


def _rel(got, ref):
    return float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max() / max(float(np.abs(ref).max()), 1e-30))


def _get(golden, key):
    return golden[key] if key in golden.files else None


def _oracle_conv(oracle, case, form, x, w, b, dy):
    """The oracle on a golden case: NCHW / OIHW, groups as channel slices, the real algebra with a leading axis of 1."""
    _, alg, n, ci, co, h, w_, kh, kw, stride, dil, padding, bias, df, fl, groups, real_in = case
    from oracle import reference_lib as ref
    pad = ref.padding_of(padding, h, w_, kh, kw, stride, dil)
    variant = oracle.VARIANT_8P if (form == "8p" and alg == cases.QUATERNION) else oracle.VARIANT_16P
    lead = alg != cases.REAL
    wq = w if lead else w[None]
    bq = None if b is None else (b if lead else b[None])
    cig, cog = ci // groups, co // groups
    ys, dws, dxs = [], [], []
    for g in range(groups):
        xg = np.ascontiguousarray(x[:, g * cig:(g + 1) * cig])
        wg = np.ascontiguousarray(wq[:, g * cog:(g + 1) * cog])
        bg = None if bq is None else np.ascontiguousarray(bq[:, g * cog:(g + 1) * cog])
        ys.append(oracle.conv2d_fwd(xg, wg, bg, stride, dil, pad, alg, variant, real_in))
    y = np.concatenate(ys, axis=1)
    for g in range(groups):
        xg = np.ascontiguousarray(x[:, g * cig:(g + 1) * cig])
        if real_in:      # a real input is the multivector input with zero non-real parts
            xg = np.concatenate([xg, np.zeros(((cases.DIMS[alg] - 1) * xg.shape[0],) + xg.shape[1:], np.float32)], 0)
        wg = np.ascontiguousarray(wq[:, g * cog:(g + 1) * cog])
        dyg = np.ascontiguousarray(dy[:, g * cog:(g + 1) * cog])
        dwg, dxg = oracle.conv2d_bwd(xg, wg, dyg, stride, dil, pad, alg, variant, not real_in)
        dws.append(dwg)
        dxs.append(dxg)
    dw = np.concatenate(dws, axis=1)
    dx = None if real_in else np.concatenate(dxs, axis=1)
    return y, (dw if lead else dw[0]), dx


@pytest.mark.parametrize("form", FORMS)
@pytest.mark.parametrize("name", list(CONV))
def test_oracle_reproduces_the_reference_conv(oracle, golden, name, form):
    x, w, b, dy = golden[name + "/x"], golden[name + "/w"], _get(golden, name + "/b"), golden[name + "/dy"]
    y, dw, dx = _oracle_conv(oracle, CONV[name], form, x, w, b, dy)
    tag = name + "/" + form
    assert _rel(y, golden[tag + "/y"]) <= 1e-6
    assert _rel(dw, golden[tag + "/dw"]) <= 1e-6
    if dx is not None:
        assert _rel(dx, golden[tag + "/dx"]) <= 1e-6


@pytest.mark.parametrize("form", FORMS)
@pytest.mark.parametrize("name", list(DENSE))
def test_oracle_reproduces_the_reference_dense(oracle, golden, name, form):
    _, alg, bsz, i, o, oi, bias = DENSE[name]
    x, w, b, dy = golden[name + "/x"], golden[name + "/w"], _get(golden, name + "/b"), golden[name + "/dy"]
    variant = oracle.VARIANT_8P if (form == "8p" and alg == cases.QUATERNION) else oracle.VARIANT_16P
    lead = alg != cases.REAL
    wq, bq = (w if lead else w[None]), (None if b is None else (b if lead else b[None]))
    y = oracle.dense_fwd(x, wq, bq, oi, alg, variant)
    dw, dx = oracle.dense_bwd(x, wq, dy, oi, alg, variant, True)
    tag = name + "/" + form
    assert _rel(y, golden[tag + "/y"]) <= 1e-6
    assert _rel(dw if lead else dw[0], golden[tag + "/dw"]) <= 1e-6
    assert _rel(dx, golden[tag + "/dx"]) <= 1e-6


def test_a_fresh_run_of_the_reference_reproduces_the_committed_vectors(golden):
    from oracle import reference_lib as ref
    if not os.path.isdir(os.path.join(ref._default_reference(), "src")):
        pytest.skip("no reference checkout on this machine")
    for name in ("q_3x3_same_bias", "q_nhwc_hwio", "q_groups2", "ga300_3x3"):
        _, alg, n, ci, co, h, w_, kh, kw, stride, dil, padding, bias, df, fl, groups, real_in = CONV[name]
        lead = 0 if alg == cases.REAL else 1
        x, w, b, dy = golden[name + "/x"], golden[name + "/w"], _get(golden, name + "/b"), golden[name + "/dy"]
        xl, wl, dyl = cases.to_layout(x, df, 0), cases.to_layout(w, fl, lead), cases.to_layout(dy, df, 0)
        for mo, form in ((False, "8p"), (True, "16p")):
            y = cases.from_layout(ref.conv2d_fwd(xl, wl, b, stride, dil, padding, alg, mo, real_in, df, fl, groups), df, 0)
            dw, dx = ref.conv2d_bwd(xl, wl, dyl, stride, dil, padding, alg, mo, True, real_in, df, fl, groups)
            assert np.array_equal(y, golden[name + "/" + form + "/y"])
            assert np.array_equal(cases.from_layout(dw, fl, lead), golden[name + "/" + form + "/dw"])
            assert np.array_equal(cases.from_layout(dx, df, 0), golden[name + "/" + form + "/dx"])


# ------------------------------------------------------------------------------------------------ CUDA path
GPU_RUNS = [("f32", "auto"), ("f32", "simt"), ("f16", "auto"), ("f16", "tensor"), ("bf16", "tensor")]


@pytest.fixture(scope="module")
def gpu():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util
    return gpu_util


def _tol(gpu, dtype):
    return gpu.TOL[dtype]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,engine", GPU_RUNS)
@pytest.mark.parametrize("form", FORMS)
@pytest.mark.parametrize("name", list(CONV))
def test_cuda_path_reproduces_the_reference_conv(gpu, golden, name, form, dtype, engine):
    import torch
    import phoenix_core_b200 as pcb
    from phoenix_core_b200 import _lib
    _, alg, n, ci, co, h, w_, kh, kw, stride, dil, padding, bias, df, fl, groups, real_in = CONV[name]
    algebra = [pcb.Algebra.REAL, pcb.Algebra.COMPLEX, pcb.Algebra.QUATERNION, pcb.Algebra.GA_300][alg]
    lead = 0 if alg == cases.REAL else 1
    x, w, b, dy = golden[name + "/x"], golden[name + "/w"], _get(golden, name + "/b"), golden[name + "/dy"]
    xl, wl, dyl = cases.to_layout(x, df, 0), cases.to_layout(w, fl, lead), cases.to_layout(dy, df, 0)
    args = (xl.shape, wl.shape, stride, dil, getattr(pcb.Padding, padding), (), groups, algebra, getattr(pcb.DataFormat, df),
            getattr(pcb.FilterLayout, fl))
    fwd = pcb.Conv2DFwdDescriptor(*args, b is not None, real_in)
    bwd = pcb.Conv2DBwdDescriptor(*args, not real_in, real_in)
    ctx, eng, td = gpu.context(form), gpu.ENGINES[engine], gpu.TORCH_DTYPES[dtype]
    y = torch.full(fwd.getOutputShape(), float("nan"), dtype=td, device="cuda")
    dw = torch.full(wl.shape, float("nan"), dtype=td, device="cuda")
    dx = None if real_in else torch.full(xl.shape, float("nan"), dtype=td, device="cuda")
    try:
        pcb.conv2DFwd(gpu.dev(xl, dtype), gpu.dev(wl, dtype), None if b is None else gpu.dev(b, dtype), y, fwd, ctx, eng)
        pcb.conv2DBwd(gpu.dev(xl, dtype), gpu.dev(wl, dtype), gpu.dev(dyl, dtype), dw, dx, bwd, ctx, eng)
    except _lib.BackendError as err:
        if engine == "tensor" and err.status == _lib.PCB_ERR_UNSUPPORTED:
            pytest.skip("no tensor-core kernel takes this configuration")
        raise
    tag = name + "/" + form
    assert _rel(cases.from_layout(gpu.host(y), df, 0), golden[tag + "/y"]) <= _tol(gpu, dtype)
    assert _rel(cases.from_layout(gpu.host(dw), fl, lead), golden[tag + "/dw"]) <= _tol(gpu, dtype)
    if dx is not None:
        assert _rel(cases.from_layout(gpu.host(dx), df, 0), golden[tag + "/dx"]) <= _tol(gpu, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,engine", GPU_RUNS)
@pytest.mark.parametrize("form", FORMS)
@pytest.mark.parametrize("name", list(DENSE))
def test_cuda_path_reproduces_the_reference_dense(gpu, golden, name, form, dtype, engine):
    import phoenix_core_b200 as pcb
    from phoenix_core_b200 import _lib
    _, alg, bsz, i, o, oi, bias = DENSE[name]
    algebra = [pcb.Algebra.REAL, pcb.Algebra.COMPLEX, pcb.Algebra.QUATERNION, pcb.Algebra.GA_300][alg]
    x, w, b, dy = golden[name + "/x"], golden[name + "/w"], _get(golden, name + "/b"), golden[name + "/dy"]
    tag = name + "/" + form
    try:
        y = gpu.run_dense_fwd(x, w, b, oi, dtype, form, engine, algebra)
        dw, dx = gpu.run_dense_bwd(x, w, dy, oi, dtype, form, engine, True, algebra)
    except _lib.BackendError as err:
        if engine == "tensor" and err.status == _lib.PCB_ERR_UNSUPPORTED:
            pytest.skip("no tensor-core kernel takes this configuration")
        raise
    assert _rel(y, golden[tag + "/y"]) <= _tol(gpu, dtype)
    assert _rel(dw, golden[tag + "/dw"]) <= _tol(gpu, dtype)
    assert _rel(dx, golden[tag + "/dx"]) <= _tol(gpu, dtype)
