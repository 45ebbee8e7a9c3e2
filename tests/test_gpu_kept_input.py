"""The backward pass that reads the staged copy of x left by the layer's forward call (``pcb_qconv2d_bwd_kept``,
``KeptInput`` in the Python operators): same results as the plain backward pass, proof that the staged copy is what
the filter gradient read, and the fall-backs (another x, a workspace reused since, layers that keep nothing)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util
    return gpu_util


def normal(seed, shape, std=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * std).astype(np.float32)


def rel_err(got, ref):
    return float(np.abs(got - ref).max() / max(float(np.abs(ref).max()), 1e-30))


# n, ci, co, h, w, k, stride, pad, real_input, keeps (whether the forward kernel's staged x serves the filter gradient)
SHAPES = [
    (3, 16, 16, 24, 24, 3, (1, 1), (1, 1, 1, 1), False, True),    # narrow forward + narrow filter gradient
    (2, 3, 16, 40, 40, 7, (2, 2), (2, 2, 3, 3), True, True),      # stem: real-valued input, space-to-depth staging
    (2, 8, 24, 17, 19, 3, (1, 1), (1, 1, 1, 1), False, True),     # narrow pair, ragged planes (general staging form)
    (2, 32, 32, 14, 14, 3, (1, 1), (1, 1, 1, 1), False, True),    # general forward + general filter gradient, 32 channels
    (2, 16, 32, 16, 16, 3, (2, 2), (0, 0, 1, 1), False, True),    # stride 2, 16 channels
    (2, 64, 64, 10, 10, 3, (1, 1), (1, 1, 1, 1), False, True),    # 64 channels: one 128-byte block per component
    (2, 24, 32, 12, 12, 3, (1, 1), (1, 1, 1, 1), False, True),    # 24 channels padded to 32
    (2, 128, 64, 8, 8, 3, (1, 1), (1, 1, 1, 1), False, False),    # two channel blocks per component: layouts differ
    (2, 48, 32, 9, 9, 3, (1, 1), (1, 1, 1, 1), False, False),     # 48 = 3 x 16 channels: blocked layout
    (2, 64, 64, 12, 12, 1, (1, 1), (0, 0, 0, 0), False, False),   # pointwise: nothing is staged
    (2, 16, 64, 16, 16, 3, (1, 1), (1, 1, 1, 1), False, True),    # 16 channels but 4 x 64 output rows: the general pair
]


def _setup(gpu, shape, dtype):
    import torch
    import phoenix_core_b200 as pcb
    n, ci, co, h, w_, k, stride, pad, real_in, keeps = shape
    x = gpu.rounded(normal(11, ((1 if real_in else 4) * n, ci, h, w_)), dtype)
    w = gpu.rounded(normal(12, (4, co, ci, k, k), std=(2.0 / (4 * ci * k * k)) ** 0.5), dtype)
    fwd, _ = gpu.conv_descriptors(x.shape, w.shape, stride, pad, False, False, real_in)
    _, bwd = gpu.conv_descriptors(x.shape, w.shape, stride, pad, False, not real_in, real_in)
    dy = gpu.rounded(normal(13, fwd.getOutputShape(), std=0.25), dtype)
    td = gpu.TORCH_DTYPES[dtype]
    t = {"x": gpu.dev(x, dtype), "w": gpu.dev(w, dtype), "dy": gpu.dev(dy, dtype),
         "y": torch.full(fwd.getOutputShape(), float("nan"), dtype=td, device="cuda"),
         "dw": torch.full(w.shape, float("nan"), dtype=td, device="cuda"),
         "dx": None if real_in else torch.full(x.shape, float("nan"), dtype=td, device="cuda")}
    return x, w, dy, fwd, bwd, t, pcb


def _oracle_bwd(oracle, x, w, dy, shape):
    n, ci, co, h, w_, k, stride, pad, real_in, keeps = shape
    xq = x
    if real_in:
        xq = np.concatenate([x, np.zeros((3 * x.shape[0],) + x.shape[1:], np.float32)], 0)
    dw, dx = oracle.conv2d_bwd(xq, w, dy, stride, (1, 1), pad, oracle.QUATERNION, oracle.VARIANT_16P, not real_in)
    return dw, dx


def _keeps(pcb, gpu, fwd, t, ctx):
    from phoenix_core_b200 import _lib, ops
    d = ops._conv_desc(fwd, t["x"].dtype, ctx, _lib.ENGINE_AUTO)
    return bool(_lib.lib().pcb_qconv2d_fwd_keeps_input(ctypes.byref(d)))


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("shape", SHAPES)
def test_backward_from_the_kept_input_vs_oracle(gpu, oracle, shape, dtype):
    """Forward with a KeptInput, then x is ZEROED in place, then the backward pass: a layer that keeps its staged
    input still produces the filter gradient of the original x (so the staged copy is what was read); a layer that
    keeps nothing sees the zeros. dx never depends on x."""
    x, w, dy, fwd, bwd, t, pcb = _setup(gpu, shape, dtype)
    keeps = shape[-1]
    ctx = gpu.context("16p")
    assert _keeps(pcb, gpu, fwd, t, ctx) == keeps
    rdw, rdx = _oracle_bwd(oracle, x, w, dy, shape)
    kept = pcb.KeptInput()
    pcb.conv2DFwd(t["x"], t["w"], None, t["y"], fwd, ctx, keep=kept)
    assert (kept.workspace is not None) == keeps
    t["x"].zero_()
    pcb.conv2DBwd(t["x"], t["w"], t["dy"], t["dw"], t["dx"], bwd, ctx, kept=kept)
    dw = gpu.host(t["dw"])
    assert np.all(np.isfinite(dw))
    if keeps:
        assert rel_err(dw, rdw) <= gpu.TOL[dtype]
    else:
        assert float(np.abs(dw).max()) == 0.0
    if t["dx"] is not None:
        assert rel_err(gpu.host(t["dx"]), rdx) <= gpu.TOL[dtype]


@pytest.mark.parametrize("shape", [SHAPES[0], SHAPES[1], SHAPES[3], SHAPES[4]])
def test_kept_and_plain_backward_agree(gpu, oracle, shape):
    x, w, dy, fwd, bwd, t, pcb = _setup(gpu, shape, "f16")
    ctx = gpu.context("16p")
    kept = pcb.KeptInput()
    pcb.conv2DFwd(t["x"], t["w"], None, t["y"], fwd, ctx, keep=kept)
    pcb.conv2DBwd(t["x"], t["w"], t["dy"], t["dw"], t["dx"], bwd, ctx, kept=kept)
    dw_kept = gpu.host(t["dw"])
    dx_kept = None if t["dx"] is None else gpu.host(t["dx"])
    t["dw"].fill_(float("nan"))
    pcb.conv2DBwd(t["x"], t["w"], t["dy"], t["dw"], t["dx"], bwd, ctx)
    # the same kernel on the same staged values; only the order of the split-K atomic additions may differ
    assert rel_err(gpu.host(t["dw"]), dw_kept) <= 1e-3
    if dx_kept is not None:
        assert np.array_equal(gpu.host(t["dx"]), dx_kept)


def test_another_input_or_a_reused_workspace_falls_back(gpu, oracle):
    """The record of what a workspace holds is (x address, problem): a backward call with another x, or after another
    forward call wrote to the workspace, stages x itself and is right all the same."""
    shape = SHAPES[3]
    x, w, dy, fwd, bwd, t, pcb = _setup(gpu, shape, "f16")
    ctx = gpu.context("16p")
    rdw, _ = _oracle_bwd(oracle, x, w, dy, shape)
    kept = pcb.KeptInput()
    pcb.conv2DFwd(t["x"], t["w"], None, t["y"], fwd, ctx, keep=kept)
    # (a) another tensor with other values at another address: its own gradient, not the kept one's
    x2 = gpu.rounded(normal(21, x.shape), "f16")
    rdw2, _ = _oracle_bwd(oracle, x2, w, dy, shape)
    pcb.conv2DBwd(gpu.dev(x2, "f16"), t["w"], t["dy"], t["dw"], t["dx"], bwd, ctx, kept=kept)
    assert rel_err(gpu.host(t["dw"]), rdw2) <= gpu.TOL["f16"]
    # (b) the workspace is used by a forward call on another input: the record now names that input
    x3 = gpu.dev(gpu.rounded(normal(22, x.shape), "f16"), "f16")
    pcb.conv2DFwd(x3, t["w"], None, t["y"], fwd, ctx, keep=kept)
    pcb.conv2DBwd(t["x"], t["w"], t["dy"], t["dw"], t["dx"], bwd, ctx, kept=kept)
    assert rel_err(gpu.host(t["dw"]), rdw) <= gpu.TOL["f16"]
    # (c) another call (here the CUDA-core forward pass) is given the workspace, which is then wiped: the record is gone
    from phoenix_core_b200 import _lib, ops
    pcb.conv2DFwd(t["x"], t["w"], None, t["y"], fwd, ctx, keep=kept)
    d = ops._conv_desc(fwd, t["x"].dtype, ctx, _lib.ENGINE_SIMT)
    import torch
    _lib.check(_lib.lib().pcb_qconv2d_fwd(ctypes.byref(d), ops._ptr(t["x"]), ops._ptr(t["w"]), None, ops._ptr(t["y"]),
                                          ops._ptr(kept.workspace), kept.workspace.numel(),
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    kept.workspace.zero_()
    pcb.conv2DBwd(t["x"], t["w"], t["dy"], t["dw"], t["dx"], bwd, ctx, kept=kept)
    assert rel_err(gpu.host(t["dw"]), rdw) <= gpu.TOL["f16"]


def test_fp32_and_simt_keep_nothing(gpu):
    import phoenix_core_b200 as pcb
    from phoenix_core_b200 import _lib, ops
    import torch
    n, ci, co, h, w_ = 2, 32, 32, 14, 14
    fwd, _ = gpu.conv_descriptors((4 * n, ci, h, w_), (4, co, ci, 3, 3), (1, 1), (1, 1, 1, 1), False, False)
    ctx = gpu.context("16p")
    L = _lib.lib()
    assert L.pcb_qconv2d_fwd_keeps_input(ctypes.byref(ops._conv_desc(fwd, torch.float16, ctx, _lib.ENGINE_AUTO))) == 1
    assert L.pcb_qconv2d_fwd_keeps_input(ctypes.byref(ops._conv_desc(fwd, torch.float32, ctx, _lib.ENGINE_AUTO))) == 0
    assert L.pcb_qconv2d_fwd_keeps_input(ctypes.byref(ops._conv_desc(fwd, torch.float16, ctx, _lib.ENGINE_SIMT))) == 0


# ---- dy staged once for both gradients of one backward call -------------------------------------------------
# n, ci, co, h, w, k, dilation, pad
SHARED_DY_SHAPES = [
    (3, 16, 16, 24, 24, 3, 1, (1, 1, 1, 1)),     # narrow pair
    (2, 8, 24, 17, 19, 3, 1, (1, 1, 1, 1)),      # narrow pair, ragged planes, three planes of dy rows
    (2, 16, 8, 20, 16, 3, 1, (0, 0, 0, 0)),      # narrow pair without padding (the copy of dy is padded by two), one plane of dy
    (2, 32, 32, 14, 14, 3, 1, (1, 1, 1, 1)),     # general pair
    (2, 32, 64, 13, 11, 5, 1, (2, 2, 2, 2)),     # general pair, 25 taps, ragged
    (2, 64, 32, 12, 12, 3, 2, (2, 2, 2, 2)),     # dilation 2
    (2, 32, 32, 12, 12, 3, 1, (0, 1, 2, 0)),     # asymmetric padding
    (1, 64, 32, 30, 21, 3, 1, (1, 1, 1, 1)),     # backward-data in halo mode
    (2, 32, 48, 9, 9, 3, 1, (1, 1, 1, 1)),       # 48 = 3 x 16 output channels: blocked dy, nothing shared
    (2, 32, 32, 14, 14, 3, 1, (1, 1, 1, 1)),     # (again, for bf16 below)
]


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("shape", SHARED_DY_SHAPES[:-1])
def test_backward_call_with_one_staged_dy_vs_oracle_and_vs_the_separate_passes(gpu, oracle, shape, dtype):
    """pcb_qconv2d_bwd stages dy once (backward-data's padded copy, read by the filter gradient through a tensor map)
    where the two kernels agree on the layout; the separate entry points stage it twice. Both against the oracle, and
    against each other (dx bit for bit)."""
    import torch
    import phoenix_core_b200 as pcb
    n, ci, co, h, w_, k, dil, pad = shape
    x = gpu.rounded(normal(31, (4 * n, ci, h, w_)), dtype)
    w = gpu.rounded(normal(32, (4, co, ci, k, k), std=(2.0 / (4 * ci * k * k)) ** 0.5), dtype)
    _, bwd = gpu.conv_descriptors(x.shape, w.shape, (1, 1), pad, False, True, dilation=(dil, dil))
    fwd, _ = gpu.conv_descriptors(x.shape, w.shape, (1, 1), pad, False, False, dilation=(dil, dil))
    dy = gpu.rounded(normal(33, fwd.getOutputShape(), std=0.25), dtype)
    rdw, rdx = oracle.conv2d_bwd(x, w, dy, (1, 1), (dil, dil), pad)
    ctx, td = gpu.context("16p"), gpu.TORCH_DTYPES[dtype]
    xd, wd, gd = gpu.dev(x, dtype), gpu.dev(w, dtype), gpu.dev(dy, dtype)
    out = {}
    for mode in ("one call", "separate passes"):
        dw = torch.full(w.shape, float("nan"), dtype=td, device="cuda")
        dx = torch.full(x.shape, float("nan"), dtype=td, device="cuda")
        pcb.conv2DBwd(xd, wd, gd, dw, dx, bwd, ctx, on_filter_grad=(None if mode == "one call" else (lambda t: None)))
        out[mode] = (gpu.host(dw), gpu.host(dx))
        assert np.all(np.isfinite(out[mode][0])) and np.all(np.isfinite(out[mode][1])), mode
        assert rel_err(out[mode][0], rdw) <= gpu.TOL[dtype], mode
        assert rel_err(out[mode][1], rdx) <= gpu.TOL[dtype], mode
    assert np.array_equal(out["one call"][1], out["separate passes"][1])
    # same kernel, same staged values; the split-K atomic additions may land in another order, which can move a result by
    # one unit in the last place of the storage type
    assert rel_err(out["one call"][0], out["separate passes"][0]) <= (2e-3 if dtype == "f16" else 1e-2)
