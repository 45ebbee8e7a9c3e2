"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle on identical seeded inputs.

Tolerances (max|got-ref| / max|ref| per output tensor): 1e-5 for fp32, 2e-2 for fp16 / bf16, the oracle
running in fp32 on inputs already rounded to the storage type.
"""
import json
import os

import numpy as np
import pytest
import torch

from helpers import normal, rel_err, uniform

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")

# (formulation, engine): under the automatic engine the 8-product request is a speed preference (tensor-core kernels where
# they exist, the factorised CUDA-core kernels elsewhere); the CUDA-core engine runs the factorised kernels always
FORMULATIONS = [("16p", "auto"), ("8p", "auto"), ("8p", "simt")]

# n, ci, co, h, w, kh, kw, stride, pad(t,l,b,r)
CONV_SHAPES = [
    (2, 3, 5, 7, 6, 3, 3, (1, 1), (1, 1, 1, 1)),
    (1, 4, 2, 9, 8, 3, 3, (2, 2), (0, 0, 1, 1)),         # asymmetric SAME-style padding, stride 2
    (3, 2, 3, 5, 5, 1, 1, (1, 1), (0, 0, 0, 0)),
    (2, 2, 4, 8, 7, 1, 1, (2, 2), (0, 0, 0, 0)),         # 1x1 stride 2
    (1, 3, 2, 10, 9, 5, 3, (2, 1), (2, 1, 2, 1)),        # ragged everything
    (2, 16, 16, 16, 16, 3, 3, (1, 1), (1, 1, 1, 1)),     # reduced copy of the 16->16 3x3 configuration
    (1, 3, 16, 20, 20, 7, 7, (2, 2), (2, 2, 3, 3)),      # stem-like 7x7 stride 2 with TF SAME padding
    (2, 40, 24, 6, 5, 1, 1, (1, 1), (0, 0, 0, 0)),
]


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


def test_reference_kats_on_gpu(gpu, oracle):
    """The reference's own quaternion known-answer vectors (tests/tests.cpp:292-369), exact."""
    with open(GOLDEN) as f:
        cases = [c for c in json.load(f)["cases"] if c["op"] == "conv2d_fwd" and c["algebra"] == "quaternion"]
    for case in cases:
        x = (np.full(case["x_shape"], case["x_fill"], np.float32) if "x_fill" in case
             else np.asarray(case["x"], np.float32).reshape(case["x_shape"]))
        w = (np.full(case["w_shape"], case["w_fill"], np.float32) if "w_fill" in case
             else np.asarray(case["w"], np.float32).reshape(case["w_shape"]))
        want = np.asarray(case["y"], np.float32).reshape(case["y_shape"])
        variants = ["16p"] if case["real_input"] else ["16p", "8p"]
        for variant in variants:
            got = gpu.run_conv_fwd(x, w, None, tuple(case["stride"]), (0, 0, 0, 0), "f32", variant, "auto",
                                   case["real_input"])
            assert np.array_equal(got, want), (case["name"], variant)


@pytest.mark.parametrize("shape", CONV_SHAPES)
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("variant,engine", FORMULATIONS)
def test_conv_fwd_bwd_vs_oracle(gpu, oracle, shape, dtype, variant, engine):
    n, ci, co, h, w_, kh, kw, stride, pad = shape
    x = gpu.rounded(uniform(1, (4 * n, ci, h, w_)), dtype)
    w = gpu.rounded(uniform(2, (4, co, ci, kh, kw)), dtype)
    b = gpu.rounded(uniform(3, (4, co)), dtype)
    ov = oracle.VARIANT_16P if variant == "16p" else oracle.VARIANT_8P
    ref = oracle.conv2d_fwd(x, w, b, stride, (1, 1), pad, oracle.QUATERNION, ov)
    got = gpu.run_conv_fwd(x, w, b, stride, pad, dtype, variant, engine)
    _check(got, ref, dtype, gpu, "y")
    nob = gpu.run_conv_fwd(x, w, None, stride, pad, dtype, variant, engine)
    _check(nob, oracle.conv2d_fwd(x, w, None, stride, (1, 1), pad, oracle.QUATERNION, ov), dtype, gpu, "y (no bias)")

    dy = gpu.rounded(normal(4, ref.shape), dtype)
    rdw, rdx = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad, oracle.QUATERNION, ov, True)
    dw, dx = gpu.run_conv_bwd(x, w, dy, stride, pad, dtype, variant, engine, True)
    _check(dw, rdw, dtype, gpu, "dw")
    _check(dx, rdx, dtype, gpu, "dx")
    dw2, none = gpu.run_conv_bwd(x, w, dy, stride, pad, dtype, variant, engine, False)
    assert none is None
    _check(dw2, rdw, dtype, gpu, "dw (no input gradient)")


# pointwise shapes the tensor-core (tcgen05) kernels take: n, ci, co, h, w
TENSOR_SHAPES = [
    (1, 16, 32, 8, 8),        # one tile, K = 64: a single pipeline stage
    (2, 32, 32, 8, 16),       # N = 256: two column tiles
    (3, 24, 40, 4, 6),        # ragged M (160), N (72) and K (96) tiles; chunks cross no image boundary
    (2, 128, 64, 16, 8),      # K = 512: the ring wraps around (8 iterations over 3 stages)
    (1, 64, 256, 12, 12),     # M = 1024: eight row tiles
    (4, 8, 8, 4, 2),          # the smallest legal sizes
    # wide layers: the persistent TMA-fed kernel (four accumulators, sign by negate flag)
    (1, 32, 128, 8, 8),       # one K stage, one tile
    (2, 128, 256, 8, 16),     # K = 128: the stage ring wraps; two channel tiles
    (3, 40, 160, 4, 6),       # ragged: partial K stage, partial channel tile, 24-pixel images (partial TMA boxes)
    (1, 136, 96, 12, 12),     # backward-data with 136 output rows per component (partial second tile)
    (5, 96, 128, 10, 8),      # odd number of 64-pixel blocks per image and in total
]


@pytest.mark.parametrize("shape", TENSOR_SHAPES)
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_pointwise_tensor_core_vs_oracle(gpu, oracle, shape, dtype):
    from phoenix_core_b200 import _lib
    n, ci, co, h, w_ = shape
    x = gpu.rounded(normal(11, (4 * n, ci, h, w_)), dtype)
    w = gpu.rounded(normal(12, (4, co, ci, 1, 1), std=(2.0 / (4 * ci)) ** 0.5), dtype)
    b = gpu.rounded(uniform(13, (4, co)), dtype)
    pad, stride = (0, 0, 0, 0), (1, 1)
    ref = oracle.conv2d_fwd(x, w, b, stride, (1, 1), pad)
    got = gpu.run_conv_fwd(x, w, b, stride, pad, dtype, "16p", "tensor")
    _check(got, ref, dtype, gpu, "y")
    dy = gpu.rounded(normal(14, ref.shape), dtype)
    rdw, rdx = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad)
    dw, dx = gpu.run_conv_bwd(x, w, dy, stride, pad, dtype, "16p", "tensor", True)
    _check(dx, rdx, dtype, gpu, "dx")
    _check(dw, rdw, dtype, gpu, "dw")
    # and the two kernel families agree with each other far inside the tolerance
    simt = gpu.run_conv_fwd(x, w, b, stride, pad, dtype, "16p", "simt")
    assert rel_err(got, simt) <= (4e-3 if dtype == "f16" else 2e-2)


@pytest.mark.parametrize("shape", TENSOR_SHAPES)
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_pointwise_8_product_on_tensor_cores_vs_oracle(gpu, oracle, shape, dtype):
    """The factorised form on its own tcgen05 kernels (lane sums in shared memory, recombination in the epilogue)
    against the oracle's restatement of the reference's 8-product path, all three passes."""
    n, ci, co, h, w_ = shape
    x = gpu.rounded(normal(15, (4 * n, ci, h, w_)), dtype)
    w = gpu.rounded(normal(16, (4, co, ci, 1, 1), std=(2.0 / (4 * ci)) ** 0.5), dtype)
    b = gpu.rounded(uniform(17, (4, co)), dtype)
    pad, stride = (0, 0, 0, 0), (1, 1)
    ref = oracle.conv2d_fwd(x, w, b, stride, (1, 1), pad, oracle.QUATERNION, oracle.VARIANT_8P)
    got = gpu.run_conv_fwd(x, w, b, stride, pad, dtype, "8p", "tensor")
    _check(got, ref, dtype, gpu, "y")
    dy = gpu.rounded(normal(18, ref.shape), dtype)
    rdw, rdx = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad, oracle.QUATERNION, oracle.VARIANT_8P, True)
    dw, dx = gpu.run_conv_bwd(x, w, dy, stride, pad, dtype, "8p", "tensor", True)
    _check(dx, rdx, dtype, gpu, "dx")
    _check(dw, rdw, dtype, gpu, "dw")


# wide pointwise layers with a multiple of 256 output channels and >= 96 input channels: forward on pairs of SMs
# (cta_group::2 MMAs, 256 x 128 tiles): n, ci, co, h, w
PAIR_SHAPES = [
    (8, 128, 256, 56, 56),      # the benchmark layer at batch 8: several tiles per pair, image boundaries inside tiles
    (10, 104, 512, 28, 36),     # two channel pairs, ragged last K slice (104 = 3 x 32 + 8), 1008-pixel images (partial last block)
    (3, 96, 256, 56, 57),       # odd number of 64-pixel blocks in total: the last tile's second half is out of range
    (8, 64, 256, 40, 40),       # two K slices per tile: half of the activation ring per tile, tiles alternate ring halves
]


@pytest.mark.parametrize("shape", PAIR_SHAPES)
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_pointwise_forward_on_sm_pairs_vs_oracle(gpu, oracle, shape, dtype):
    import ctypes
    from phoenix_core_b200 import _lib
    n, ci, co, h, w_ = shape
    x = gpu.rounded(normal(21, (4 * n, ci, h, w_)), dtype)
    w = gpu.rounded(normal(22, (4, co, ci, 1, 1), std=(2.0 / (4 * ci)) ** 0.5), dtype)
    b = gpu.rounded(uniform(23, (4, co)), dtype)
    ref = oracle.conv2d_fwd(x, w, b)
    got = gpu.run_conv_fwd(x, w, b, (1, 1), (0, 0, 0, 0), dtype, "16p", "tensor")
    _check(got, ref, dtype, gpu, "y")
    nob = gpu.run_conv_fwd(x, w, None, (1, 1), (0, 0, 0, 0), dtype, "16p", "tensor")
    _check(nob, oracle.conv2d_fwd(x, w, None), dtype, gpu, "y (no bias)")


# the filter gradient of such layers on pairs of SMs (256 x 128 blocks, K split over the pairs) and backward-data beside it
PAIR_FILTER_SHAPES = PAIR_SHAPES + [
    (6, 200, 256, 40, 40),      # two input-channel tiles, the second ragged (200 = 128 + 72: rows past the end read as zeros)
    (12, 64, 512, 28, 28),      # two output-channel pairs, one 64-row half of the x tile out of range in the odd CTA
]


@pytest.mark.parametrize("shape", PAIR_FILTER_SHAPES)
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_pointwise_backward_on_sm_pairs_vs_oracle(gpu, oracle, shape, dtype):
    n, ci, co, h, w_ = shape
    x = gpu.rounded(normal(31, (4 * n, ci, h, w_)), dtype)
    w = gpu.rounded(normal(32, (4, co, ci, 1, 1), std=(2.0 / (4 * ci)) ** 0.5), dtype)
    dy = gpu.rounded(normal(33, (4 * n, co, h, w_), std=0.25), dtype)
    rdw, rdx = oracle.conv2d_bwd(x, w, dy)
    dw, dx = gpu.run_conv_bwd(x, w, dy, (1, 1), (0, 0, 0, 0), dtype, "16p", "tensor", True)
    _check(dx, rdx, dtype, gpu, "dx")
    _check(dw, rdw, dtype, gpu, "dw")


def test_sm_margin_leaves_results_unchanged(gpu, oracle):
    """With SMs held back for a collective's kernel the persistent kernels run on smaller grids (73 pairs / 146 CTAs on a B200);
    the results are the same."""
    import phoenix_core_b200 as pcb
    n, ci, co, h, w_ = 8, 128, 256, 56, 56
    x = gpu.rounded(normal(51, (4 * n, ci, h, w_)), "f16")
    w = gpu.rounded(normal(52, (4, co, ci, 1, 1), std=(2.0 / (4 * ci)) ** 0.5), "f16")
    dy = gpu.rounded(normal(53, (4 * n, co, h, w_), std=0.25), "f16")
    ref = oracle.conv2d_fwd(x, w, None)
    rdw, rdx = oracle.conv2d_bwd(x, w, dy)
    assert pcb.getSmMargin() == 0
    try:
        for margin in (2, 5):
            pcb.setSmMargin(margin)
            assert pcb.getSmMargin() == margin
            _check(gpu.run_conv_fwd(x, w, None, (1, 1), (0, 0, 0, 0), "f16", "16p", "tensor"), ref, "f16", gpu, "y")
            dw, dx = gpu.run_conv_bwd(x, w, dy, (1, 1), (0, 0, 0, 0), "f16", "16p", "tensor", True)
            _check(dx, rdx, "f16", gpu, "dx")
            _check(dw, rdw, "f16", gpu, "dw")
    finally:
        pcb.setSmMargin(0)


# shapes for the general implicit-GEMM tensor-core kernel (staged channels-last activations, expanded filters):
# n, ci, co, h, w, kh, kw, stride, pad(t,l,b,r)
GENERAL_TENSOR_SHAPES = [
    (2, 16, 16, 14, 14, 3, 3, (1, 1), (1, 1, 1, 1)),     # 16-channel K slices (32-byte swizzle), M = 64 padded to 128
    (2, 32, 64, 14, 14, 3, 3, (2, 2), (0, 0, 1, 1)),     # stride 2 through the tensor map's element stride; M = 256
    (1, 3, 16, 32, 32, 7, 7, (2, 2), (2, 2, 3, 3)),      # stem: 3 channels padded to 16, 49 taps
    (3, 64, 32, 7, 7, 3, 3, (1, 1), (1, 1, 1, 1)),       # 7x7 images: tile box spans images
    (2, 16, 32, 28, 28, 1, 1, (2, 2), (0, 0, 0, 0)),     # 1x1 stride 2 (downsample branch)
    (2, 24, 16, 6, 5, 1, 1, (1, 1), (0, 0, 0, 0)),       # narrow pointwise layer with unaligned planes
    (1, 48, 40, 9, 11, 3, 2, (1, 2), (1, 0, 1, 1)),      # ragged everything, mixed strides, 48 = 3 x 16 channels
    (5, 32, 32, 28, 28, 3, 3, (1, 1), (1, 1, 1, 1)),     # several tiles per CTA: both accumulator buffers in use
    (2, 128, 64, 8, 8, 3, 3, (1, 1), (1, 1, 1, 1)),      # filter gradient with two channel blocks per component (N = 512: two tiles)
    (2, 64, 128, 10, 6, 3, 3, (2, 2), (1, 1, 1, 1)),     # strided backward-data by zero insertion; M = 512
    (1, 64, 32, 30, 21, 3, 3, (1, 1), (1, 1, 1, 1)),     # halo mode: ragged 30 x 21 plane, two 32-channel slices
    (2, 32, 48, 56, 24, 5, 5, (1, 1), (2, 2, 2, 2)),     # halo mode: 25 taps (two stages fit), two tiles per column, M = 192
    (1, 32, 32, 26, 26, 3, 3, (2, 2), (0, 0, 1, 1)),     # halo mode in backward-data only (zero-inserted 26 x 26 plane)
    (2, 64, 32, 16, 16, 1, 1, (2, 2), (0, 0, 0, 0)),     # strided 1x1 on a compact copy (8-pixel vectors), then the direct pointwise kernels
    (1, 96, 160, 9, 9, 3, 3, (1, 1), (1, 1, 1, 1)),      # tiled filter packing with partial 64-column tiles on both sides (96 and 160 channels)
    (1, 72, 64, 9, 9, 3, 3, (1, 1), (1, 1, 1, 1)),       # tiled filter packing with K-side channels padded (72 -> 80): zero columns
    (1, 40, 32, 9, 9, 1, 1, (1, 1), (0, 0, 0, 0)),       # one tap: 32- and 64-element runs in the tiled filter packing
    (1, 24, 40, 9, 7, 1, 1, (2, 3), (1, 1, 0, 1)),       # strided 1x1 with padding, stride 3 across, odd planes (scalar copies)
    (2, 32, 32, 12, 12, 1, 1, (2, 2), (0, 0, 0, 0)),     # strided 1x1: 6 x 6 compact planes (4-pixel vectors), staged general kernel
    (5, 32, 128, 7, 7, 1, 1, (1, 1), (0, 0, 0, 0)),      # whole 7 x 7 planes per tile (4 images, the last tile ragged): bulk-copy epilogue
    (2, 128, 256, 14, 14, 1, 1, (1, 1), (0, 0, 0, 0)),   # whole 14 x 14 planes, 64-channel K slices with three stages, both directions
    (3, 128, 128, 14, 14, 3, 3, (2, 2), (1, 1, 1, 1)),   # bulk-copy epilogue behind a 3x3 stride-2 layer (7 x 7 output planes); backward-data by stride classes
    (2, 128, 64, 10, 12, 3, 3, (2, 2), (0, 0, 1, 1)),    # stride classes with SAME-style padding (first tap of a class at 0 or 1)
    (1, 128, 32, 9, 11, 3, 2, (1, 2), (1, 0, 1, 1)),     # stride classes along one axis only, odd planes (scalar interleave)
    (1, 128, 16, 9, 9, 5, 5, (2, 2), (2, 2, 2, 2)),      # stride classes of a 5x5 layer: 3x3, 3x2, 2x3 and 2x2 taps
]


@pytest.mark.parametrize("shape", GENERAL_TENSOR_SHAPES)
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_general_conv_tensor_core_vs_oracle(gpu, oracle, shape, dtype):
    n, ci, co, h, w_, kh, kw, stride, pad = shape
    x = gpu.rounded(uniform(41, (4 * n, ci, h, w_)), dtype)
    w = gpu.rounded(normal(42, (4, co, ci, kh, kw), std=(2.0 / (4 * ci * kh * kw)) ** 0.5), dtype)
    b = gpu.rounded(uniform(43, (4, co)), dtype)
    ref = oracle.conv2d_fwd(x, w, b, stride, (1, 1), pad)
    got = gpu.run_conv_fwd(x, w, b, stride, pad, dtype, "16p", "tensor")
    _check(got, ref, dtype, gpu, "y")
    dy = gpu.rounded(normal(44, ref.shape), dtype)
    rdw, rdx = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad)
    dw, dx = gpu.run_conv_bwd(x, w, dy, stride, pad, dtype, "16p", "tensor", True)
    _check(dx, rdx, dtype, gpu, "dx")
    _check(dw, rdw, dtype, gpu, "dw")


# shapes for the narrow-layer kernels (<= 16 reduced channels; halo tiles in shared memory serve every tap):
# n, ci, co, h, w, kh, kw, stride, pad(t,l,b,r), dilation
NARROW_SHAPES = [
    (2, 16, 16, 56, 56, 3, 3, (1, 1), (1, 1, 1, 1), (1, 1)),     # the 16-channel stage: two 8 x 28 tiles per column
    (3, 16, 32, 19, 13, 3, 3, (1, 1), (1, 1, 1, 1), (1, 1)),     # ragged plane, all 128 rows in use
    (2, 12, 24, 20, 17, 5, 5, (1, 1), (2, 2, 2, 2), (1, 1)),     # 25 taps (weights fill the shared memory), 3 planes of dy
    (2, 16, 8, 18, 22, 3, 3, (1, 1), (2, 2, 2, 2), (2, 2)),      # dilation 2: a 12 x .. halo tile
    (2, 9, 16, 40, 12, 1, 3, (1, 1), (0, 1, 0, 1), (1, 1)),      # 1 x 3 filter, 40 rows = two tiles of 20
    (2, 32, 16, 17, 15, 3, 3, (2, 2), (1, 1, 1, 1), (1, 1)),     # backward-data of a stride-2 layer: zero insertion, 16 reduced channels
    (2, 2, 16, 24, 20, 3, 3, (2, 2), (0, 0, 1, 1), (1, 1)),      # stride 2 with 2 channels: space-to-depth, four components
    (1, 4, 8, 33, 31, 5, 5, (2, 2), (1, 1, 2, 2), (1, 1)),       # space-to-depth with an odd 5 x 5 filter
]


@pytest.mark.parametrize("shape", NARROW_SHAPES)
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_narrow_layers_tensor_core_vs_oracle(gpu, oracle, shape, dtype):
    n, ci, co, h, w_, kh, kw, stride, pad, dil = shape
    x = gpu.rounded(uniform(91, (4 * n, ci, h, w_)), dtype)
    w = gpu.rounded(normal(92, (4, co, ci, kh, kw), std=(2.0 / (4 * ci * kh * kw)) ** 0.5), dtype)
    b = gpu.rounded(uniform(93, (4, co)), dtype)
    ref = oracle.conv2d_fwd(x, w, b, stride, dil, pad)
    got = gpu.run_conv_fwd(x, w, b, stride, pad, dtype, "16p", "tensor", dilation=dil)
    _check(got, ref, dtype, gpu, "y")
    dy = gpu.rounded(normal(94, ref.shape), dtype)
    rdw, rdx = oracle.conv2d_bwd(x, w, dy, stride, dil, pad)
    dw, dx = gpu.run_conv_bwd(x, w, dy, stride, pad, dtype, "16p", "tensor", True, dilation=dil)
    _check(dx, rdx, dtype, gpu, "dx")
    _check(dw, rdw, dtype, gpu, "dw")


@pytest.mark.parametrize("shape", GENERAL_TENSOR_SHAPES + [(2, 40, 24, 6, 5, 1, 1, (1, 1), (0, 0, 0, 0))])
def test_fp32_on_tensor_cores_3xtf32_vs_oracle(gpu, oracle, shape):
    """fp32 tensors through the error-compensated TF32 kernels must hold the fp32 tolerance (1e-5), and agree with
    the CUDA-core fp32 kernels."""
    n, ci, co, h, w_, kh, kw, stride, pad = shape
    x = uniform(51, (4 * n, ci, h, w_))
    w = normal(52, (4, co, ci, kh, kw), std=(2.0 / (4 * ci * kh * kw)) ** 0.5)
    b = uniform(53, (4, co))
    ref = oracle.conv2d_fwd(x, w, b, stride, (1, 1), pad)
    got = gpu.run_conv_fwd(x, w, b, stride, pad, "f32", "16p", "tensor")
    _check(got, ref, "f32", gpu, "y")
    dy = normal(54, ref.shape)
    rdw, rdx = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad)
    dw, dx = gpu.run_conv_bwd(x, w, dy, stride, pad, "f32", "16p", "tensor", True)
    _check(dx, rdx, "f32", gpu, "dx")
    _check(dw, rdw, "f32", gpu, "dw")
    simt = gpu.run_conv_fwd(x, w, b, stride, pad, "f32", "16p", "simt")
    assert rel_err(got, simt) <= 1e-5


@pytest.mark.parametrize("shape", [(3, 5, 7), (32, 64, 48), (17, 130, 70), (256, 512, 512)])
@pytest.mark.parametrize("oi", [False, True])
def test_dense_fp32_on_tensor_cores_vs_oracle(gpu, oracle, shape, oi):
    b_, i, o = shape
    x = normal(61, (4 * b_, i))
    w = normal(62, (4, o, i) if oi else (4, i, o), std=(2.0 / (4 * i)) ** 0.5)
    bias = uniform(63, (4, o))
    ref = oracle.dense_fwd(x, w, bias, oi)
    _check(gpu.run_dense_fwd(x, w, bias, oi, "f32", "16p", "tensor"), ref, "f32", gpu, "y")
    dy = normal(64, ref.shape)
    rdw, rdx = oracle.dense_bwd(x, w, dy, oi)
    dw, dx = gpu.run_dense_bwd(x, w, dy, oi, "f32", "16p", "tensor", True)
    _check(dw, rdw, "f32", gpu, "dw")
    _check(dx, rdx, "f32", gpu, "dx")


def test_tensor_engine_refuses_unsupported_shapes(gpu):
    from phoenix_core_b200 import _lib
    x = uniform(1, (4, 3, 5, 5))
    w = uniform(2, (4, 2, 3, 3, 3))
    with pytest.raises(_lib.BackendError) as e:      # stride 3 has no tensor-core kernel
        gpu.run_conv_fwd(x, w, None, (3, 3), (1, 1, 1, 1), "f16", "16p", "tensor")
    assert e.value.status == _lib.PCB_ERR_UNSUPPORTED
    with pytest.raises(_lib.BackendError) as e:      # the factorised tensor-core kernels cover pointwise layers only
        gpu.run_conv_fwd(x, w, None, (1, 1), (1, 1, 1, 1), "f16", "8p", "tensor")
    assert e.value.status == _lib.PCB_ERR_UNSUPPORTED


def test_fp16_policies_give_one_result(gpu, oracle):
    """UPSTRIDE_CONV_FP16_POLICY is carried for API parity and not consulted: under each of the three policies the same
    kernels run (products exact, fp32 accumulation), so the outputs are bit-identical and within tolerance of the oracle."""
    import phoenix_core_b200 as pcb
    from phoenix_core_b200.context import Context
    x = gpu.rounded(uniform(81, (4 * 2, 32, 10, 12)), "f16")
    w = gpu.rounded(uniform(82, (4, 32, 32, 3, 3)) * 0.1, "f16")
    ref = oracle.conv2d_fwd(x, w, None, (1, 1), (1, 1), (1, 1, 1, 1))
    fwd, _ = gpu.conv_descriptors(x.shape, w.shape, (1, 1), (1, 1, 1, 1), False, False)
    outs = []
    for policy in ("full16", "backward32", "fp32"):
        ctx = Context({"UPSTRIDE_MEMORY_OPTIMIZED": "1", "UPSTRIDE_CONV_FP16_POLICY": policy})
        y = torch.full(fwd.getOutputShape(), float("nan"), dtype=torch.float16, device="cuda")
        pcb.conv2DFwd(gpu.dev(x, "f16"), gpu.dev(w, "f16"), None, y, fwd, ctx)
        outs.append(gpu.host(y))
        _check(outs[-1], ref, "f16", gpu, "y under " + policy)
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])


def test_real_valued_input(gpu, oracle):
    x = uniform(21, (3, 4, 9, 7))
    w = uniform(22, (4, 6, 4, 3, 3))
    ref = oracle.conv2d_fwd(x, w, None, (2, 2), (1, 1), (1, 1, 1, 1), real_input=True)
    got = gpu.run_conv_fwd(x, w, None, (2, 2), (1, 1, 1, 1), "f32", "8p", "auto", real_input=True)
    _check(got, ref, "f32", gpu, "y (real input)")


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_real_valued_input_on_tensor_cores(gpu, oracle, dtype):
    """The stem configuration: real RGB input, 7x7 stride 2, SAME padding; forward and filter gradient (the
    input gradient of a real-valued input does not exist)."""
    import ctypes
    import phoenix_core_b200 as pcb
    from phoenix_core_b200 import _lib
    x = gpu.rounded(uniform(23, (3, 3, 30, 26)), dtype)
    w = gpu.rounded(normal(24, (4, 16, 3, 7, 7), std=0.08), dtype)
    stride, pad = (2, 2), (2, 2, 3, 3)
    ref = oracle.conv2d_fwd(x, w, None, stride, (1, 1), pad, real_input=True)
    got = gpu.run_conv_fwd(x, w, None, stride, pad, dtype, "16p", "tensor", real_input=True)
    _check(got, ref, dtype, gpu, "y (real input)")
    # filter gradient: a real input is the quaternion input with zero imaginary parts
    dy = gpu.rounded(normal(25, ref.shape), dtype)
    xq = np.concatenate([x, np.zeros((9,) + x.shape[1:], np.float32)], 0)
    rdw, _ = oracle.conv2d_bwd(xq, w, dy, stride, (1, 1), pad, need_dx=False)
    _, bwd = gpu.conv_descriptors(x.shape, w.shape, stride, pad, False, False, real_input=True)
    dw = torch.full(w.shape, float("nan"), dtype=gpu.TORCH_DTYPES[dtype], device="cuda")
    pcb.conv2DBwd(gpu.dev(x, dtype), gpu.dev(w, dtype), gpu.dev(dy, dtype), dw, None, bwd, gpu.context("16p"), _lib.ENGINE_TENSOR)
    _check(gpu.host(dw), rdw, dtype, gpu, "dw (real input)")


def test_empty_batch(gpu):
    import phoenix_core_b200 as pcb
    fwd, bwd = gpu.conv_descriptors((0, 3, 5, 5), (4, 2, 3, 3, 3), (1, 1), (1, 1, 1, 1), False, True)
    x = torch.zeros((0, 3, 5, 5), device="cuda")
    w = torch.ones((4, 2, 3, 3, 3), device="cuda")
    y = torch.zeros(fwd.getOutputShape(), device="cuda")
    pcb.conv2DFwd(x, w, None, y, fwd)
    dw = torch.ones_like(w)
    pcb.conv2DBwd(x, w, y, dw, x.clone(), bwd)
    assert float(dw.abs().sum()) == 0.0


DENSE_SHAPES = [(3, 5, 7), (8, 16, 4), (1, 1, 1), (32, 64, 48), (17, 130, 70)]


@pytest.mark.parametrize("shape", DENSE_SHAPES)
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("variant,engine", FORMULATIONS)
@pytest.mark.parametrize("oi", [False, True])
def test_dense_fwd_bwd_vs_oracle(gpu, oracle, shape, dtype, variant, engine, oi):
    b_, i, o = shape
    x = gpu.rounded(normal(31, (4 * b_, i)), dtype)
    w = gpu.rounded(normal(32, (4, o, i) if oi else (4, i, o), std=(2.0 / (4 * i)) ** 0.5), dtype)
    bias = gpu.rounded(uniform(33, (4, o)), dtype)
    ov = oracle.VARIANT_16P if variant == "16p" else oracle.VARIANT_8P
    ref = oracle.dense_fwd(x, w, bias, oi, oracle.QUATERNION, ov)
    got = gpu.run_dense_fwd(x, w, bias, oi, dtype, variant, engine)
    _check(got, ref, dtype, gpu, "y")
    dy = gpu.rounded(normal(34, ref.shape), dtype)
    rdw, rdx = oracle.dense_bwd(x, w, dy, oi, oracle.QUATERNION, ov, True)
    dw, dx = gpu.run_dense_bwd(x, w, dy, oi, dtype, variant, engine, True)
    _check(dw, rdw, dtype, gpu, "dw")
    _check(dx, rdx, dtype, gpu, "dx")


def test_baseline_config1_conv3x3_fp32(gpu, oracle):
    """Single quaternion conv2d forward, fp32: N=8, 16->16 channels, 32x32, 3x3, stride 1, pad 1, U[-1,1]."""
    x = uniform(101, (4 * 8, 16, 32, 32))
    w = uniform(102, (4, 16, 16, 3, 3))
    for variant, engine in FORMULATIONS:
        ov = oracle.VARIANT_16P if variant == "16p" else oracle.VARIANT_8P
        ref = oracle.conv2d_fwd(x, w, None, (1, 1), (1, 1), (1, 1, 1, 1), oracle.QUATERNION, ov)
        got = gpu.run_conv_fwd(x, w, None, (1, 1), (1, 1, 1, 1), "f32", variant, engine)
        _check(got, ref, "f32", gpu, "config 1 " + variant + " " + engine)


def test_baseline_config2_dense_fp32(gpu, oracle):
    """Quaternion dense fwd+bwd, fp32: batch 256, 512 -> 512, He-normal weights, N(0,1) upstream gradient."""
    x = normal(201, (4 * 256, 512))
    w = normal(202, (4, 512, 512), std=(2.0 / (4 * 512)) ** 0.5)
    bias = np.zeros((4, 512), np.float32)
    dy = normal(203, (4 * 256, 512))
    for variant, engine in FORMULATIONS:
        ov = oracle.VARIANT_16P if variant == "16p" else oracle.VARIANT_8P
        _check(gpu.run_dense_fwd(x, w, bias, False, "f32", variant, engine),
               oracle.dense_fwd(x, w, bias, False, oracle.QUATERNION, ov), "f32", gpu, "config 2 y " + variant + " " + engine)
        rdw, rdx = oracle.dense_bwd(x, w, dy, False, oracle.QUATERNION, ov, True)
        dw, dx = gpu.run_dense_bwd(x, w, dy, False, "f32", variant, engine, True)
        _check(dw, rdw, "f32", gpu, "config 2 dw " + variant)
        _check(dx, rdx, "f32", gpu, "config 2 dx " + variant)


def test_baseline_config3_pointwise_fp16_reduced_batch(gpu, oracle):
    """Pointwise 1x1 conv fwd+bwd, fp16 in/out, 128 -> 256 channels, 56x56 (batch reduced from 64 to 1 so that
    the oracle finishes in seconds), both formulations; the 16-product one runs on the tensor cores."""
    from phoenix_core_b200 import _lib
    x = gpu.rounded(normal(301, (4 * 1, 128, 56, 56)), "f16")
    w = gpu.rounded(normal(302, (4, 256, 128, 1, 1), std=(2.0 / (4 * 128)) ** 0.5), "f16")
    pad, stride = (0, 0, 0, 0), (1, 1)
    for variant, engine in FORMULATIONS:
        ov = oracle.VARIANT_16P if variant == "16p" else oracle.VARIANT_8P
        ref = oracle.conv2d_fwd(x, w, None, stride, (1, 1), pad, oracle.QUATERNION, ov)
        _check(gpu.run_conv_fwd(x, w, None, stride, pad, "f16", variant, engine), ref, "f16", gpu, "config 3 y " + variant)
        dy = gpu.rounded(normal(303, ref.shape), "f16")
        rdw, rdx = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad, oracle.QUATERNION, ov, True)
        dw, dx = gpu.run_conv_bwd(x, w, dy, stride, pad, "f16", variant, engine, True)
        _check(dw, rdw, "f16", gpu, "config 3 dw " + variant)
        _check(dx, rdx, "f16", gpu, "config 3 dx " + variant)
