"""Parity at the real channel counts of the ResNet-stage sweep (256 channels at 14x14, 512 at 7x7): 3x3 stride 1 and 2
and 1x1, all three passes, fp16 / bf16 / fp32 (3 x TF32), batch 2, and the pointwise benchmark layer at batch 2.

Reference: the independent float64 block-matrix formulation (tests/helpers.py; the direct-loop oracle needs minutes at
512 channels), which test_oracle.py holds equal to the oracle. The depth of the reduction is what these cases add:
K = 4*512*9 = 18432 products per output, 288 K stages per tile, an 18.9 MB expanded filter matrix. The fp32 error of
the error-compensated TF32 path grows with the number of MMAs per accumulator, so it is printed and bounded here.
"""
import numpy as np
import pytest
import torch

from helpers import conv_bwd_f64, conv_fwd_f64, normal, rel_err, uniform

pytestmark = pytest.mark.gpu

# ci = co, h = w, k, stride, pad
STAGE_SHAPES = [
    (256, 14, 3, 1, 1),
    (256, 14, 3, 2, 1),
    (256, 14, 1, 1, 0),
    (256, 14, 1, 2, 0),
    (512, 7, 3, 1, 1),
    (512, 7, 3, 2, 1),
    (512, 7, 1, 1, 0),
    (512, 7, 1, 2, 0),
]


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util
    return gpu_util


@pytest.mark.parametrize("shape", STAGE_SHAPES)
@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
def test_stage_shapes_at_real_channel_counts(gpu, shape, dtype):
    c, hw, k, s, p = shape
    n = 2
    x = gpu.rounded(uniform(71, (4 * n, c, hw, hw)), dtype)
    w = gpu.rounded(uniform(72, (4, c, c, k, k)), dtype)          # U[-1,1] as the sweep configuration states
    stride, pad = (s, s), (p, p, p, p)
    ref = conv_fwd_f64(x, w, None, stride, pad)
    got = gpu.run_conv_fwd(x, w, None, stride, pad, dtype, "16p", "tensor")
    errs = {"y": rel_err(got, ref)}
    dy = gpu.rounded(normal(73, ref.shape), dtype)
    rdw, rdx = conv_bwd_f64(x, w, dy, stride, pad)
    dw, dx = gpu.run_conv_bwd(x, w, dy, stride, pad, dtype, "16p", "tensor", True)
    errs["dw"], errs["dx"] = rel_err(dw, rdw), rel_err(dx, rdx)
    print("stage shape %s %s: relative errors %s (K = %d products per output)" % (shape, dtype, errs, 4 * c * k * k))
    for name, e in errs.items():
        assert np.isfinite(e) and e <= gpu.TOL[dtype], "%s: %.3e > %.1e" % (name, e, gpu.TOL[dtype])


@pytest.mark.parametrize("variant,engine", [("16p", "tensor"), ("8p", "tensor"), ("8p", "simt")])
def test_benchmark_layer_at_batch_2(gpu, variant, engine):
    """The pointwise benchmark layer (128 -> 256 channels, 56x56, fp16) at batch 2: several tiles per CTA, the image
    boundary inside a tile pair, both formulations."""
    n = 2
    x = gpu.rounded(normal(301, (4 * n, 128, 56, 56)), "f16")
    w = gpu.rounded(normal(302, (4, 256, 128, 1, 1), std=(2.0 / (4 * 128)) ** 0.5), "f16")
    ref = conv_fwd_f64(x, w, None, (1, 1), (0, 0, 0, 0))
    got = gpu.run_conv_fwd(x, w, None, (1, 1), (0, 0, 0, 0), "f16", variant, engine)
    assert rel_err(got, ref) <= 2e-2
    dy = gpu.rounded(normal(303, ref.shape), "f16")
    rdw, rdx = conv_bwd_f64(x, w, dy, (1, 1), (0, 0, 0, 0))
    dw, dx = gpu.run_conv_bwd(x, w, dy, (1, 1), (0, 0, 0, 0), "f16", variant, engine, True)
    assert rel_err(dw, rdw) <= 2e-2 and rel_err(dx, rdx) <= 2e-2
