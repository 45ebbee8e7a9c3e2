"""CPU tests of the oracle: the reference's own known-answer vectors, then identities that pin the parts
the reference never tested (backward, bias, dense, 8-product vs 16-product)."""
import json
import os

import numpy as np
import pytest

from helpers import (QUAT_BLOCK, algebra_block, conv_bwd_f64, conv_fwd_f64, dense_bwd_f64, dense_fwd_f64, integers,
                     normal, rel_err, uniform)

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")
ALG = {"real": 0, "complex": 1, "quaternion": 2, "ga_300": 3}


def _cases(op):
    with open(GOLDEN) as f:
        return [c for c in json.load(f)["cases"] if c["op"] == op]


def _tensor(case, key):
    shape = case[key + "_shape"]
    if key + "_fill" in case:
        return np.full(shape, case[key + "_fill"], np.float32)
    return np.asarray(case[key], np.float32).reshape(shape)


@pytest.mark.parametrize("case", _cases("conv2d_fwd"), ids=lambda c: c["name"])
@pytest.mark.parametrize("variant", [0, 1])
def test_reference_conv_kats(oracle, case, variant):
    if variant == 1 and (case["algebra"] != "quaternion" or case["real_input"]):
        pytest.skip("8-product form exists for full quaternion inputs only")
    x, w, y = _tensor(case, "x"), _tensor(case, "w"), _tensor(case, "y")
    got = oracle.conv2d_fwd(x, w, None, tuple(case["stride"]), tuple(case["dilation"]), (0, 0, 0, 0),
                            ALG[case["algebra"]], variant, case["real_input"])
    assert got.shape == tuple(case["y_shape"])
    assert np.array_equal(got, y)       # the reference compares with threshold 0


@pytest.mark.parametrize("case", _cases("dense_fwd"), ids=lambda c: c["name"])
def test_reference_dense_kats(oracle, case):
    x, w, y = _tensor(case, "x"), _tensor(case, "w"), _tensor(case, "y")
    got = oracle.dense_fwd(x, w, None, False, ALG[case["algebra"]], 0)
    assert np.array_equal(got, y)


def test_reference_same_padding_shape(oracle):
    (case,) = _cases("output_shape")
    # NHWC input, OHWI filter: H = W = 224, kh = kw = 3
    h = case["x_shape"][1]
    k = case["w_shape"][2]
    out, before, after = oracle.same_or_valid_padding(h, k, case["dilation"][0], case["stride"][0], oracle.SAME)
    assert out == case["y_shape"][1]
    assert oracle.output_size(h, k, case["dilation"][0], case["stride"][0], before, after) == out


def test_sign_table_is_the_4x4_block(oracle):
    table = oracle.quaternion_sign_table()
    assert len(table) == 16
    for idx, (l, r, s) in enumerate(table):
        d = idx // 4
        assert QUAT_BLOCK[l][d] == (r, s)


@pytest.mark.parametrize("name,code", [("REAL", 0), ("COMPLEX", 1), ("QUATERNION", 2), ("GA_300", 3)])
def test_sign_tables_equal_the_reference_lists(oracle, name, code):
    """The oracle's tables (GA(3,0,0) is derived from the blade algebra) against the reference's lists as data."""
    with open(os.path.join(os.path.dirname(GOLDEN), "reference_sign_tables.json")) as f:
        ref = json.load(f)[name]["entries"]
    assert [list(e) for e in oracle.sign_table(code)] == ref


def test_ga300_table_is_an_associative_algebra_with_unit_squares(oracle):
    """Independent of the transcription: e1, e2, e3 square to +1, anticommute, and the product is associative."""
    block = {}
    for idx, (l, r, s) in enumerate(oracle.sign_table(oracle.GA_300)):
        block[(l, r)] = (idx // 8, s)           # blade l times blade r = s * blade d
    for g in (1, 2, 3):
        assert block[(g, g)] == (0, 1)
    for a in (1, 2, 3):
        for b in (1, 2, 3):
            if a != b:
                assert block[(a, b)][0] == block[(b, a)][0] and block[(a, b)][1] == -block[(b, a)][1]
    assert block[(1, 2)] == (4, 1) and block[(1, 3)] == (5, 1) and block[(2, 3)] == (6, 1) and block[(4, 3)] == (7, 1)
    for a in range(8):
        for b in range(8):
            for c in range(8):
                ab, s1 = block[(a, b)]
                left, s2 = block[(ab, c)]
                bc, s3 = block[(b, c)]
                right, s4 = block[(a, bc)]
                assert (left, s1 * s2) == (right, s3 * s4)


ALGEBRA_CASES = [("REAL", 0), ("COMPLEX", 1), ("GA_300", 3)]


@pytest.mark.parametrize("name,code", ALGEBRA_CASES)
@pytest.mark.parametrize("shape", [(2, 3, 5, 7, 6, 3, 3, (1, 1), (1, 1, 1, 1)), (1, 4, 2, 9, 8, 3, 3, (2, 2), (0, 0, 1, 1))])
def test_other_algebras_conv_matches_float64_block_form(oracle, name, code, shape):
    """Complex, GA(3,0,0) and real convolution (forward, both gradients) against the float64 block formulation built from
    the reference's tables; real tensors carry a leading axis of one component here."""
    n, ci, co, h, w_, kh, kw, stride, pad = shape
    block = algebra_block(name)
    D = len(block)
    x = uniform(21, (D * n, ci, h, w_))
    w = uniform(22, (D, co, ci, kh, kw))
    b = uniform(23, (D, co))
    got = oracle.conv2d_fwd(x, w, b, stride, (1, 1), pad, code, 0)
    ref = conv_fwd_f64(x, w, b, stride, pad, block)
    assert got.shape == ref.shape and rel_err(got, ref) < 2e-6
    dy = normal(24, ref.shape)
    dw, dx = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad, code, 0, True)
    rdw, rdx = conv_bwd_f64(x, w, dy, stride, pad, block)
    assert rel_err(dw, rdw) < 2e-6 and rel_err(dx, rdx) < 2e-6


@pytest.mark.parametrize("name,code", ALGEBRA_CASES)
@pytest.mark.parametrize("oi", [False, True])
def test_other_algebras_dense_matches_float64_block_form(oracle, name, code, oi):
    block = algebra_block(name)
    D = len(block)
    b_, i_, o_ = 5, 7, 4
    x = uniform(31, (D * b_, i_))
    w = uniform(32, (D, o_, i_) if oi else (D, i_, o_))
    bias = uniform(33, (D, o_))
    assert rel_err(oracle.dense_fwd(x, w, bias, oi, code, 0), dense_fwd_f64(x, w, bias, oi, block)) < 2e-6
    dy = normal(34, (D * b_, o_))
    dw, dx = oracle.dense_bwd(x, w, dy, oi, code, 0, True)
    rdw, rdx = dense_bwd_f64(x, w, dy, oi, block)
    assert rel_err(dw, rdw) < 2e-6 and rel_err(dx, rdx) < 2e-6


def test_tf_padding_rules(oracle):
    # SAME: out = ceil(in / stride), extra pixel goes after
    assert oracle.same_or_valid_padding(7, 3, 1, 2, oracle.SAME) == (4, 1, 1)
    assert oracle.same_or_valid_padding(8, 3, 1, 2, oracle.SAME) == (4, 0, 1)
    assert oracle.same_or_valid_padding(224, 7, 1, 2, oracle.SAME) == (112, 2, 3)
    assert oracle.same_or_valid_padding(5, 3, 1, 1, oracle.VALID) == (3, 0, 0)
    assert oracle.same_or_valid_padding(5, 3, 2, 1, oracle.VALID) == (1, 0, 0)


CONV_SHAPES = [
    # n, ci, co, h, w, kh, kw, stride, pad(t,l,b,r)
    (2, 3, 5, 7, 6, 3, 3, (1, 1), (1, 1, 1, 1)),
    (1, 4, 2, 9, 8, 3, 3, (2, 2), (0, 0, 1, 1)),      # asymmetric SAME-style padding
    (3, 2, 3, 5, 5, 1, 1, (1, 1), (0, 0, 0, 0)),
    (2, 2, 4, 8, 7, 1, 1, (2, 2), (0, 0, 0, 0)),
    (1, 3, 2, 10, 9, 5, 3, (2, 1), (2, 1, 2, 1)),
]


@pytest.mark.parametrize("shape", CONV_SHAPES)
@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("use_bias", [False, True])
def test_conv_fwd_matches_float64_block_form(oracle, shape, variant, use_bias):
    n, ci, co, h, w_, kh, kw, stride, pad = shape
    x = uniform(1, (4 * n, ci, h, w_))
    w = uniform(2, (4, co, ci, kh, kw))
    b = uniform(3, (4, co)) if use_bias else None
    got = oracle.conv2d_fwd(x, w, b, stride, (1, 1), pad, oracle.QUATERNION, variant)
    ref = conv_fwd_f64(x, w, b, stride, pad)
    assert got.shape == ref.shape
    assert rel_err(got, ref) < 2e-6


@pytest.mark.parametrize("shape", CONV_SHAPES)
@pytest.mark.parametrize("variant", [0, 1])
def test_conv_bwd_matches_float64_autograd(oracle, shape, variant):
    n, ci, co, h, w_, kh, kw, stride, pad = shape
    x = uniform(4, (4 * n, ci, h, w_))
    w = uniform(5, (4, co, ci, kh, kw))
    y = oracle.conv2d_fwd(x, w, None, stride, (1, 1), pad)
    dy = normal(6, y.shape)
    dw, dx = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad, oracle.QUATERNION, variant, True)
    rdw, rdx = conv_bwd_f64(x, w, dy, stride, pad)
    assert rel_err(dw, rdw) < 2e-6
    assert rel_err(dx, rdx) < 2e-6
    dw2, none = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad, oracle.QUATERNION, variant, False)
    assert none is None and np.array_equal(dw, dw2)


def test_conv_integer_inputs_16p_equals_8p_exactly(oracle):
    # with small integers every intermediate is exact in float, so the two forms must agree bit for bit
    x = integers(7, (8, 3, 6, 6))
    w = integers(8, (4, 4, 3, 3, 3)) * 2      # even weights keep the 0.5 factor of the 8-product form exact
    a = oracle.conv2d_fwd(x, w, None, (1, 1), (1, 1), (1, 1, 1, 1), variant=0)
    b = oracle.conv2d_fwd(x, w, None, (1, 1), (1, 1), (1, 1, 1, 1), variant=1)
    assert np.array_equal(a, b)


def test_conv_finite_difference(oracle):
    """dW and dX of the oracle against central differences of its own forward, in one random direction."""
    x = uniform(9, (4, 2, 5, 5))
    w = uniform(10, (4, 3, 2, 3, 3))
    pad, stride = (1, 1, 1, 1), (1, 1)
    dy = normal(11, oracle.conv2d_fwd(x, w, None, stride, (1, 1), pad).shape)
    dw, dx = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad)
    vx, vw = normal(12, x.shape), normal(13, w.shape)
    eps = 1e-2

    def loss(xx, ww):
        return float(np.sum(conv_fwd_f64(xx, ww, None, stride, pad) * dy.astype(np.float64)))

    fd_x = (loss(x + eps * vx, w) - loss(x - eps * vx, w)) / (2 * eps)
    fd_w = (loss(x, w + eps * vw) - loss(x, w - eps * vw)) / (2 * eps)
    assert abs(fd_x - float(np.sum(dx.astype(np.float64) * vx))) < 1e-3 * max(1.0, abs(fd_x))
    assert abs(fd_w - float(np.sum(dw.astype(np.float64) * vw))) < 1e-3 * max(1.0, abs(fd_w))


def test_conv_empty_input(oracle):
    x = np.zeros((0, 3, 5, 5), np.float32)
    w = uniform(14, (4, 2, 3, 3, 3))
    y = oracle.conv2d_fwd(x, w, None, (1, 1), (1, 1), (1, 1, 1, 1))
    assert y.shape == (0, 2, 5, 5)
    dw, _ = oracle.conv2d_bwd(x, w, y, (1, 1), (1, 1), (1, 1, 1, 1))
    assert np.all(dw == 0)


@pytest.mark.parametrize("b,i,o", [(3, 5, 7), (8, 16, 4), (1, 1, 1)])
@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("oi", [False, True])
def test_dense_matches_float64(oracle, b, i, o, variant, oi):
    x = normal(20, (4 * b, i))
    w = normal(21, (4, o, i) if oi else (4, i, o))
    bias = uniform(22, (4, o))
    y = oracle.dense_fwd(x, w, bias, oi, oracle.QUATERNION, variant)
    assert rel_err(y, dense_fwd_f64(x, w, bias, oi)) < 2e-6
    dy = normal(23, y.shape)
    dw, dx = oracle.dense_bwd(x, w, dy, oi, oracle.QUATERNION, variant, True)
    rdw, rdx = dense_bwd_f64(x, w, dy, oi)
    assert dw.shape == (4, i, o)        # always input-major, as both reference backends emit it
    assert rel_err(dw, rdw) < 2e-6
    assert rel_err(dx, rdx) < 2e-6


@pytest.mark.parametrize("variant8", [False, True])
def test_library_orchestration_agrees_with_oracle(oracle, variant8):
    """The torch-CPU (oneDNN) orchestration used as timed CPU baseline computes what the C oracle computes."""
    import torch
    from oracle import ref_orchestration as ro
    x = uniform(41, (4 * 2, 6, 9, 8))
    w = uniform(42, (4, 5, 6, 3, 3))
    b = uniform(43, (4, 5))
    stride, pad = (2, 2), (0, 0, 1, 1)
    v = 1 if variant8 else 0
    y = ro.conv2d_fwd(torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(b), stride, pad, variant8).numpy()
    ref = oracle.conv2d_fwd(x, w, b, stride, (1, 1), pad, oracle.QUATERNION, v)
    assert rel_err(y, ref) < 1e-5
    dy = normal(44, ref.shape)
    dw, dx = ro.conv2d_bwd(torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(dy), stride, pad, variant8)
    rdw, rdx = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad, oracle.QUATERNION, v)
    assert rel_err(dw.numpy(), rdw) < 1e-5 and rel_err(dx.numpy(), rdx) < 1e-5
    xd, wd, bd = normal(45, (4 * 7, 12)), normal(46, (4, 12, 9)), uniform(47, (4, 9))
    yd = ro.dense_fwd(torch.from_numpy(xd), torch.from_numpy(wd), torch.from_numpy(bd), variant8).numpy()
    assert rel_err(yd, oracle.dense_fwd(xd, wd, bd, False, oracle.QUATERNION, v)) < 1e-5
    gd = normal(48, yd.shape)
    ddw, ddx = ro.dense_bwd(torch.from_numpy(xd), torch.from_numpy(wd), torch.from_numpy(gd), variant8)
    rddw, rddx = oracle.dense_bwd(xd, wd, gd, False, oracle.QUATERNION, v)
    assert rel_err(ddw.numpy(), rddw) < 1e-5 and rel_err(ddx.numpy(), rddx) < 1e-5


@pytest.mark.parametrize("h,w_,kh,kw,stride,pad", [
    (10, 12, 3, 3, (2, 2), (1, 1, 1, 1)),     # the ResNet downsampling layer
    (10, 12, 3, 3, (2, 2), (0, 0, 1, 1)),     # SAME-style padding: the classes start at the other tap
    (9, 11, 3, 2, (1, 2), (1, 0, 1, 1)),      # classes along one axis, odd planes
    (9, 9, 5, 5, (2, 2), (2, 2, 2, 2)),       # 3 / 2 taps per class and axis
    (8, 8, 1, 1, (2, 2), (0, 0, 0, 0)),       # strided 1x1: one class holds every tap, the others are zero
    (11, 7, 7, 7, (2, 2), (2, 2, 3, 3)),      # the stem's geometry
])
def test_strided_backward_data_by_stride_classes(oracle, h, w_, kh, kw, stride, pad):
    """The identity behind the GPU path's strided backward-data: input pixels of class (ih mod SH, iw mod SW) receive
    only the taps r + S k' with r = (a + pad) mod S, and their gradient is a stride-1 correlation of dy with those taps,
    dx[S i + a] = sum_k' dy[i + c - k'] w[r + S k'] with c = (a + pad) div S. Checked against the oracle's strided
    backward-data pass (real algebra, one channel: the algebra and the channels do not enter the identity)."""
    sh, sw = stride
    pt, pl = pad[0], pad[1]
    x = uniform(81, (1, 1, h, w_))
    w = uniform(82, (1, 1, kh, kw))
    y = oracle.conv2d_fwd(x, w, None, stride, (1, 1), pad, oracle.REAL)
    dy = normal(83, y.shape)
    _, dx_ref = oracle.conv2d_bwd(x, w, dy, stride, (1, 1), pad, oracle.REAL, oracle.VARIANT_16P, True)
    ho, wo = y.shape[2], y.shape[3]
    dx = np.zeros((h, w_), np.float64)
    for a in range(sh):
        for b in range(sw):
            rh, ch = (a + pt) % sh, (a + pt) // sh
            rw, cw = (b + pl) % sw, (b + pl) // sw
            taps_h = range(0, (kh - rh + sh - 1) // sh) if rh < kh else range(0)
            taps_w = range(0, (kw - rw + sw - 1) // sw) if rw < kw else range(0)
            for i in range((h - a + sh - 1) // sh):
                for j in range((w_ - b + sw - 1) // sw):
                    acc = 0.0
                    for u in taps_h:
                        for v in taps_w:
                            oh, ow = i + ch - u, j + cw - v
                            if 0 <= oh < ho and 0 <= ow < wo:
                                acc += float(dy[0, 0, oh, ow]) * float(w[0, 0, rh + sh * u, rw + sw * v])
                    dx[sh * i + a, sw * j + b] = acc
    assert rel_err(dx.astype(np.float32), dx_ref[0, 0]) < 1e-6
