"""Shared helpers for the tests: seeded inputs, an independent float64 formulation, error norms."""
import json
import os

import numpy as np
import torch

# 4x4 signed block of the Hamilton product y = x (x) w with the input on the left: entry [l][d] = (r, s)
# means that input component l contributes s * w_r to output component d.
QUAT_BLOCK = [
    [(0, +1), (1, +1), (2, +1), (3, +1)],
    [(1, -1), (0, +1), (3, -1), (2, +1)],
    [(2, -1), (3, +1), (0, +1), (1, -1)],
    [(3, -1), (2, -1), (1, +1), (0, +1)],
]


def algebra_block(name):
    """The D x D signed block of an algebra ("REAL", "COMPLEX", "QUATERNION", "GA_300") in the form of QUAT_BLOCK,
    built from the reference's product table as transcribed in golden/reference_sign_tables.json."""
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_sign_tables.json")) as f:
        entries = json.load(f)[name]["entries"]
    dims = int(round(len(entries) ** 0.5))
    block = [[None] * dims for _ in range(dims)]
    for idx, (l, r, s) in enumerate(entries):
        block[l][idx // dims] = (r, s)
    assert all(e is not None for row in block for e in row)
    return block


def rng(seed):
    return np.random.default_rng(seed)


def uniform(seed, shape, lo=-1.0, hi=1.0):
    return rng(seed).uniform(lo, hi, size=shape).astype(np.float32)


def normal(seed, shape, std=1.0):
    return (rng(seed).standard_normal(size=shape) * std).astype(np.float32)


def integers(seed, shape, lo=-3, hi=4):
    return rng(seed).integers(lo, hi, size=shape).astype(np.float32)


def block_weights_conv(w, block=QUAT_BLOCK):
    """[D, Co, Ci, kh, kw] -> real conv weights [D*Co, D*Ci, kh, kw] (float64 torch tensor)."""
    D = len(block)
    w = torch.as_tensor(np.asarray(w), dtype=torch.float64)
    _, co, ci, kh, kw = w.shape
    big = torch.zeros(D, co, D, ci, kh, kw, dtype=torch.float64)
    for l in range(D):
        for d in range(D):
            r, s = block[l][d]
            big[d, :, l] = s * w[r]
    return big.reshape(D * co, D * ci, kh, kw)


def to_real_layout(x, D=4):
    """[D*N, C, ...] (component-major on the batch axis) -> [N, D*C, ...] float64 torch tensor."""
    x = torch.as_tensor(np.asarray(x), dtype=torch.float64)
    n = x.shape[0] // D
    x = x.reshape(D, n, *x.shape[1:])
    x = x.transpose(0, 1)
    return x.reshape(n, D * x.shape[2], *x.shape[3:])


def from_real_layout(y, D=4):
    """[N, D*C, ...] -> [D*N, C, ...] numpy float64."""
    n = y.shape[0]
    c = y.shape[1] // D
    y = y.reshape(n, D, c, *y.shape[2:]).transpose(0, 1)
    return y.reshape(D * n, c, *y.shape[3:]).detach().numpy()


def conv_fwd_f64(x, w, bias, stride, pad, block=QUAT_BLOCK, dilation=(1, 1)):
    """Independent float64 formulation: one real convolution with the D x D signed block (via torch, CPU)."""
    D = len(block)
    xr = to_real_layout(x, D)
    pt, pl, pb, pr = pad
    xr = torch.nn.functional.pad(xr, (pl, pr, pt, pb))
    b = None if bias is None else torch.as_tensor(np.asarray(bias), dtype=torch.float64).reshape(-1)
    y = torch.nn.functional.conv2d(xr, block_weights_conv(w, block), b, stride=stride, dilation=dilation)
    return from_real_layout(y, D)


def conv_bwd_f64(x, w, dy, stride, pad, block=QUAT_BLOCK, dilation=(1, 1)):
    """dW, dX in float64 by automatic differentiation of the block-matrix formulation."""
    D = len(block)
    xt = torch.as_tensor(np.asarray(x), dtype=torch.float64).requires_grad_(True)
    wt = torch.as_tensor(np.asarray(w), dtype=torch.float64).requires_grad_(True)
    n = xt.shape[0] // D
    xr = xt.reshape(D, n, *xt.shape[1:]).transpose(0, 1).reshape(n, D * xt.shape[1], *xt.shape[2:])
    pt, pl, pb, pr = pad
    xr = torch.nn.functional.pad(xr, (pl, pr, pt, pb))
    _, co, ci, kh, kw = wt.shape
    rows = []
    for d in range(D):
        cols = []
        for l in range(D):
            r, s = block[l][d]
            cols.append(s * wt[r])
        rows.append(torch.cat(cols, dim=1))
    big = torch.cat(rows, dim=0)
    y = torch.nn.functional.conv2d(xr, big, None, stride=stride, dilation=dilation)
    yq = y.reshape(n, D, co, *y.shape[2:]).transpose(0, 1).reshape(D * n, co, *y.shape[2:])
    yq.backward(torch.as_tensor(np.asarray(dy), dtype=torch.float64))
    return wt.grad.numpy(), xt.grad.numpy()


def dense_fwd_f64(x, w, bias, oi=False, block=QUAT_BLOCK):
    D = len(block)
    x = np.asarray(x, np.float64)
    w = np.asarray(w, np.float64)
    if oi:
        w = np.swapaxes(w, 1, 2)
    b = x.shape[0] // D
    xs = x.reshape(D, b, -1)
    y = np.zeros((D, b, w.shape[2]))
    for l in range(D):
        for d in range(D):
            r, s = block[l][d]
            y[d] += s * xs[l] @ w[r]
    if bias is not None:
        y += np.asarray(bias, np.float64)[:, None, :]
    return y.reshape(D * b, -1)


def dense_bwd_f64(x, w, dy, oi=False, block=QUAT_BLOCK):
    """Returns dW in [D, I, O] orientation and dX."""
    D = len(block)
    x = np.asarray(x, np.float64)
    w = np.asarray(w, np.float64)
    dy = np.asarray(dy, np.float64)
    if oi:
        w = np.swapaxes(w, 1, 2)
    b = x.shape[0] // D
    xs, gs = x.reshape(D, b, -1), dy.reshape(D, b, -1)
    dw = np.zeros_like(w)
    dx = np.zeros_like(xs)
    for l in range(D):
        for d in range(D):
            r, s = block[l][d]
            dw[r] += s * xs[l].T @ gs[d]
            dx[l] += s * gs[d] @ w[r].T
    return dw, dx.reshape(D * b, -1)


def rel_err(got, ref):
    """max|got - ref| / max|ref|  (the per-tensor relative error the tolerances are stated in)."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    denom = np.max(np.abs(ref))
    if denom == 0:
        return float(np.max(np.abs(got)))
    return float(np.max(np.abs(got - ref)) / denom)
