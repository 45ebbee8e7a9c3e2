"""The reference's CPU orchestration, timed: 8 or 16 real-valued library convolutions / matrix products plus
the element-wise lane and accumulate passes, executed with torch CPU ops (which run oneDNN, the library
family the reference's CPU backend calls). TEST / BENCHMARK INFRASTRUCTURE ONLY -- used as the CPU baseline
and as a second opinion on the C oracle; never imported by the product package.

Follows the reference's call structure: one scalar op per term, float32 intermediates between them
(``src/conv2d.hpp:167-275``, ``:433-562``; ``src/dense.hpp:64-181``, ``:238-378``; lane formulas
``src/backend/onednn/tensor.hpp:62-170``; sign table ``src/algebras.cc:28-53``). It is NOT the reference binary:
the reference's oneDNN submodule is absent and its sources use the pre-3.0 oneDNN API.
"""
import torch
import torch.nn.functional as F

SIGNTABLE = [  # (left, right, positive) rows of 4 per output component
    (0, 0, True), (1, 1, False), (2, 2, False), (3, 3, False),
    (0, 1, True), (1, 0, True), (2, 3, True), (3, 2, False),
    (0, 2, True), (1, 3, False), (2, 0, True), (3, 1, True),
    (0, 3, True), (1, 2, True), (2, 1, False), (3, 0, True)]
BACKPROP_ORDER = [10, 11, 12, 13, 0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 14, 15]


def _lanes_x(x):
    return [x[3] + x[1], x[0] - x[2], x[0] + x[2], x[3] - x[1], x[3] - x[2], x[1] + x[0], x[0] - x[1], x[3] + x[2]]


def _lanes_w(w):
    return [w[1] + w[2], w[0] + w[3], w[0] - w[3], w[1] - w[2], w[2] - w[3], w[1] + w[0], w[2] + w[3], w[0] - w[1]]


def _lanes_g(g):
    t1, t3, t2, t4 = g[0] + g[1], g[0] - g[1], g[2] + g[3], g[2] - g[3]
    return [0.5 * (t2 - t1), 0.5 * (t3 - t4), 0.5 * (t3 + t4), 0.5 * (t1 + t2), g[0], g[1], g[2], g[3]]


def _recompose_y(L):
    a2 = L[0] + L[1] + L[2]
    a5 = 0.5 * (a2 + L[3])
    return [a5 - L[0] + L[4], a5 - a2 + L[5], a5 - L[1] + L[6], a5 - L[2] + L[7]]


def _recompose_dx(p):
    return [p[1] + p[2] + p[5] + p[6], p[0] - p[3] + p[5] - p[6], p[2] - p[1] - p[4] + p[7], p[0] + p[3] + p[4] + p[7]]


def _recompose_dw(p):
    return [p[1] + p[2] + p[5] + p[7], p[0] + p[3] + p[5] - p[7], p[0] - p[3] + p[4] + p[6], p[1] - p[2] - p[4] + p[6]]


def _split(t):
    n = t.shape[0] // 4
    return [t[i * n:(i + 1) * n] for i in range(4)]


def _conv(x, w, b, stride, pad):
    pt, pl, pb, pr = pad
    if (pt, pl) != (pb, pr):
        x = F.pad(x, (pl, pr, pt, pb))
        return F.conv2d(x, w, b, stride=stride)
    return F.conv2d(x, w, b, stride=stride, padding=(pt, pl))


def conv2d_fwd(x, w, bias, stride, pad, variant8):
    xs, ws = _split(x), [w[i] for i in range(4)]
    bs = [None] * 4 if bias is None else [bias[i] for i in range(4)]
    if variant8:
        xl, wl = _lanes_x(xs), _lanes_w(ws)
        L = [_conv(xl[i], wl[i], bs[i - 4] if i >= 4 else None, stride, pad) for i in range(8)]
        return torch.cat(_recompose_y(L), 0)
    ys = []
    for dim in range(4):
        row = SIGNTABLE[4 * dim:4 * dim + 4]
        y = _conv(xs[row[0][0]], ws[row[0][1]], bs[dim], stride, pad)
        for (l, r, pos) in row[1:]:
            buf = _conv(xs[l], ws[r], None, stride, pad)
            y = y + buf if pos else y - buf
        ys.append(y)
    return torch.cat(ys, 0)


def _grads(x, w, g, stride, pad, need_dx):
    pt, pl, pb, pr = pad
    if (pt, pl) != (pb, pr):
        xp = F.pad(x, (pl, pr, pt, pb))
        dw = torch.nn.grad.conv2d_weight(xp, w.shape, g, stride=stride)
        dx = None
        if need_dx:
            dxp = torch.nn.grad.conv2d_input(xp.shape, w, g, stride=stride)
            dx = dxp[:, :, pt:pt + x.shape[2], pl:pl + x.shape[3]]
        return dw, dx
    dw = torch.nn.grad.conv2d_weight(x, w.shape, g, stride=stride, padding=(pt, pl))
    dx = torch.nn.grad.conv2d_input(x.shape, w, g, stride=stride, padding=(pt, pl)) if need_dx else None
    return dw, dx


def conv2d_bwd(x, w, dy, stride, pad, variant8, need_dx=True):
    xs, ws, gs = _split(x), [w[i] for i in range(4)], _split(dy)
    if variant8:
        xl, wl, gl = _lanes_x(xs), _lanes_w(ws), _lanes_g(gs)
        res = [_grads(xl[i], wl[i], gl[i], stride, pad, need_dx) for i in range(8)]
        dw = torch.stack(_recompose_dw([r[0] for r in res]), 0)
        dx = torch.cat(_recompose_dx([r[1] for r in res]), 0) if need_dx else None
        return dw, dx
    dws, dxs = [None] * 4, [None] * 4
    for i, j in enumerate(BACKPROP_ORDER):
        l, r, pos = SIGNTABLE[j]
        dim = j // 4
        bw, bx = _grads(xs[l], ws[r], gs[dim], stride, pad, need_dx)
        if i < 4:
            dws[r], dxs[l] = bw, bx
        else:
            dws[r] = dws[r] + bw if pos else dws[r] - bw
            if need_dx:
                dxs[l] = dxs[l] + bx if pos else dxs[l] - bx
    return torch.stack(dws, 0), (torch.cat(dxs, 0) if need_dx else None)


def dense_fwd(x, w, bias, variant8):
    """w is [4, I, O]."""
    xs, ws = _split(x), [w[i] for i in range(4)]
    bs = [None] * 4 if bias is None else [bias[i] for i in range(4)]
    mm = lambda a, b, c: torch.addmm(c, a, b) if c is not None else a @ b
    if variant8:
        xl, wl = _lanes_x(xs), _lanes_w(ws)
        L = [mm(xl[i], wl[i], bs[i - 4] if i >= 4 else None) for i in range(8)]
        return torch.cat(_recompose_y(L), 0)
    ys = []
    for dim in range(4):
        row = SIGNTABLE[4 * dim:4 * dim + 4]
        y = mm(xs[row[0][0]], ws[row[0][1]], bs[dim])
        for (l, r, pos) in row[1:]:
            buf = xs[l] @ ws[r]
            y = y + buf if pos else y - buf
        ys.append(y)
    return torch.cat(ys, 0)


def dense_bwd(x, w, dy, variant8, need_dx=True):
    xs, ws, gs = _split(x), [w[i] for i in range(4)], _split(dy)
    if variant8:
        xl, wl, gl = _lanes_x(xs), _lanes_w(ws), _lanes_g(gs)
        dw = torch.stack(_recompose_dw([xl[i].t() @ gl[i] for i in range(8)]), 0)
        dx = torch.cat(_recompose_dx([gl[i] @ wl[i].t() for i in range(8)]), 0) if need_dx else None
        return dw, dx
    dws, dxs = [None] * 4, [None] * 4
    for i, j in enumerate(BACKPROP_ORDER):
        l, r, pos = SIGNTABLE[j]
        dim = j // 4
        bw = xs[l].t() @ gs[dim]
        bx = gs[dim] @ ws[r].t() if need_dx else None
        if i < 4:
            dws[r], dxs[l] = bw, bx
        else:
            dws[r] = dws[r] + bw if pos else dws[r] - bw
            if need_dx:
                dxs[l] = dxs[l] + bx if pos else dxs[l] - bx
    return torch.stack(dws, 0), (torch.cat(dxs, 0) if need_dx else None)
