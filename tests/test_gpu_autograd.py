"""The public PyTorch autograd front end (phoenix_core_b200.autograd) against the float64 block form: a layer's output,
and the gradients autograd hands back for the input, the filters and the bias."""
import numpy as np
import pytest
import torch

from helpers import conv_bwd_f64, conv_fwd_f64, dense_bwd_f64, dense_fwd_f64, normal, rel_err, uniform

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 2e-2), (torch.float32, 1e-5)])
def test_conv_function_gradients(dtype, tol):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import phoenix_core_b200 as pcb
    from phoenix_core_b200.autograd import QConv2dFunction
    n, ci, co, h, w_, k = 2, 8, 16, 9, 7, 3
    to = lambda a: torch.from_numpy(a).to(dtype)
    xh, wh, bh = to(uniform(1, (4 * n, ci, h, w_))), to(uniform(2, (4, co, ci, k, k)) * 0.2), to(uniform(3, (4, co)))
    x = xh.cuda().requires_grad_(True)
    w = wh.cuda().requires_grad_(True)
    b = bh.cuda().requires_grad_(True)
    y = QConv2dFunction.apply(x, w, b, 2, 1, pcb.Padding.SAME)
    out, pb, pa = zip(*[pcb.compute_windowed_output_size_and_padding(s, k, 1, 2, pcb.Padding.SAME) for s in (h, w_)])
    pad = (pb[0], pb[1], pa[0], pa[1])
    ref = conv_fwd_f64(xh.float().numpy(), wh.float().numpy(), bh.float().numpy(), (2, 2), pad)
    assert tuple(y.shape) == ref.shape
    assert rel_err(y.detach().float().cpu().numpy(), ref) <= tol
    gh = to(normal(4, ref.shape))
    y.backward(gh.cuda())
    rdw, rdx = conv_bwd_f64(xh.float().numpy(), wh.float().numpy(), gh.float().numpy(), (2, 2), pad)
    assert rel_err(w.grad.float().cpu().numpy(), rdw) <= tol
    assert rel_err(x.grad.float().cpu().numpy(), rdx) <= tol
    rdb = gh.float().numpy().reshape(4, n, co, -1).sum(axis=(1, 3))
    assert rel_err(b.grad.float().cpu().numpy(), rdb) <= tol


@pytest.mark.parametrize("oi", [False, True])
def test_dense_function_gradients(oi):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import phoenix_core_b200 as pcb
    from phoenix_core_b200.autograd import QDenseFunction
    b_, i, o = 6, 40, 24
    xh, bh = normal(11, (4 * b_, i)), uniform(13, (4, o))
    wh = normal(12, (4, o, i) if oi else (4, i, o), std=0.1)
    x = torch.from_numpy(xh).cuda().requires_grad_(True)
    w = torch.from_numpy(wh).cuda().requires_grad_(True)
    b = torch.from_numpy(bh).cuda().requires_grad_(True)
    y = QDenseFunction.apply(x, w, b, pcb.Algebra.QUATERNION, pcb.FilterLayout.OI if oi else pcb.FilterLayout.IO)
    assert rel_err(y.detach().cpu().numpy(), dense_fwd_f64(xh, wh, bh, oi)) <= 1e-5
    gh = normal(14, (4 * b_, o))
    y.backward(torch.from_numpy(gh).cuda())
    rdw, rdx = dense_bwd_f64(xh, wh, gh, oi)                 # [4, I, O] whatever the layout
    want_dw = np.swapaxes(rdw, 1, 2) if oi else rdw           # the gradient has the shape of the parameter
    assert tuple(w.grad.shape) == wh.shape
    assert rel_err(w.grad.cpu().numpy(), want_dw) <= 1e-5
    assert rel_err(x.grad.cpu().numpy(), rdx) <= 1e-5
    assert rel_err(b.grad.cpu().numpy(), gh.reshape(4, b_, o).sum(1)) <= 1e-5


def test_modules_train_one_step():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from phoenix_core_b200.autograd import QConv2d, QDense
    torch.manual_seed(0)
    conv, fc = QConv2d(8, 16, 3), QDense(16, 5)
    x = torch.randn(4 * 3, 8, 10, 10, device="cuda", dtype=torch.float16)
    y = conv(x).relu().view(4, 3, 16, 100).mean(-1).view(12, 16)      # global average pool per component
    loss = fc(y).float().pow(2).mean()
    loss.backward()
    for p in list(conv.parameters()) + list(fc.parameters()):
        assert p.grad is not None and torch.isfinite(p.grad).all()
