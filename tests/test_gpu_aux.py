"""GPU tests of the harness's auxiliary batch-norm (+ ReLU) kernels against a float64 torch formulation."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(x, gamma, beta, dy, eps, relu):
    x = x.double().requires_grad_(True)
    gamma = gamma.double().requires_grad_(True)
    beta = beta.double().requires_grad_(True)
    mean = x.mean(dim=(0, 2, 3), keepdim=True)
    var = x.var(dim=(0, 2, 3), unbiased=False, keepdim=True)
    y = (x - mean) / torch.sqrt(var + eps) * gamma.view(1, -1, 1, 1) + beta.view(1, -1, 1, 1)
    if relu:
        y = y.clamp_min(0)
    y.backward(dy.double())
    return y.detach(), x.grad, gamma.grad, beta.grad


@pytest.mark.parametrize("shape", [(8, 16, 12, 12), (12, 5, 7, 7), (4, 64, 14, 14), (16, 3, 6, 10), (8, 6, 7, 7), (16, 128, 7, 7), (8, 3, 3, 3)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("relu", [False, True])
def test_bn_relu_helpers(shape, dtype, relu):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from phoenix_core_b200.qresnet import _BNReLUFn
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(shape, generator=g) * 1.5 + 0.3).to(dtype).cuda()
    gamma = (torch.rand(shape[1], generator=g) + 0.5).cuda().requires_grad_(True)
    beta = (torch.randn(shape[1], generator=g) * 0.2).cuda().requires_grad_(True)
    dy = torch.randn(shape, generator=g).to(dtype).cuda()
    xin = x.clone().requires_grad_(True)
    y = _BNReLUFn.apply(xin, gamma, beta, 1e-5, relu)
    y.backward(dy)
    ry, rdx, rdg, rdb = _ref(x.cpu().float(), gamma.detach().cpu(), beta.detach().cpu(), dy.cpu().float(), 1e-5, relu)
    tol = 2e-2

    def err(a, b):
        return float((a.detach().cpu().double() - b).abs().max() / b.abs().max().clamp_min(1e-12))

    assert err(y, ry) < tol
    # the ReLU mask of the reference is taken from the float64 output; outputs within rounding of zero may differ
    assert err(xin.grad, rdx) < 5e-2
    assert err(gamma.grad, rdg) < tol
    assert err(beta.grad, rdb) < tol


@pytest.mark.parametrize("shape", [(8, 16, 12, 12), (12, 5, 7, 7), (4, 64, 14, 14), (16, 3, 6, 10), (8, 6, 7, 7), (16, 128, 7, 7)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_bn_add_relu_helper(shape, dtype):
    """relu(batch_norm(x) + residual) in the batch-norm's own passes, and its three gradients, against float64."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from phoenix_core_b200.qresnet import BNReLU
    g = torch.Generator().manual_seed(6)
    x = (torch.randn(shape, generator=g) * 1.5 + 0.3).to(dtype).cuda()
    res = torch.randn(shape, generator=g).to(dtype).cuda()
    dy = torch.randn(shape, generator=g).to(dtype).cuda()
    bn = BNReLU(shape[1], torch.device("cuda"), relu=False)
    with torch.no_grad():
        bn.weight.copy_((torch.rand(shape[1], generator=g) + 0.5).cuda())
        bn.bias.copy_((torch.randn(shape[1], generator=g) * 0.2).cuda())
    xin, rin = x.clone().requires_grad_(True), res.clone().requires_grad_(True)
    y = bn.add_relu(xin, rin)
    y.backward(dy)

    xr, rr = x.cpu().double().requires_grad_(True), res.cpu().double().requires_grad_(True)
    gr, br = bn.weight.detach().cpu().double().requires_grad_(True), bn.bias.detach().cpu().double().requires_grad_(True)
    mean = xr.mean(dim=(0, 2, 3), keepdim=True)
    var = xr.var(dim=(0, 2, 3), unbiased=False, keepdim=True)
    yr = ((xr - mean) / torch.sqrt(var + 1e-5) * gr.view(1, -1, 1, 1) + br.view(1, -1, 1, 1) + rr).clamp_min(0)
    yr.backward(dy.cpu().double())

    def err(a, b):
        return float((a.detach().cpu().double() - b).abs().max() / b.abs().max().clamp_min(1e-12))

    assert err(y, yr.detach()) < 2e-2
    # the mask of the float64 formulation is taken from its own output; outputs within rounding of zero may differ
    assert err(xin.grad, xr.grad) < 5e-2
    assert err(rin.grad, rr.grad) < 5e-2 or float(((rin.grad.cpu().double() - rr.grad).abs() > 1e-2).double().mean()) < 2e-3
    assert err(bn.weight.grad, gr.grad) < 2e-2
    assert err(bn.bias.grad, br.grad) < 2e-2


@pytest.mark.parametrize("shape", [(8, 16, 12, 16), (4, 5, 6, 8), (2, 3, 16, 24), (4, 16, 112, 112)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_bn_relu_maxpool_helper(shape, dtype):
    """The fused stem tail against the two separate helpers (batch-norm + ReLU, then max-pool): the same pooled values to
    within a unit in the last place; the same gradients except where two window elements tie after rounding to the storage type (the separate form stores the
    normalised tensor in 16 bits before pooling, the fused form compares in fp32)."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from phoenix_core_b200.qresnet import BNReLU, max_pool_3x3_s2
    g = torch.Generator().manual_seed(8)
    x = (torch.randn(shape, generator=g) * 1.5 + 0.3).to(dtype).cuda()
    outs = []
    for fused in (True, False):
        bn = BNReLU(shape[1], torch.device("cuda"), relu=True)
        gg = torch.Generator().manual_seed(9)
        with torch.no_grad():
            bn.weight.copy_((torch.rand(shape[1], generator=gg) + 0.5).cuda())
            bn.bias.copy_((torch.randn(shape[1], generator=gg) * 0.2).cuda())
        xin = x.clone().requires_grad_(True)
        y = bn.relu_pool(xin) if fused else max_pool_3x3_s2(bn(xin))
        dy = torch.randn(y.shape, generator=gg).to(dtype).cuda()
        y.backward(dy)
        outs.append((y.detach().float(), xin.grad.float(), bn.weight.grad.clone(), bn.bias.grad.clone()))
    (yf, dxf, dgf, dbf), (ys, dxs, dgs, dbs) = outs
    # the statistics are summed with atomics, so mean and 1/std can differ in their last bits between two runs
    assert yf.shape == ys.shape and float((yf - ys).abs().max()) <= 4e-3 * float(ys.abs().max())
    differing = float(((dxf - dxs).abs() > 1e-3 * dxs.abs().max()).float().mean())
    # ties after rounding are rare in fp16 and common in bf16 (8 bits of mantissa)
    assert differing < (1e-2 if dtype == torch.float16 else 6e-2), differing
    assert float((dgf - dgs).abs().max() / dgs.abs().max()) < 2e-2
    assert float((dbf - dbs).abs().max() / dbs.abs().max()) < 2e-2


@pytest.mark.parametrize("shape", [(8, 16, 12, 12), (4, 5, 9, 7), (2, 3, 16, 11), (2, 3, 16, 24), (1, 2, 112, 112), (3, 2, 9, 8)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_maxpool_helpers(shape, dtype):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from phoenix_core_b200.qresnet import max_pool_3x3_s2
    g = torch.Generator().manual_seed(9)
    x = torch.randn(shape, generator=g).to(dtype).cuda()
    xin = x.clone().requires_grad_(True)
    y = max_pool_3x3_s2(xin)
    xref = x.clone().float().requires_grad_(True)
    yref = torch.nn.functional.max_pool2d(xref, 3, 2, 1)
    assert y.shape == yref.shape and torch.equal(y.float(), yref)
    dy = torch.randn(y.shape, generator=g).to(dtype).cuda()
    y.backward(dy)
    yref.backward(dy.float())
    # random data has no ties inside a window, so the arg-max is unique
    assert torch.allclose(xin.grad.float(), xref.grad, atol=2e-2, rtol=2e-2)


def test_clock_probe_reports_a_plausible_sm_clock():
    """The measurement aid: a million SM cycles against the device's nanosecond timer, and its argument checks."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import ctypes
    from phoenix_core_b200 import _lib
    L = _lib.lib()
    out = torch.zeros(2, dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert L.pcb_aux_clock_probe(1000000, ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(stream)) == _lib.PCB_OK
    torch.cuda.synchronize()
    cycles, ns = out.tolist()
    assert 1000000 <= cycles < 1100000 and ns > 0
    assert 300 < cycles / ns * 1e3 < 3000            # MHz
    assert L.pcb_aux_clock_probe(0, ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(stream)) == _lib.PCB_ERR_INVALID_ARGUMENT
    assert L.pcb_aux_clock_probe(1000, None, ctypes.c_void_p(stream)) == _lib.PCB_ERR_INVALID_ARGUMENT
