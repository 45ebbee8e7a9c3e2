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


@pytest.mark.parametrize("shape", [(8, 16, 12, 12), (12, 5, 7, 7), (4, 64, 14, 14), (16, 3, 6, 10)])
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
