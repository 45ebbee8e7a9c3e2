"""The bounded device-side waits: a wait that runs out is reported, never a hang, and the report survives the call.

Every tensor-core kernel bounds its barrier waits; on expiry it sets a bit in the status word at the head of the
workspace and leaves through its normal teardown. Each API call clears the word once and kernels only OR into it.
The expiry here is made in the only permitted way: a self-test kernel waits a few thousand clocks on a barrier that
nothing signals and then returns -- no trap, no fault, no endless loop.
"""
import ctypes

import numpy as np
import pytest
import torch

from helpers import rel_err, uniform

pytestmark = pytest.mark.gpu


def _fwd_desc(_lib, n, ci, co, h, w, engine):
    return _lib.ConvDesc(dtype=_lib.PCB_F32, n=n, ci=ci, co=co, h=h, w=w, kh=1, kw=1, stride_h=1, stride_w=1, dilation_h=1,
                         dilation_w=1, groups=1, engine=engine)


def test_expired_wait_is_reported_and_survives_later_launches_of_the_call(oracle):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from phoenix_core_b200 import _lib
    L = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    x = uniform(1, (4 * 2, 3, 5, 4))
    w = uniform(2, (4, 2, 3, 1, 1))
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    y = torch.full((4 * 2, 2, 5, 4), float("nan"), device="cuda")
    d = _fwd_desc(_lib, 2, 3, 2, 5, 4, _lib.ENGINE_SIMT)
    ws = torch.zeros(max(L.pcb_qconv2d_fwd_workspace_size(ctypes.byref(d)), 4096), dtype=torch.uint8, device="cuda")

    # clean workspace: ok
    assert L.pcb_check_device_status(ws.data_ptr(), ws.numel(), stream) == _lib.PCB_OK
    # 1. the wait runs out (2^12 clocks, a few microseconds); the kernel returns and the word is set
    _lib.check(L.pcb_selftest_wait_expiry(None, None, None, None, ws.data_ptr(), ws.numel(), 1 << 12, stream))
    assert L.pcb_check_device_status(ws.data_ptr(), ws.numel(), stream) == _lib.PCB_ERR_DEVICE_TIMEOUT
    assert b"wait expired" in L.pcb_last_error_message()
    # 2. a second launch inside the same call (a forward pass) must not erase the record
    _lib.check(L.pcb_selftest_wait_expiry(ctypes.byref(d), xd.data_ptr(), wd.data_ptr(), y.data_ptr(), ws.data_ptr(), ws.numel(),
                                          1 << 12, stream))
    assert L.pcb_check_device_status(ws.data_ptr(), ws.numel(), stream) == _lib.PCB_ERR_DEVICE_TIMEOUT
    ref = oracle.conv2d_fwd(x, w)
    assert rel_err(y.cpu().numpy(), ref) <= 1e-5          # that launch itself ran to completion
    # 3. the context is intact and the next ordinary call on the same workspace starts clean and is correct
    y.fill_(float("nan"))
    _lib.check(L.pcb_qconv2d_fwd(ctypes.byref(d), xd.data_ptr(), wd.data_ptr(), None, y.data_ptr(), ws.data_ptr(), ws.numel(), stream))
    assert L.pcb_check_device_status(ws.data_ptr(), ws.numel(), stream) == _lib.PCB_OK
    assert rel_err(y.cpu().numpy(), ref) <= 1e-5


def test_backward_call_keeps_one_status_for_both_of_its_launches(oracle):
    """pcb_qconv2d_bwd runs the filter gradient and then backward-data on one workspace; after a clean call on the
    tensor-core kernels the word reads ok, and the Python layer's Device.checkStatus reads the same word."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util
    import phoenix_core_b200 as pcb
    from phoenix_core_b200.ops import Device
    x = gpu_util.rounded(uniform(3, (4 * 2, 32, 8, 8)), "f16")
    w = gpu_util.rounded(uniform(4, (4, 32, 32, 1, 1)) * 0.1, "f16")
    dy = gpu_util.rounded(uniform(5, (4 * 2, 32, 8, 8)), "f16")
    dw, dx = gpu_util.run_conv_bwd(x, w, dy, (1, 1), (0, 0, 0, 0), "f16", "16p", "tensor")
    Device.get(torch.device("cuda", torch.cuda.current_device())).checkStatus()      # raises on a recorded expiry
    rdw, rdx = oracle.conv2d_bwd(x, w, dy)
    assert rel_err(dw, rdw) <= 2e-2 and rel_err(dx, rdx) <= 2e-2


def test_selftest_rejects_unbounded_limits():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from phoenix_core_b200 import _lib
    L = _lib.lib()
    ws = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    assert L.pcb_selftest_wait_expiry(None, None, None, None, ws.data_ptr(), ws.numel(), 1 << 40, None) == _lib.PCB_ERR_INVALID_ARGUMENT
    assert L.pcb_selftest_wait_expiry(None, None, None, None, None, 0, 1 << 12, None) == _lib.PCB_ERR_WORKSPACE
