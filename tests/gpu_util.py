"""Helpers for the GPU parity tests: run one operator through the product path (torch tensors -> C ABI ->
CUDA kernels) and through the CPU oracle on the same seeded inputs."""
import numpy as np
import torch

import phoenix_core_b200 as pcb
from phoenix_core_b200 import _lib
from phoenix_core_b200.context import Context

TORCH_DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
# tolerances of the parity contract: max|got-ref| / max|ref| per output tensor
TOL = {"f32": 1e-5, "f16": 2e-2, "bf16": 2e-2}
ENGINES = {"auto": _lib.ENGINE_AUTO, "simt": _lib.ENGINE_SIMT, "tensor": _lib.ENGINE_TENSOR}


def context(variant):
    """variant: '16p' (UPSTRIDE_MEMORY_OPTIMIZED=1) or '8p' (the reference default)."""
    return Context({"UPSTRIDE_MEMORY_OPTIMIZED": "1" if variant == "16p" else "0"})


def rounded(a, dtype):
    """Rounds a float32 numpy array to the storage dtype and back (the oracle sees what the GPU sees)."""
    t = torch.from_numpy(np.ascontiguousarray(a)).to(TORCH_DTYPES[dtype])
    return t.to(torch.float32).numpy()


def dev(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a)).to(TORCH_DTYPES[dtype]).cuda().contiguous()


def host(t):
    torch.cuda.synchronize()
    return t.detach().to(torch.float32).cpu().numpy()


def conv_descriptors(xshape, wshape, stride, pad, use_bias, need_dx, real_input=False, algebra=pcb.Algebra.QUATERNION,
                     dilation=(1, 1), groups=1):
    pt, pl, pb, pr = pad
    args = (xshape, wshape, stride, dilation, pcb.Padding.EXPLICIT, (pt, pl, pb, pr), groups, algebra,
            pcb.DataFormat.NCHW, pcb.FilterLayout.OIHW)
    fwd = pcb.Conv2DFwdDescriptor(*args, use_bias, real_input)
    bwd = pcb.Conv2DBwdDescriptor(*args, need_dx, real_input)
    return fwd, bwd


def run_conv_fwd(x, w, bias, stride, pad, dtype, variant, engine, real_input=False, algebra=pcb.Algebra.QUATERNION,
                 dilation=(1, 1), groups=1):
    fwd, _ = conv_descriptors(x.shape, w.shape, stride, pad, bias is not None, False, real_input, algebra, dilation, groups)
    xd, wd = dev(x, dtype), dev(w, dtype)
    bd = None if bias is None else dev(bias, dtype)
    y = torch.full(fwd.getOutputShape(), float("nan"), dtype=TORCH_DTYPES[dtype], device="cuda")
    pcb.conv2DFwd(xd, wd, bd, y, fwd, context(variant), ENGINES[engine])
    return host(y)


def run_conv_bwd(x, w, dy, stride, pad, dtype, variant, engine, need_dx=True, algebra=pcb.Algebra.QUATERNION, dilation=(1, 1), groups=1):
    _, bwd = conv_descriptors(x.shape, w.shape, stride, pad, False, need_dx, False, algebra, dilation, groups)
    xd, wd, gd = dev(x, dtype), dev(w, dtype), dev(dy, dtype)
    dw = torch.full(w.shape, float("nan"), dtype=TORCH_DTYPES[dtype], device="cuda")
    dx = torch.full(x.shape, float("nan"), dtype=TORCH_DTYPES[dtype], device="cuda") if need_dx else None
    pcb.conv2DBwd(xd, wd, gd, dw, dx, bwd, context(variant), ENGINES[engine])
    return host(dw), (host(dx) if need_dx else None)


def run_dense_fwd(x, w, bias, oi, dtype, variant, engine, algebra=pcb.Algebra.QUATERNION):
    layout = pcb.FilterLayout.OI if oi else pcb.FilterLayout.IO
    desc = pcb.DenseFwdDescriptor(x.shape, w.shape, algebra, layout, bias is not None)
    xd, wd = dev(x, dtype), dev(w, dtype)
    bd = None if bias is None else dev(bias, dtype)
    y = torch.full(desc.getOutputShape(), float("nan"), dtype=TORCH_DTYPES[dtype], device="cuda")
    pcb.denseFwd(xd, wd, bd, y, desc, context(variant), ENGINES[engine])
    return host(y)


def run_dense_bwd(x, w, dy, oi, dtype, variant, engine, need_dx=True, algebra=pcb.Algebra.QUATERNION):
    layout = pcb.FilterLayout.OI if oi else pcb.FilterLayout.IO
    desc = pcb.DenseBwdDescriptor(x.shape, w.shape, algebra, layout, need_dx)
    xd, wd, gd = dev(x, dtype), dev(w, dtype), dev(dy, dtype)
    i, o = desc.getInputChannels(), desc.getOutputChannels()
    dwshape = (i, o) if algebra == pcb.Algebra.REAL else (w.shape[0], i, o)
    dw = torch.full(dwshape, float("nan"), dtype=TORCH_DTYPES[dtype], device="cuda")
    dx = torch.full(x.shape, float("nan"), dtype=TORCH_DTYPES[dtype], device="cuda") if need_dx else None
    pcb.denseBwd(xd, wd, gd, dw, dx, desc, context(variant), ENGINES[engine])
    return host(dw), (host(dx) if need_dx else None)
