"""Benchmark of the quaternion conv2d hot path: forward + backward of the pointwise configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step" = forward, backward-filter and backward-data of one batch): pointwise 1x1 quaternion
conv2d, fp16 in/out, batch 64 per GPU, 128 -> 256 quaternion channels, 56x56, stride 1, NCHW, 16-product
formulation on the tcgen05 kernels; activations N(0,1), weights He-normal, seeded synthetic data.
Work per step and GPU: 3 passes x 32*N*H*W*Co*Ci = 631.4 GFLOP. Under torchrun every rank runs its own
batch (weak scaling) and the filter gradient is summed across ranks with one NCCL all-reduce per step, started on
a side stream as soon as the filter gradient is enqueued so that it runs beside backward-data.

Prints one JSON line:
  value          device-timed throughput with inputs resident in HBM
  parity         relative errors of the timed tensors themselves (batch 64) against the CPU checker
  roofline       the slowest of the three kernels, timed alone for >= 2 s of back-to-back launches against the measured
                 SUSTAINED tensor peak (and the same kernel in a short window against the BURST peak), with the SM
                 clock sampled during each
  e2e            the same metric through the public API from pinned host buffers, with a plain pinned-copy
                 roofline of the same byte counts timed beside it
  eight_product  the factorised 8-product formulation of the same step on its own tcgen05 kernels
  dense          the quaternion dense configuration (batch 256, 512 -> 512, fp32) forward + backward
  sweep          the ResNet-stage shape sweep (batch 128, fp16): every pass of every shape
  sweep_f32      the same sweep in fp32 (error-compensated TF32 kernels), with the executed-TF32 fraction
  qresnet18      images/s of a quaternion ResNet-18 training step (batch 128 per GPU, 224x224, fp16, data-parallel)
  cpu_baseline   the reference's CPU orchestration (8-product default and 16-product) over oneDNN via torch CPU
                 ops on a bounded sample, on the box's host cores
`--impl reference` times only that CPU orchestration.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD = dict(n=64, ci=128, co=256, h=56, w=56)
SEED = 1234
STAGES = [(16, 112), (64, 56), (128, 28), (256, 14), (512, 7)]     # quaternion channels @ plane size of the sweep


def flops_per_pass(n, ci, co, h, w):
    return 32.0 * n * h * w * co * ci


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], tflops_burst=p["bf16_tflops"], tflops_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only) from a thread while the timed region
    runs; falls back to one nvidia-smi query if NVML is not importable."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.samples, self.reason_bits, self.max_mhz = [], 0, None
        self._stop = False
        self._thread = None

    def _loop(self, nvml, handle):
        while not self._stop:
            try:
                self.samples.append(nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM))
                get = getattr(nvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or nvml.nvmlDeviceGetCurrentClocksThrottleReasons
                self.reason_bits |= int(get(handle))
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        import threading
        try:
            import pynvml as nvml
            nvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = self.gpu_index
            if visible:
                try:
                    index = int(visible.split(",")[self.gpu_index])
                except ValueError:
                    index = self.gpu_index
            handle = nvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM)
            self._thread = threading.Thread(target=self._loop, args=(nvml, handle), daemon=True)
            self._thread.start()
        except Exception:
            self._thread = None
        return self

    def stop(self):
        if self._thread is not None:
            self._stop = True
            self._thread.join(timeout=2)
            reasons = sorted(name for bit, name in self.REASONS.items() if self.reason_bits & bit)
            return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                    "samples": len(self.samples), "reasons": reasons, "source": "nvml"}
        try:
            out = subprocess.run(["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=clocks.sm,clocks.max.sm",
                                  "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=20).stdout
            a, b = [float(v) for v in out.strip().split(",")[:2]]
            return {"sm_mhz": a, "sm_max_mhz": b, "samples": 1, "reasons": [], "source": "nvidia-smi after the run"}
        except Exception:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["clock query unavailable"]}


def make_inputs(torch, n, ci, co, h, w, device, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn((4 * n, ci, h, w), generator=g, dtype=torch.float32).to(torch.float16)
    wt = (torch.randn((4, co, ci, 1, 1), generator=g, dtype=torch.float32) * (2.0 / (4 * ci)) ** 0.5).to(torch.float16)
    dy = torch.randn((4 * n, co, h, w), generator=g, dtype=torch.float32).to(torch.float16)
    if device is None:
        return x, wt, dy
    return x.to(device), wt.to(device), dy.to(device)


def cpu_baseline(torch, sample_n, reps, speed_over_memory=True):
    """The reference's CPU orchestration over oneDNN (its default 8-product form, or the 16-product form of
    UPSTRIDE_MEMORY_OPTIMIZED=1), fp32, all host cores, on a reduced batch of the same layer.
    Returns (TFLOP/s, cores, description, seconds per step)."""
    from oracle import ref_orchestration as ro
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x, wt, dy = make_inputs(torch, sample_n, WORKLOAD["ci"], WORKLOAD["co"], WORKLOAD["h"], WORKLOAD["w"], None, SEED)
    x, wt, dy = x.float(), wt.float(), dy.float()
    pad, stride = (0, 0, 0, 0), (1, 1)
    times = []
    for r in range(reps + 1):
        t0 = time.perf_counter()
        ro.conv2d_fwd(x, wt, None, stride, pad, speed_over_memory)
        ro.conv2d_bwd(x, wt, dy, stride, pad, speed_over_memory, True)
        if r > 0:
            times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    fl = 3 * flops_per_pass(sample_n, WORKLOAD["ci"], WORKLOAD["co"], WORKLOAD["h"], WORKLOAD["w"])
    sample = ("batch %d of the same layer (fp32, %s orchestration, torch CPU ops = oneDNN), median of %d steps"
              % (sample_n, "8-product" if speed_over_memory else "16-product", reps))
    return fl / t / 1e12, cores, sample, t


def run_reference(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    reps = max(1, args.steps)
    value, cores, sample, t = cpu_baseline(torch, args.cpu_sample, reps, True)
    v16, _, sample16, _ = cpu_baseline(torch, args.cpu_sample, max(1, min(reps, 5)), False)
    line = {
        "impl": "reference", "metric": "quaternion conv2d fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": reps, "warmup": 1, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "pointwise 1x1 quaternion conv2d fwd+bwd, 128->256 ch, 56x56 (CPU sample: batch %d)" % args.cpu_sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample,
                         "sixteen_product": {"value": v16, "unit": "TFLOP/s", "sample": sample16}},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def event_time(torch, fn, reps, warm=1):
    """Mean milliseconds of `fn` over `reps` back-to-back launches on the current stream (CUDA events)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


class ClockProbe:
    """The clock the SMs really run at while other kernels execute: the library's one-thread probe kernel, launched on a second
    stream in the middle of a timed loop, counts a million of its own cycles against the device's nanosecond timer. (NVML's
    clock is sampled every few hundred milliseconds; the power cap pulls the clock down within a burst of launches.)"""

    def __init__(self, torch, lib, cycles=1000000):
        self.torch, self.lib, self.cycles = torch, lib, cycles
        self.out = torch.zeros(2, dtype=torch.int64, device=torch.device("cuda", torch.cuda.current_device()))
        self.stream = torch.cuda.Stream()

    def launch(self):
        self.lib.pcb_aux_clock_probe(self.cycles, ctypes.c_void_p(self.out.data_ptr()), ctypes.c_void_p(self.stream.cuda_stream))

    def mhz(self):
        self.stream.synchronize()
        c, ns = self.out.tolist()
        return round(c / ns * 1e3) if ns > 0 else None


def event_time_probed(torch, fn, reps, probe, warm=1):
    """event_time with the clock probe launched beside the middle of the loop; returns (ms, effective SM MHz)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(reps):
        fn()
        if i == reps // 2:
            probe.launch()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps, probe.mhz()


def check_parity(torch, x, wt, dy, y, dw, dx, n):
    """Compares the tensors the timed steps produced with the CPU checker: y and dx on three whole images against the
    direct-loop oracle, the full filter gradient against the float64 block form of the product (sixteen matrix
    products over all pixels of all images). Relative errors as max|got - ref| / max|ref|."""
    import numpy as np
    from oracle import oracle as orc
    orc.build()
    sel = sorted({0, n // 2, n - 1})
    rows = [c * n + i for c in range(4) for i in sel]
    xs, dys = x[rows].float().cpu().numpy(), dy[rows].float().cpu().numpy()
    wh = wt.float().cpu().numpy()
    y_ref = orc.conv2d_fwd(xs, wh)
    _, dx_ref = orc.conv2d_bwd(xs, wh, dys)

    def rel(got, ref):
        got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
        return float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-30))

    out = {"y": rel(y[rows].float().cpu().numpy(), y_ref), "dx": rel(dx[rows].float().cpu().numpy(), dx_ref)}
    # dW_r = sum over (l, d = l ^ r) of s(l, d) * x_l^T dy_d, in float64, image chunks bound the host memory
    neg = {(1, 0), (1, 2), (2, 0), (2, 3), (3, 0), (3, 1)}
    ci, co = wt.shape[2], wt.shape[1]
    ref = torch.zeros((4, co, ci), dtype=torch.float64)
    chunk = 8
    for i0 in range(0, n, chunk):
        i1 = min(n, i0 + chunk)
        xc = [x[c * n + i0:c * n + i1].to(torch.float64).cpu().permute(1, 0, 2, 3).reshape(ci, -1) for c in range(4)]
        gc = [dy[c * n + i0:c * n + i1].to(torch.float64).cpu().permute(1, 0, 2, 3).reshape(co, -1) for c in range(4)]
        for l in range(4):
            for d in range(4):
                r = l ^ d
                ref[r] += (-1.0 if (l, d) in neg else 1.0) * (gc[d] @ xc[l].T)
    out["dw"] = rel(dw.float().cpu().reshape(4, co, ci).numpy(), ref.numpy())
    out["checked"] = "y, dx: images %s of the timed batch vs the direct-loop oracle; dw: the full tensor vs the float64 block form" % sel
    out["tolerance"] = 2e-2
    out["ok"] = bool(max(out["y"], out["dx"], out["dw"]) <= 2e-2)
    return out


def dense_leg(torch, pcb, _lib, peaks):
    """Quaternion dense forward + backward at batch 256, 512 -> 512 (fp32 on the error-compensated TF32 kernels, and
    fp16): milliseconds, effective TFLOP/s (F = 32*B*I*O per pass, three passes) and, for fp32, the executed TF32 rate
    (three MMAs per product) against a TF32 cuBLAS GEMM timed in the same run."""
    from phoenix_core_b200.context import Context
    B, I, O = 256, 512, 512
    out = {"config": "batch %d, %d -> %d quaternion units, IO filters, bias, N(0,1) input and gradient, He-normal weights" % (B, I, O)}
    g = torch.Generator(device="cpu").manual_seed(SEED + 7)
    xh = torch.randn((4 * B, I), generator=g)
    wh = torch.randn((4, I, O), generator=g) * (2.0 / (4 * I)) ** 0.5
    gh = torch.randn((4 * B, O), generator=g)
    fl = 32.0 * B * I * O
    ctx = Context({"UPSTRIDE_MEMORY_OPTIMIZED": "1"})
    keep = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    a = torch.randn(8192, 8192, device="cuda"); b = torch.randn(8192, 8192, device="cuda"); c = torch.empty(8192, 8192, device="cuda")
    tf32_peak = 2.0 * 8192 ** 3 / (event_time(torch, lambda: torch.matmul(a, b, out=c), 10, 3) * 1e-3) / 1e12
    torch.backends.cuda.matmul.allow_tf32 = keep
    del a, b, c
    for name, tdt in (("f32", torch.float32), ("f16", torch.float16)):
        x, w, dy = xh.to(tdt).cuda(), wh.to(tdt).cuda(), gh.to(tdt).cuda()
        bias = torch.zeros((4, O), dtype=tdt, device="cuda")
        y, dw, dx = torch.empty((4 * B, O), dtype=tdt, device="cuda"), torch.empty_like(w), torch.empty_like(x)
        fd = pcb.DenseFwdDescriptor(tuple(x.shape), tuple(w.shape), pcb.Algebra.QUATERNION, pcb.FilterLayout.IO, True)
        bd = pcb.DenseBwdDescriptor(tuple(x.shape), tuple(w.shape), pcb.Algebra.QUATERNION, pcb.FilterLayout.IO, True)
        t_f = event_time(torch, lambda: pcb.denseFwd(x, w, bias, y, fd, ctx), 50, 3)
        t_b = event_time(torch, lambda: pcb.denseBwd(x, w, dy, dw, dx, bd, ctx), 50, 3)
        rec = {"fwd_ms": t_f, "bwd_ms": t_b, "effective_tflops": 3 * fl / ((t_f + t_b) * 1e-3) / 1e12}
        if name == "f32":
            rec["executed_tf32_tflops"] = 3 * rec["effective_tflops"]
            rec["tf32_peak_tflops_measured"] = tf32_peak
            rec["frac_of_tf32_peak"] = rec["executed_tf32_tflops"] / tf32_peak
        else:
            rec["frac_of_tensor_peak_burst"] = rec["effective_tflops"] / peaks["tflops_burst"]
        # HBM view: x + w + y in, dy + x + w in, dw + dx out (a dense layer this small lives in L2; reported for scale)
        eb = 4 if name == "f32" else 2
        rec["algorithmic_bytes"] = eb * (2 * x.numel() + 2 * w.numel() + 2 * y.numel() + dw.numel() + dx.numel())
        out[name] = rec
    return out


def sweep_leg(torch, pcb, _lib, peaks, reps=5, batch=128, only=None, layouts=("nchw",), extra_nhwc=((64, 56, 3, 1),), dtype="f16",
              tf32_peak=None):
    """The ResNet-stage sweep, fp16 or fp32: 3x3 (pad 1) and 1x1, stride 1 and 2, forward / backward-data / backward-filter of each
    shape timed separately (3 warm-up + `reps` launches, CUDA events; times include every staging kernel of the call).
    Inputs are seeded U[-1,1] generated on the device; every shape's tensors exceed the L2 or are rewritten each launch.
    `extra_nhwc`: shapes repeated with channels-last activations and OHWI filters (read in place by the tensor-core kernels).
    `only` = (c, hw, k, stride) restricts the sweep to one shape (profiling)."""
    from phoenix_core_b200.context import Context
    from phoenix_core_b200.ops import Device, _conv_desc, _ptr, _stream
    L = _lib.lib()
    ctx = Context({"UPSTRIDE_MEMORY_OPTIMIZED": "1"})
    dev = torch.device("cuda", torch.cuda.current_device())
    rows = []
    gen = torch.Generator(device=dev).manual_seed(SEED + 11)
    tdt = torch.float32 if dtype == "f32" else torch.float16
    eb = 4 if dtype == "f32" else 2
    cases = [(c, hw, k, s_, lay) for lay in layouts for c, hw in STAGES for k in (3, 1) for s_ in (1, 2)]
    cases += [(c, hw, k, s_, "nhwc") for c, hw, k, s_ in extra_nhwc if "nhwc" not in layouts]
    for c, hw, k, stride, layout in cases:
        if only is not None and tuple(only) != (c, hw, k, stride):
            continue
        pad = 1 if k == 3 else 0
        nhwc = layout == "nhwc"
        xshape = (4 * batch, hw, hw, c) if nhwc else (4 * batch, c, hw, hw)
        wshape = (4, c, k, k, c) if nhwc else (4, c, c, k, k)
        a = (xshape, wshape, stride, 1, pcb.Padding.EXPLICIT, (pad, pad, pad, pad), 1, pcb.Algebra.QUATERNION,
             pcb.DataFormat.NHWC if nhwc else pcb.DataFormat.NCHW, pcb.FilterLayout.OHWI if nhwc else pcb.FilterLayout.OIHW)
        fwd, bwd = pcb.Conv2DFwdDescriptor(*a, False), pcb.Conv2DBwdDescriptor(*a, True)
        x = (torch.rand(xshape, generator=gen, device=dev) * 2 - 1).to(tdt)
        w = (torch.rand(wshape, generator=gen, device=dev) * 2 - 1).to(tdt)
        y = torch.empty(fwd.getOutputShape(), dtype=tdt, device=dev)
        dy = (torch.rand(tuple(y.shape), generator=gen, device=dev) * 2 - 1).to(tdt)
        dw, dx = torch.empty_like(w), torch.empty_like(x)
        d = _conv_desc(bwd, tdt, ctx, _lib.ENGINE_AUTO, require_input_grad=True)
        ws = Device.get(dev).requestWorkspace(max(L.pcb_qconv2d_bwd_workspace_size(ctypes.byref(d)),
                                                  L.pcb_qconv2d_fwd_workspace_size(ctypes.byref(d))))
        ho = y.shape[1] if nhwc else y.shape[2]
        fl = 32.0 * batch * ho * ho * c * c * k * k
        xb, yb, wb = eb * x.numel(), eb * y.numel(), eb * w.numel()
        passes = (
            ("fwd", lambda: pcb.conv2DFwd(x, w, None, y, fwd, ctx), xb + yb + wb, 0),
            ("bwd_data", lambda: _lib.check(L.pcb_qconv2d_bwd_data(ctypes.byref(d), _ptr(w), _ptr(dy), _ptr(dx), _ptr(ws), ws.numel(), _stream())), yb + wb + xb, 1),
            ("bwd_filter", lambda: _lib.check(L.pcb_qconv2d_bwd_filter(ctypes.byref(d), _ptr(x), _ptr(dy), _ptr(dw), _ptr(ws), ws.numel(), _stream())), xb + yb + 2 * wb, 2),
        )
        for name, fn, nbytes, pid in passes:
            ms = event_time(torch, fn, reps, 3)
            row = {"c": c, "hw": hw, "k": k, "s": stride, "layout": layout, "dtype": dtype, "pass": name, "ms": round(ms, 4),
                   "tflops": round(fl / (ms * 1e-3) / 1e12, 1), "gbs": round(nbytes / (ms * 1e-3) / 1e9, 0),
                   "f_hbm": round(nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 3),
                   "engine": L.pcb_qconv2d_engine_for(ctypes.byref(d), pid)}
            if dtype == "f32":       # the fp32 kernels execute three TF32 MMAs per product
                if tf32_peak:
                    row["f_tf32_executed"] = round(3 * fl / (ms * 1e-3) / 1e12 / tf32_peak, 3)
            else:
                row["f_tensor"] = round(fl / (ms * 1e-3) / 1e12 / peaks["tflops_sustained"], 3)
            rows.append(row)
        _lib.check(L.pcb_check_device_status(_ptr(ws), ws.numel(), _stream()))
        del x, w, y, dy, dw, dx
        torch.cuda.empty_cache()
    return {"config": "batch %d, %s, 16-product, U[-1,1]; layout nchw = NCHW activations + OIHW filters, nhwc = channels-last activations "
                      "+ OHWI filters; f_tensor against the sustained tensor peak (fp16), f_tf32_executed = 3 x FLOPs / time against a TF32 "
                      "cuBLAS GEMM timed in this run (fp32: three TF32 MMAs per product), f_hbm = algorithmic bytes / time against the "
                      "copy bandwidth; engine 2 = tcgen05, 1 = CUDA cores" % (batch, "fp32" if dtype == "f32" else "fp16"),
            "reps": reps, "rows": rows}


def run_ours(args):
    import torch
    import torch.distributed as dist
    import phoenix_core_b200 as pcb
    from phoenix_core_b200 import _lib
    from phoenix_core_b200.context import Context
    from phoenix_core_b200.ops import Device, _conv_desc, _ptr, _stream

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    if args.sweep_only:            # profiling: one leg of the record on its own, e.g. one shape for an ncu capture
        only = tuple(int(v) for v in args.sweep_shape.split(",")) if args.sweep_shape else None
        out = sweep_leg(torch, pcb, _lib, read_peaks(), reps=args.sweep_reps, batch=args.sweep_batch, only=only,
                        layouts=(args.sweep_layout,), extra_nhwc=(), dtype=args.sweep_dtype)
        print(json.dumps(out), flush=True)
        return
    if args.dense_only:
        print(json.dumps(dense_leg(torch, pcb, _lib, read_peaks())), flush=True)
        return

    n, ci, co, h, w = (WORKLOAD[k] for k in ("n", "ci", "co", "h", "w"))
    ctx16 = Context({"UPSTRIDE_MEMORY_OPTIMIZED": "1", "UPSTRIDE_CONV_FP16_POLICY": "full16"})
    main_engine = _lib.ENGINE_AUTO
    if args.formulation == "8p":   # profiling: the factorised tensor-core kernels as the main step (the line is marked)
        ctx16 = Context({"UPSTRIDE_MEMORY_OPTIMIZED": "0", "UPSTRIDE_CONV_FP16_POLICY": "full16"})
        main_engine = _lib.ENGINE_TENSOR
    if args.engine != "auto":
        main_engine = _lib.ENGINE_SIMT if args.engine == "simt" else _lib.ENGINE_TENSOR
    args_d = ((4 * n, ci, h, w), (4, co, ci, 1, 1), (1, 1), (1, 1), pcb.Padding.VALID, (), 1, pcb.Algebra.QUATERNION,
              pcb.DataFormat.NCHW, pcb.FilterLayout.OIHW)
    fwd_desc = pcb.Conv2DFwdDescriptor(*args_d, False)
    bwd_desc = pcb.Conv2DBwdDescriptor(*args_d, True)

    x, wt, dy = make_inputs(torch, n, ci, co, h, w, device, SEED + rank)
    y = torch.empty(fwd_desc.getOutputShape(), dtype=torch.float16, device=device)
    dw = torch.empty_like(wt)
    dx = torch.empty_like(x)
    comm = torch.cuda.Stream(priority=-1) if world > 1 else None
    pending = []
    # data-parallel runs leave a few SMs free of the persistent kernels so that the all-reduce's kernel runs beside backward-data
    sm_margin = args.sm_margin if args.sm_margin is not None else (2 if world > 1 else 0)
    pcb.setSmMargin(sm_margin)

    def start_allreduce(grad):
        # the filter gradient is complete once the kernels enqueued so far have run: sum it across ranks on the side
        # stream while backward-data (which does not read it) runs on this one
        comm.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(comm):
            pending.append(dist.all_reduce(grad, async_op=True))

    def step():
        pcb.conv2DFwd(x, wt, None, y, fwd_desc, ctx16, main_engine)
        if world > 1:
            pcb.conv2DBwd(x, wt, dy, dw, dx, bwd_desc, ctx16, main_engine, on_filter_grad=start_allreduce)
            pending.pop().wait()                      # the current stream waits for the sum; the host does not block
        else:
            pcb.conv2DBwd(x, wt, dy, dw, dx, bwd_desc, ctx16, main_engine)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step()
    sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    sync_all()
    elapsed_ms = e0.elapsed_time(e1)
    if world > 1:
        tm = torch.tensor([elapsed_ms], device=device)
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        elapsed_ms = float(tm.item())
    clocks = sampler.stop() if rank == 0 else None

    # the results of the timed region, checked on rank 0 against the CPU checker (before anything overwrites them)
    parity = None
    if rank == 0 and not args.kernels_only:
        if world > 1:      # dw was summed over the ranks: recompute this rank's own gradient into a scratch tensor
            dw_own = torch.empty_like(dw)
            pcb.conv2DBwd(x, wt, dy, dw_own, dx, bwd_desc, ctx16)
        else:
            dw_own = dw
        torch.cuda.synchronize()
        parity = check_parity(torch, x, wt, dy, y, dw_own, dx, n)

    # per-kernel device times (same inputs, same stream): a short window (burst clocks) and >= kernel_seconds of
    # back-to-back launches (sustained clocks), the SM clock sampled during each
    L = _lib.lib()
    d = _conv_desc(bwd_desc, torch.float16, ctx16, main_engine, require_input_grad=True)
    ws = Device.get(device).requestWorkspace(L.pcb_qconv2d_bwd_workspace_size(ctypes.byref(d)))
    kernel_fns = {
        "forward": lambda: pcb.conv2DFwd(x, wt, None, y, fwd_desc, ctx16, main_engine),
        "backward_filter": lambda: _lib.check(L.pcb_qconv2d_bwd_filter(ctypes.byref(d), _ptr(x), _ptr(dy), _ptr(dw), _ptr(ws), ws.numel(), _stream())),
        "backward_data": lambda: _lib.check(L.pcb_qconv2d_bwd_data(ctypes.byref(d), _ptr(wt), _ptr(dy), _ptr(dx), _ptr(ws), ws.numel(), _stream())),
    }
    kreps = 1 if args.kernels_only else max(3, args.steps)
    kernels, kernels_long, kernel_clocks = {}, {}, {}
    probe = ClockProbe(torch, L)
    for name, fn in kernel_fns.items():
        cs = ClockSampler(local_rank).start()
        kernels[name] = event_time(torch, fn, kreps, 1)      # (no probe here: it would share an SM with a CTA for a sixth of the window)
        kernel_clocks[name] = {"short": cs.stop()["sm_mhz"]}
    if not args.kernels_only:
        for name, fn in kernel_fns.items():
            reps_long = max(kreps, int(args.kernel_seconds * 1e3 / max(kernels[name], 1e-3)))
            cs = ClockSampler(local_rank).start()
            kernels_long[name], mhz_eff = event_time_probed(torch, fn, reps_long, probe, 1)
            c = cs.stop()
            kernel_clocks[name].update({"long": c["sm_mhz"], "long_effective": mhz_eff, "long_reasons": c["reasons"], "long_launches": reps_long})
    _lib.check(L.pcb_check_device_status(_ptr(ws), ws.numel(), _stream()))
    gemm_probe = None
    if rank == 0 and not args.kernels_only:     # a library GEMM as the yardstick of "per clock" (measurement only, not on the path)
        ga, gb = (torch.randn(8192, 8192, device=device, dtype=torch.bfloat16) for _ in range(2))
        g_ms, g_mhz = event_time_probed(torch, lambda: torch.mm(ga, gb), max(20, int(args.kernel_seconds * 400)), probe, 3)
        g_tf = 2 * 8192 ** 3 / (g_ms * 1e-3) / 1e12
        gemm_probe = {"tflops": g_tf, "sm_mhz_effective": g_mhz,
                      "frac_of_8192_flop_per_clk_sm": (g_tf * 1e12 / (torch.cuda.get_device_properties(device).multi_processor_count * 8192 * g_mhz * 1e6)) if g_mhz else None}
        del ga, gb

    # the factorised 8-product formulation of the same step on its own tensor-core kernels (rank 0, no collective)
    eight = None
    if rank == 0 and not args.kernels_only:
        ctx8 = Context({"UPSTRIDE_MEMORY_OPTIMIZED": "0", "UPSTRIDE_CONV_FP16_POLICY": "full16"})
        d8 = _conv_desc(bwd_desc, torch.float16, ctx8, _lib.ENGINE_TENSOR, require_input_grad=True)
        if all(L.pcb_qconv2d_engine_for(ctypes.byref(d8), p_) == _lib.ENGINE_TENSOR for p_ in (0, 1, 2)):
            engine8, kind = _lib.ENGINE_TENSOR, "tcgen05 (lane sums formed in shared memory, recombination in the epilogue)"
        else:
            engine8, kind = _lib.ENGINE_SIMT, "CUDA cores (lane sums in the gather, recombination in the epilogue)"
        ws8 = Device.get(device).requestWorkspace(L.pcb_qconv2d_bwd_workspace_size(ctypes.byref(d8)))
        t8 = {
            "forward": event_time(torch, lambda: pcb.conv2DFwd(x, wt, None, y, fwd_desc, ctx8, engine8), 5, 2),
            "backward_filter": event_time(torch, lambda: _lib.check(L.pcb_qconv2d_bwd_filter(ctypes.byref(d8), _ptr(x), _ptr(dy), _ptr(dw), _ptr(ws8), ws8.numel(), _stream())), 5, 2),
            "backward_data": event_time(torch, lambda: _lib.check(L.pcb_qconv2d_bwd_data(ctypes.byref(d8), _ptr(wt), _ptr(dy), _ptr(dx), _ptr(ws8), ws8.numel(), _stream())), 5, 2),
        }

        def step8():
            pcb.conv2DFwd(x, wt, None, y, fwd_desc, ctx8, engine8)
            pcb.conv2DBwd(x, wt, dy, dw, dx, bwd_desc, ctx8, engine8)

        t8_step = event_time(torch, step8, 5, 2)
        torch.cuda.synchronize()
        par8 = check_parity(torch, x, wt, dy, y, dw, dx, n)
        fl3 = 3 * flops_per_pass(n, ci, co, h, w)
        eight = {"value": fl3 / (t8_step * 1e-3) / 1e12, "unit": "effective TFLOP/s", "ms_per_step": t8_step, "kernel_ms": t8,
                 "executed_fraction_of_flops": 0.5,
                 "executed_tflops": 0.5 * fl3 / (t8_step * 1e-3) / 1e12,
                 "executed_frac_of_tensor_peak_burst": 0.5 * fl3 / (t8_step * 1e-3) / 1e12 / read_peaks()["tflops_burst"],
                 "kernels": kind, "parity": par8}
        # leave the 16-product results in the output tensors
        pcb.conv2DFwd(x, wt, None, y, fwd_desc, ctx16)
        pcb.conv2DBwd(x, wt, dy, dw, dx, bwd_desc, ctx16)

    # end to end through the public API from pinned host buffers
    e2e = None
    if (rank == 0 or world > 1) and not args.kernels_only:
        hx, hw, hdy = make_inputs(torch, n, ci, co, h, w, None, SEED + rank)
        hx, hw, hdy = hx.pin_memory(), hw.pin_memory(), hdy.pin_memory()
        hy = torch.empty(y.shape, dtype=torch.float16).pin_memory()
        hdx = torch.empty(x.shape, dtype=torch.float16).pin_memory()
        hdw = torch.empty(wt.shape, dtype=torch.float16).pin_memory()

        # Three streams and two sets of device buffers: the copy-in of step i+1 and the copy-out of step i-1 run beside
        # the kernels of step i (PCIe is full duplex). Every step still copies all its inputs in and all its results out.
        s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        sets = [dict(x=x, wt=wt, dy=dy, y=y, dw=dw, dx=dx),
                dict(x=torch.empty_like(x), wt=torch.empty_like(wt), dy=torch.empty_like(dy), y=torch.empty_like(y), dw=torch.empty_like(dw),
                     dx=torch.empty_like(dx))]
        in_done = [torch.cuda.Event() for _ in range(2)]
        cmp_done = [torch.cuda.Event() for _ in range(2)]
        out_done = [torch.cuda.Event() for _ in range(2)]

        def copies_in(b_):
            b_["x"].copy_(hx, non_blocking=True)
            b_["wt"].copy_(hw, non_blocking=True)
            b_["dy"].copy_(hdy, non_blocking=True)

        def copies_out(b_):
            hy.copy_(b_["y"], non_blocking=True)
            hdw.copy_(b_["dw"], non_blocking=True)
            hdx.copy_(b_["dx"], non_blocking=True)

        def e2e_step(i, compute=True):
            b_ = sets[i & 1]
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(cmp_done[i & 1])         # the kernels of step i-2 have read this set's inputs
                copies_in(b_)
                in_done[i & 1].record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(in_done[i & 1])
                if i >= 2:
                    s_cmp.wait_event(out_done[i & 1])        # the results of step i-2 have left this set
                if compute:
                    pcb.conv2DFwd(b_["x"], b_["wt"], None, b_["y"], fwd_desc, ctx16)
                    pcb.conv2DBwd(b_["x"], b_["wt"], b_["dy"], b_["dw"], b_["dx"], bwd_desc, ctx16)
                    if world > 1:
                        dist.all_reduce(b_["dw"])
                cmp_done[i & 1].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(cmp_done[i & 1])
                copies_out(b_)
                out_done[i & 1].record(s_out)

        def timed_e2e(steps_, compute):
            for i in range(2):
                e2e_step(i, compute)
            sync_all()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(s_in)
            for i in range(steps_):
                e2e_step(i + 2, compute)
            s_out.wait_stream(s_cmp)
            s_out.wait_stream(s_in)
            b.record(s_out)
            sync_all()
            ms = a.elapsed_time(b)
            if world > 1:
                tm_ = torch.tensor([ms], device=device)
                dist.all_reduce(tm_, op=dist.ReduceOp.MAX)
                ms = float(tm_.item())
            return ms

        e2e_steps = min(args.steps, 8)
        e2e_ms = timed_e2e(e2e_steps, True)
        copy_ms = timed_e2e(e2e_steps, False)       # the same copies in the same stream structure, no kernels: the roofline of e2e
        nb = lambda t_: t_.numel() * t_.element_size()
        h2d, d2h = nb(hx) + nb(hw) + nb(hdy), nb(hy) + nb(hdw) + nb(hdx)
        fl3 = 3 * flops_per_pass(n, ci, co, h, w)
        e2e = {"value": fl3 * world * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
               "copy_roofline": {"ms_per_step": copy_ms / e2e_steps,
                                 "h2d_gbs_per_gpu": h2d / (copy_ms / e2e_steps * 1e-3) / 1e9, "d2h_gbs_per_gpu": d2h / (copy_ms / e2e_steps * 1e-3) / 1e9,
                                 "value_if_copy_bound": fl3 * world * e2e_steps / (copy_ms * 1e-3) / 1e12,
                                 "frac": copy_ms / e2e_ms,
                                 "note": "pinned host<->device copies of the same byte counts in the same stream structure, no kernels, "
                                         "timed in this run; the %d rank(s) share one host's memory and PCIe root complex, so the "
                                         "end-to-end number does not scale with the GPU count" % world}}
        del hx, hw, hdy, hy, hdx, hdw, sets

    peaks = read_peaks()
    dense = sweep = sweep_f32 = None
    if world == 1 and not args.kernels_only and args.batch is None:      # single-GPU records; the scaling runs skip them
        torch.cuda.empty_cache()
        dense = dense_leg(torch, pcb, _lib, peaks)
        if not args.no_sweep:
            sweep = sweep_leg(torch, pcb, _lib, peaks)
            tf32_peak = dense["f32"].get("tf32_peak_tflops_measured") if dense and "f32" in dense else None
            sweep_f32 = sweep_leg(torch, pcb, _lib, peaks, reps=3, extra_nhwc=(), dtype="f32", tf32_peak=tf32_peak)
    if world > 1:
        dist.barrier()

    # second headline of the metric: quaternion ResNet-18 training images/s on the same ranks
    qres = None
    if not args.kernels_only and args.batch is None and not args.no_qresnet:
        torch.cuda.empty_cache()
        from phoenix_core_b200 import qresnet
        qres = qresnet.run(batch=128, steps=max(3, min(args.steps, 10)), warmup=3, quiet=True)
        if rank == 0 and world == 1 and qres is not None:     # every distinct convolution layer of the network on its own
            qres["layers"] = qresnet.layer_table(128, 10, peaks["tflops_sustained"])

    if rank == 0:
        fl = flops_per_pass(n, ci, co, h, w)
        total = 3 * fl * world * args.steps
        value = total / (elapsed_ms * 1e-3) / 1e12
        timing = kernels_long if kernels_long else kernels
        worst = max(timing, key=timing.get)
        achieved = fl / (timing[worst] * 1e-3) / 1e12
        achieved_short = fl / (kernels[worst] * 1e-3) / 1e12
        # the same kernel per SM clock: 8192 dense 16-bit FLOPs per clock and SM, at the clock the probe saw beside the kernel, with a
        # cuBLAS bf16 GEMM measured the same way in this run beside it
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        per_clock = None
        eff = kernel_clocks[worst].get("long_effective")
        if eff:
            per_clock = {"sm_mhz_effective": eff, "frac_of_8192_flop_per_clk_sm": achieved * 1e12 / (sms * 8192 * eff * 1e6),
                         "cublas_bf16_gemm": gemm_probe}
        traffic = traffic_note = None
        traffic_path = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(traffic_path) and n == 64:
            with open(traffic_path) as f:
                tj = json.load(f)
            traffic, traffic_note = tj.get(worst), tj.get("_comment")
        algorithmic_bytes = {"forward": 2 * (x.numel() + 4 * n * co * h * w + wt.numel()),
                             "backward_data": 2 * (4 * n * co * h * w + wt.numel() + x.numel()),
                             "backward_filter": 2 * (x.numel() + 4 * n * co * h * w) + 4 * wt.numel()}
        cpu = cpu16 = None
        if world == 1 and not args.kernels_only:
            cpu = cpu_baseline(torch, args.cpu_sample, 5, True)
            cpu16 = cpu_baseline(torch, args.cpu_sample, 3, False)
        line = {
            "metric": "quaternion conv2d fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": elapsed_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "pointwise 1x1 quaternion conv2d fwd+bwd, fp16 in/out, fp32 accumulate, batch %d/GPU, "
                                   "%d->%d quaternion channels, %dx%d, 16-product, NCHW" % (n, ci, co, h, w),
                       "parallelism": "dp%d" % world, "l2": "inputs (196 MiB) and outputs (392 MiB) exceed the 126 MB L2",
                       "flop_per_step_per_gpu": 3 * fl,
                       "allreduce": "filter gradient, started after backward-filter on a side stream, beside backward-data" if world > 1 else None,
                       "sm_margin": sm_margin},
            "parity": parity,
            "pct_of_tensor_peak": {"sustained": value / world / peaks["tflops_sustained"], "burst": value / world / peaks["tflops_burst"],
                                   "peaks": peaks["source"]},
            "kernel_ms": kernels, "kernel_ms_sustained": kernels_long or None, "kernel_sm_mhz": kernel_clocks,
            "roofline": {"bound": "tensor", "kernel": worst, "achieved": achieved, "peak": peaks["tflops_sustained"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["tflops_sustained"],
                         "peak_source": "%s, sustained bf16 GEMM; the kernel was timed alone over %s back-to-back launches (>= %.1f s) at a median of %s MHz"
                                        % (peaks["source"], kernel_clocks[worst].get("long_launches", kreps), args.kernel_seconds, kernel_clocks[worst].get("long")),
                         "short_window": {"achieved": achieved_short, "peak": peaks["tflops_burst"], "frac": achieved_short / peaks["tflops_burst"],
                                          "launches": kreps, "sm_mhz": kernel_clocks[worst]["short"], "peak_source": peaks["source"] + ", burst bf16 GEMM"},
                         "per_clock": per_clock,
                         "algorithmic_bytes": algorithmic_bytes[worst],
                         "hbm_frac": algorithmic_bytes[worst] / (timing[worst] * 1e-3) / 1e9 / peaks["hbm_gbs"],
                         "traffic": traffic, "traffic_note": traffic_note},
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": 4 * args.steps,
        }
        if qres is not None:
            line["qresnet18"] = qres
        if eight is not None:
            line["eight_product"] = eight
        if dense is not None:
            line["dense"] = dense
        if sweep is not None:
            line["sweep"] = sweep
        if sweep_f32 is not None:
            line["sweep_f32"] = sweep_f32
        if args.batch is not None:
            line["reduced_batch"] = "profiling run, not a benchmark value"
        if args.formulation != "16p" or args.engine != "auto":
            line["formulation"] = "profiling run (formulation %s, engine %s), not a benchmark value" % (args.formulation, args.engine)
        if cpu is not None:
            line["cpu_baseline"] = {"value": cpu[0], "unit": "TFLOP/s", "cores": cpu[1], "kind": "port", "sample": cpu[2],
                                    "sixteen_product": {"value": cpu16[0], "unit": "TFLOP/s", "sample": cpu16[2]}}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-sample", type=int, default=32, help="batch size of the CPU baseline sample")
    ap.add_argument("--kernel-seconds", type=float, default=2.0, help="length of each kernel's sustained timing run")
    ap.add_argument("--no-sweep", action="store_true", help="skip the ResNet-stage shape sweep")
    ap.add_argument("--no-qresnet", action="store_true", help="skip the QResNet-18 training leg")
    ap.add_argument("--batch", type=int, default=None,
                    help="profiling only: per-GPU batch instead of 64 (the line is then marked 'reduced_batch' and is not a benchmark value)")
    ap.add_argument("--formulation", default="16p", choices=["16p", "8p"],
                    help="profiling only: 8p times the factorised tensor-core kernels as the main step (use with --kernels-only)")
    ap.add_argument("--sweep-only", action="store_true", help="profiling only: run the shape sweep (or one shape of it) and print its record")
    ap.add_argument("--sm-margin", type=int, default=None, help="SMs left free of the persistent kernels (default: 2 on more than one GPU, else 0)")
    ap.add_argument("--sweep-shape", default=None, help="channels,size,kernel,stride of the single sweep shape to run")
    ap.add_argument("--sweep-batch", type=int, default=128)
    ap.add_argument("--sweep-reps", type=int, default=5)
    ap.add_argument("--sweep-layout", default="nchw", choices=["nchw", "nhwc"])
    ap.add_argument("--sweep-dtype", default="f16", choices=["f16", "f32"])
    ap.add_argument("--engine", default="auto", choices=["auto", "simt", "tensor"],
                    help="profiling only: kernel family of the main step (with --formulation 8p: simt = the factorised CUDA-core kernels)")
    ap.add_argument("--dense-only", action="store_true", help="profiling only: run the dense leg and print its record")
    ap.add_argument("--kernels-only", action="store_true",
                    help="profiling only: skip the end-to-end, per-kernel and CPU-baseline legs")
    args = ap.parse_args()
    if args.batch is not None:
        WORKLOAD["n"] = args.batch
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
