// SM clock probe: one thread counts its own cycles (clock64) against the nanosecond timer (globaltimer) for a given number of
// cycles and writes both differences. Launched on a second stream beside other kernels, it tells at which clock the SMs really
// run while those kernels execute (the clock NVML reports is sampled every few hundred milliseconds and does not show how far
// the power cap pulls the clock down inside a burst of launches). One block of one thread: it fits beside any resident CTA.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/phoenix_core_b200.h"

namespace {

__global__ void clock_probe_kernel(long long spin_cycles, long long* out) {
    long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    const long long c0 = clock64();
    long long c1 = c0;
    while (c1 - c0 < spin_cycles) c1 = clock64();      // bounded by its argument
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    out[0] = c1 - c0;
    out[1] = t1 - t0;
}

}  // namespace

extern "C" int pcb_aux_clock_probe(long long spin_cycles, long long* out_cycles_and_ns, void* stream) {
    if (spin_cycles < 1 || spin_cycles > (1ll << 32) || out_cycles_and_ns == nullptr) return PCB_ERR_INVALID_ARGUMENT;
    clock_probe_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(spin_cycles, out_cycles_and_ns);
    return cudaGetLastError() == cudaSuccess ? PCB_OK : PCB_ERR_CUDA;
}
