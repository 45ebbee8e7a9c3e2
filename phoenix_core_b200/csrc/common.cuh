// Shared definitions of the B200 quaternion Conv2D / Dense backend: problem geometry, the quaternion
// sign/permutation block, dtype helpers and error plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/phoenix_core_b200.h"

namespace pcb {

// ---------------------------------------------------------------------------------------------------
// The Hamilton product y = x (x) w with the input on the left, as a 4x4 block of signed weight
// components (reference sign table: src/algebras.cc:28-49): input component l contributes
// sign(l,d) * w_{l^d} to output component d. The permutation is a XOR; the negative entries are
// (l,d) in {(1,0),(1,2),(2,0),(2,3),(3,0),(3,1)}, packed below as bit (4*l + d).
// For the filter gradient the same term is read as: dW_r gets sign(l, l^r) * <x_l, dy_{l^r}>.
// ---------------------------------------------------------------------------------------------------
constexpr uint32_t QUAT_NEG_MASK = 0x3950u;
__host__ __device__ __forceinline__ int quat_weight_component(int l, int d) { return l ^ d; }
__host__ __device__ __forceinline__ bool quat_negative(int l, int d) { return (QUAT_NEG_MASK >> (4 * l + d)) & 1u; }

enum Pass : int { PASS_FWD = 0, PASS_BWD_DATA = 1, PASS_BWD_FILTER = 2 };

// Every operator of the backend is one of three passes over this geometry. A dense layer is the
// 1x1 convolution of 1x1 images (H = W = 1, Nb = batch) with optionally input-major weights.
struct Geom {
    int Nb;              // quaternion batch
    int Ci, Co;          // quaternion channels
    int H, W, HO, WO;
    int KH, KW, SH, SW, DH, DW, PT, PL;
    int w_io;            // weights stored [r][ci][co] (dense IO layout; taps == 1)
    int dw_io;           // filter gradient written [r][ci][co]
    int real_in;         // x holds the real component only ([Nb, Ci, H, W])
    int has_bias;
};

template <typename T> struct DType;
template <> struct DType<float> {
    static __device__ __forceinline__ float load(const float* p) { return __ldg(p); }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct DType<__half> {
    static __device__ __forceinline__ float load(const __half* p) { return __half2float(__ldg(p)); }
    static __device__ __forceinline__ void store(__half* p, float v) { *p = __float2half_rn(v); }
};
template <> struct DType<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(__ldg(p)); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

inline size_t dtype_size(int dtype) { return dtype == PCB_F32 ? 4 : 2; }

// Error plumbing (host side). The message of the last failure is kept per host thread.
void set_error(const char* fmt, ...);
#define PCB_CUDA_TRY(expr)                                                                      \
    do {                                                                                        \
        cudaError_t _e = (expr);                                                                \
        if (_e != cudaSuccess) {                                                                \
            ::pcb::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
            return PCB_ERR_CUDA;                                                                \
        }                                                                                       \
    } while (0)

// Launchers implemented by the kernel translation units. Operand roles per pass:
//   forward:         a = filters, b = input,          out = output
//   backward-data:   a = filters, b = output gradient, out = input gradient
//   backward-filter: a = output gradient, b = input,   out = filter gradient
// `scratch` is fp32 scratch for split-K accumulation when the output type is not fp32 (may be null
// otherwise).
int simt_launch(Pass pass, int dtype, int variant, const Geom& g, const void* a, const void* b, const void* bias,
                void* out, float* scratch, cudaStream_t stream);
size_t simt_scratch_bytes(Pass pass, int dtype, int variant, const Geom& g);
// Backward-filter whose split-K accumulator is a fixed array inside the library (no workspace, no allocation).
int simt_bwd_filter_static(int dtype, int variant, const Geom& g, const void* dy, const void* x, void* dw, cudaStream_t stream);
size_t simt_static_scratch_capacity();

}  // namespace pcb
