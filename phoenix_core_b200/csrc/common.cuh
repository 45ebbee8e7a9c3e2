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
// The product y = x (x) w of a hyper-complex layer with the input on the left, as an nc x nc block of
// signed weight components: input component l contributes sign(l,d) * w_{r(l,d)} to output component d.
// For the filter gradient the same term reads: dW_r gets sign(l,d) * <x_l, dy_d> with d = r(l,r).
//
// Quaternions (reference sign table: src/algebras.cc:28-49): r(l,d) = l ^ d, negative entries
// (l,d) in {(1,0),(1,2),(2,0),(2,3),(3,0),(3,1)}. Complex numbers (src/algebras.cc:12-23): r = l ^ d,
// negative (1,0). GA(3,0,0) (src/algebras.cc:58-145): the components are the blades
// 1, e1, e2, e3, e12, e13, e23, e123; with a blade written as the bit set of its generators the
// product blade is the XOR of the sets and the sign is the parity of the transpositions that sort the
// concatenated generators (all generators square to +1). Components 3 (e3 = bit set 100) and 4
// (e12 = 011) are the only ones whose position differs from their bit set.
// The negative entries of any of these are kept as bit (8*l + d) of a 64-bit mask in the geometry.
// ---------------------------------------------------------------------------------------------------
constexpr uint32_t QUAT_NEG_MASK = 0x3950u;           // bit (4*l + d): the quaternion-only kernels use this form
__host__ __device__ __forceinline__ int quat_weight_component(int l, int d) { return l ^ d; }
__host__ __device__ __forceinline__ bool quat_negative(int l, int d) { return (QUAT_NEG_MASK >> (4 * l + d)) & 1u; }

__host__ __device__ __forceinline__ int ga_bits(int c) { return c == 3 ? 4 : (c == 4 ? 3 : c); }   // component <-> bit set (an involution)
// Weight component that pairs input component l with output component d (also: output component for (l, r)).
__host__ __device__ __forceinline__ int alg_pair(int ga, int l, int d) { return ga ? ga_bits(ga_bits(l) ^ ga_bits(d)) : (l ^ d); }
__host__ __device__ __forceinline__ bool alg_negative(unsigned long long neg, int l, int d) { return (neg >> (8 * l + d)) & 1ull; }

enum Pass : int { PASS_FWD = 0, PASS_BWD_DATA = 1, PASS_BWD_FILTER = 2 };

// Every operator of the backend is one of three passes over this geometry. A dense layer is the
// 1x1 convolution of 1x1 images (H = W = 1, Nb = batch) with optionally input-major weights.
struct Geom {
    int nc;              // components of the algebra: 1 real, 2 complex, 4 quaternion, 8 GA(3,0,0)
    int ga;              // GA(3,0,0) component order (see alg_pair)
    unsigned long long neg;   // negative entries of the nc x nc block, bit (8*l + d)
    int Nb;              // hyper-complex batch
    int Ci, Co;          // hyper-complex channels
    int H, W, HO, WO;
    int KH, KW, SH, SW, DH, DW, PT, PL;
    int w_io;            // weights stored [r][ci][co] (dense IO layout; taps == 1)
    int dw_io;           // filter gradient written [r][ci][co]
    int real_in;         // x holds the real component only ([Nb, Ci, H, W])
    int has_bias;
    // Element strides (the CUDA-core kernels address every tensor through them; the tensor-core kernels need `plain`).
    //   x (and dx):  plane * xp + c * xc + h * xh + w * xw      with plane = comp * Nb + img
    //   y (and dy):  plane * yp + c * yc + h * yh + w * yw
    //   filters:     r * wr + co * wo + ci * wi + kh * wh + kw * ww;   filter gradient: the same with the d-prefixed strides
    int xp, xc, xh, xw, yp, yc, yh, yw;
    int wr, wo, wi, wh, ww, dr, dco, dci, dkh, dkw;
    int bias_ld;         // bias is [components][bias_ld]
    int plain;           // NCHW activations, OIHW (or dense) filters, one group: the layouts the tensor-core kernels read
    int groups;          // host side only: groups of the convolution; Ci / Co above are the channels of ONE group
};

enum { LAYOUT_NCHW = 0, LAYOUT_NHWC = 1 };
enum { FILTER_OIHW = 0, FILTER_OHWI = 1, FILTER_HWIO = 2 };

// Fills the strides for a convolution over full tensors of Ci_total / Co_total channels of which this geometry covers
// g.Ci / g.Co (one group); filters hold g.Ci input channels per output channel.
inline void set_conv_strides(Geom& g, int data_format, int filter_layout, int Ci_total, int Co_total) {
    const int T = g.KH * g.KW;
    if (data_format == LAYOUT_NCHW) {
        g.xp = Ci_total * g.H * g.W; g.xc = g.H * g.W; g.xh = g.W; g.xw = 1;
        g.yp = Co_total * g.HO * g.WO; g.yc = g.HO * g.WO; g.yh = g.WO; g.yw = 1;
    } else {
        g.xp = Ci_total * g.H * g.W; g.xc = 1; g.xh = g.W * Ci_total; g.xw = Ci_total;
        g.yp = Co_total * g.HO * g.WO; g.yc = 1; g.yh = g.WO * Co_total; g.yw = Co_total;
    }
    g.wr = Co_total * g.Ci * T;
    if (filter_layout == FILTER_OIHW)      { g.wo = g.Ci * T; g.wi = T; g.wh = g.KW; g.ww = 1; }
    else if (filter_layout == FILTER_OHWI) { g.wo = T * g.Ci; g.wh = g.KW * g.Ci; g.ww = g.Ci; g.wi = 1; }
    else                                   { g.wh = g.KW * g.Ci * Co_total; g.ww = g.Ci * Co_total; g.wi = Co_total; g.wo = 1; }
    g.dr = g.wr; g.dco = g.wo; g.dci = g.wi; g.dkh = g.wh; g.dkw = g.ww;
    g.bias_ld = Co_total;
}

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

// Fills nc / ga / neg of the geometry for a pcb_algebra value; false if the value is unknown.
inline bool algebra_setup(int algebra, Geom& g) {
    g.ga = 0; g.neg = 0ull;
    switch (algebra) {
        case PCB_ALGEBRA_REAL: g.nc = 1; return true;
        case PCB_ALGEBRA_COMPLEX: g.nc = 2; g.neg = 1ull << (8 * 1 + 0); return true;
        case PCB_ALGEBRA_QUATERNION:
            g.nc = 4;
            for (int l = 0; l < 4; ++l)
                for (int d = 0; d < 4; ++d)
                    if (quat_negative(l, d)) g.neg |= 1ull << (8 * l + d);
            return true;
        case PCB_ALGEBRA_GA_300:
            g.nc = 8; g.ga = 1;
            for (int l = 0; l < 8; ++l)
                for (int r = 0; r < 8; ++r) {
                    // x_l * w_r: count the transpositions that move each generator of w_r left past the higher generators of x_l
                    const int a = ga_bits(l), b = ga_bits(r);
                    int swaps = 0;
                    for (int s = a >> 1; s; s >>= 1) swaps += __builtin_popcount(s & b);
                    if (swaps & 1) g.neg |= 1ull << (8 * l + alg_pair(1, l, r));
                }
            return true;
        default: return false;
    }
}

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
