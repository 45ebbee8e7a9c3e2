// Auxiliary kernels of the QResNet-18 harness: batch-norm (+ ReLU) and 3x3 stride-2 max pooling.
//
// Batch-norm (+ ReLU) over stacked hyper-complex activations [planes = D*N, C, H, W]: one mean / variance per channel,
// shared by the D components. Auxiliary kernels of the QResNet-18 harness -- the reference has no normalisation layer
// (its TensorFlow plugin relies on TensorFlow's); they exist because the framework kernels launch one block per channel
// and leave the GPU idle at 16 channels. Three passes over the data forward (statistics; apply: read, write), five to seven
// backward (statistics: x and dy, and the stored output where the ReLU mask cannot be recomputed from x; apply: the same
// reads and one or two writes). Variants: the residual add of a block's tail inside the apply pass, the stem's max-pool
// fused into the apply pass (the normalised tensor is never stored), flat 16-byte kernels for rows of 7 x 7 elements.
// The per-channel coefficients are computed inside the apply kernels from the channel sums; there is no finalize launch.
//
// Every kernel sees the tensor as rows of HW contiguous elements, row r = plane * C + c.
#include "common.cuh"

namespace pcb {
namespace {

constexpr int BN_THREADS = 256;

// V consecutive elements (8, 4 or 1) as floats.
template <typename T, int V> struct VecIO;
template <typename T> struct VecIO<T, 1> {
    static __device__ __forceinline__ void load(const T* p, float (&f)[1]) { f[0] = DType<T>::load(p); }
    static __device__ __forceinline__ void store(T* p, const float (&f)[1]) { DType<T>::store(p, f[0]); }
};
template <int V> struct VecIO<__half, V> {
    static __device__ __forceinline__ void load(const __half* p, float (&f)[V]) {
        alignas(16) __half2 h[V / 2];
        if (V == 8) *reinterpret_cast<uint4*>(h) = __ldg(reinterpret_cast<const uint4*>(p));
        else *reinterpret_cast<uint2*>(h) = __ldg(reinterpret_cast<const uint2*>(p));
#pragma unroll
        for (int i = 0; i < V / 2; ++i) { const float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    }
    static __device__ __forceinline__ void store(__half* p, const float (&f)[V]) {
        alignas(16) __half2 h[V / 2];
#pragma unroll
        for (int i = 0; i < V / 2; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        if (V == 8) *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(h);
        else *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(h);
    }
};
template <int V> struct VecIO<__nv_bfloat16, V> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[V]) {
        alignas(16) __nv_bfloat162 h[V / 2];
        if (V == 8) *reinterpret_cast<uint4*>(h) = __ldg(reinterpret_cast<const uint4*>(p));
        else *reinterpret_cast<uint2*>(h) = __ldg(reinterpret_cast<const uint2*>(p));
#pragma unroll
        for (int i = 0; i < V / 2; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[V]) {
        alignas(16) __nv_bfloat162 h[V / 2];
#pragma unroll
        for (int i = 0; i < V / 2; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        if (V == 8) *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(h);
        else *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(h);
    }
};
template <> struct VecIO<__half, 1> {
    static __device__ __forceinline__ void load(const __half* p, float (&f)[1]) { f[0] = DType<__half>::load(p); }
    static __device__ __forceinline__ void store(__half* p, const float (&f)[1]) { DType<__half>::store(p, f[0]); }
};
template <> struct VecIO<__nv_bfloat16, 1> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[1]) { f[0] = DType<__nv_bfloat16>::load(p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[1]) { DType<__nv_bfloat16>::store(p, f[0]); }
};

// The forward coefficients of a channel recomputed in the backward pass (relu == 2: the ReLU mask is taken from
// x * k0 + k1 > 0 instead of from the stored output, which then need not be read).
struct BnFwdParams { const float* gamma; const float* beta; const float* mean; const float* invstd; };
__device__ __forceinline__ void bn_fwd_coef(const BnFwdParams& f, int c, float& k0, float& k1) {
    k0 = f.gamma[c] * f.invstd[c];
    k1 = f.beta[c] - f.mean[c] * k0;
}

// Per-channel coefficients of the apply passes, computed where they are used from the channel sums (there is no separate
// finalize launch). Forward (MODE 0): y = x * k0 + k1 with k0 = gamma / std, k1 = beta - mean * k0; block 0 also saves mean
// and 1/std through out0 / out1. Backward (MODE 1): dx = k0 * g + k1 * x + k2 from
//   xhat = (x - mean) * invstd;  dgamma = sum(g * xhat);  dbeta = sum(g);  dx = gamma * invstd * (g - dbeta / m - xhat * dgamma / m);
// block 0 writes dgamma / dbeta through out0 / out1.
struct BnCoef {
    const float* sums;                                          // [2][C]: (x, x*x) forward, (g, g*x) backward
    const float* gamma; const float* beta; const float* mean; const float* invstd;
    float* out0; float* out1;
    float count, eps;
};
template <int MODE>
__device__ __forceinline__ void bn_coef(const BnCoef& q, int C, int c, float& k0, float& k1, float& k2) {
    if (MODE == 0) {
        const float m = q.sums[c] / q.count;
        const float var = fmaxf(q.sums[C + c] / q.count - m * m, 0.f);
        k0 = q.gamma[c] * rsqrtf(var + q.eps);
        k1 = q.beta[c] - m * k0;
        k2 = 0.f;
    } else {
        const float sg = q.sums[c], sgx = q.sums[C + c], is = q.invstd[c], mu = q.mean[c];
        const float dg = (sgx - mu * sg) * is;
        k0 = q.gamma[c] * is;
        k1 = -k0 * is * dg / q.count;
        k2 = -k0 * sg / q.count - k1 * mu;
    }
}
template <int MODE>
__device__ __forceinline__ void bn_coef_outputs(const BnCoef& q, int C) {
    if (blockIdx.x != 0) return;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        if (MODE == 0) {
            const float m = q.sums[c] / q.count;
            const float var = fmaxf(q.sums[C + c] / q.count - m * m, 0.f);
            q.out0[c] = m; q.out1[c] = rsqrtf(var + q.eps);
        } else {
            const float sg = q.sums[c];
            q.out0[c] = (q.sums[C + c] - q.mean[c] * sg) * q.invstd[c]; q.out1[c] = sg;
        }
    }
}

// Sums of two quantities per channel. MODE 0: (x, x*x). MODE 1: (g, g*x) with g = dy masked by y > 0 when relu.
// Block (c, s): the planes s, s + S, ... of channel c, walked as one flat index space of V-element groups (so that small
// rows, e.g. 7 x 7 planes, still occupy every thread); one atomic pair per block into sums[0..C) and sums[C..2C).
template <typename T, int MODE, int V>
__global__ void __launch_bounds__(BN_THREADS)
bn_sums_kernel(const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ dy, float* __restrict__ sums, int planes, int C, int HW, int relu,
               BnFwdParams fw) {
    const int c = blockIdx.x, s = blockIdx.y, S = gridDim.y;
    float m0 = 0.f, m1 = 0.f;
    if (MODE == 1 && relu == 2) bn_fwd_coef(fw, c, m0, m1);
    const int per_row = HW / V;
    const int my_planes = s < planes ? (planes - s + S - 1) / S : 0;
    float a0 = 0.f, a1 = 0.f;
    for (int j = threadIdx.x; j < my_planes * per_row; j += BN_THREADS) {
        const int pi = j / per_row, i = j - pi * per_row;
        const size_t off = ((size_t)(s + pi * S) * C + c) * HW + (size_t)i * V;
        float fx[V];
        VecIO<T, V>::load(x + off, fx);
        if (MODE == 0) {
#pragma unroll
            for (int e = 0; e < V; ++e) { a0 += fx[e]; a1 = fmaf(fx[e], fx[e], a1); }
        } else {
            float fg[V], fy[V];
            VecIO<T, V>::load(dy + off, fg);
            if (relu == 1) VecIO<T, V>::load(y + off, fy);
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const float out = relu == 2 ? fmaf(fx[e], m0, m1) : fy[e];
                const float g = (relu && !(out > 0.f)) ? 0.f : fg[e];
                a0 += g; a1 = fmaf(g, fx[e], a1);
            }
        }
    }
    __shared__ float red[2][BN_THREADS / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { a0 += __shfl_xor_sync(0xffffffffu, a0, o); a1 += __shfl_xor_sync(0xffffffffu, a1, o); }
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = a0; red[1][threadIdx.x >> 5] = a1; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float t0 = 0.f, t1 = 0.f;
#pragma unroll
        for (int w = 0; w < BN_THREADS / 32; ++w) { t0 += red[0][w]; t1 += red[1][w]; }
        atomicAdd(sums + c, t0);
        atomicAdd(sums + C + c, t1);
    }
}

// MODE 0: y = max(x*coef0 + coef1 [+ res], 0 if relu).  MODE 1: dx = coef0*g + coef1*x + coef2 with g = dy masked by y > 0
// [and dres = g: the gradient of the residual branch that was added before the ReLU].
template <typename T, int MODE, int V>
__global__ void __launch_bounds__(BN_THREADS)
bn_apply_kernel(const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ out, BnCoef coef,
                size_t rows, int C, int HW, int relu, const T* __restrict__ res, T* __restrict__ dres, BnFwdParams fw) {
    bn_coef_outputs<MODE>(coef, C);
    const int per_row = HW / V;
    const size_t total = rows * per_row;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t row = idx / per_row;
        const int i = (int)(idx - row * per_row);
        const int c = (int)(row % C);
        float k0, k1, k2;
        bn_coef<MODE>(coef, C, c, k0, k1, k2);
        float m0 = 0.f, m1 = 0.f;
        if (MODE == 1 && relu == 2) bn_fwd_coef(fw, c, m0, m1);
        const size_t off = row * HW + (size_t)i * V;
        float fx[V], fo[V];
        VecIO<T, V>::load(x + off, fx);
        if (MODE == 0) {
            float fr[V];
            if (res) VecIO<T, V>::load(res + off, fr);
#pragma unroll
            for (int e = 0; e < V; ++e) { const float v = fmaf(fx[e], k0, k1) + (res ? fr[e] : 0.f); fo[e] = relu ? fmaxf(v, 0.f) : v; }
        } else {
            float fg[V], fy[V];
            VecIO<T, V>::load(dy + off, fg);
            if (relu == 1) VecIO<T, V>::load(y + off, fy);
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const float out = relu == 2 ? fmaf(fx[e], m0, m1) : fy[e];
                const float g = (relu && !(out > 0.f)) ? 0.f : fg[e];
                fo[e] = fmaf(k0, g, fmaf(k1, fx[e], k2));
                fg[e] = g;
            }
            if (dres) VecIO<T, V>::store(dres + off, fg);
        }
        VecIO<T, V>::store(out + off, fo);
    }
}

// ---- rows that are not a multiple of 4 elements (7 x 7 planes) --------------------------------------------------------------
// The kernels above then fall back to 2-byte accesses. These two walk the tensor as one flat sequence of 16-byte groups
// instead (the whole tensor is a multiple of 8 elements and 16-byte aligned even if its rows are not): the 8 elements of a
// group belong to at most two channels when rows are at least 8 elements long, and the channel is tracked per element.
template <typename T, int MODE>
__global__ void __launch_bounds__(BN_THREADS)
bn_sums_flat_kernel(const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ dy, float* __restrict__ sums, size_t groups, int C, int HW,
                    int relu, BnFwdParams fw) {
    extern __shared__ float bins[];                               // [2][C]
    for (int i = threadIdx.x; i < 2 * C; i += BN_THREADS) bins[i] = 0.f;
    __syncthreads();
    for (size_t gi = (size_t)blockIdx.x * BN_THREADS + threadIdx.x; gi < groups; gi += (size_t)gridDim.x * BN_THREADS) {
        const size_t i0 = gi * 8;
        const size_t row = i0 / HW;
        int r = (int)(i0 - row * HW), c = (int)(row % C);
        float fx[8], fg[8], fy[8];
        VecIO<T, 8>::load(x + i0, fx);
        if (MODE == 1) {
            VecIO<T, 8>::load(dy + i0, fg);
            if (relu == 1) VecIO<T, 8>::load(y + i0, fy);
        }
        float a0 = 0.f, a1 = 0.f, m0 = 0.f, m1 = 0.f;
        if (MODE == 1 && relu == 2) bn_fwd_coef(fw, c, m0, m1);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            if (MODE == 0) { a0 += fx[e]; a1 = fmaf(fx[e], fx[e], a1); }
            else {
                const float out = relu == 2 ? fmaf(fx[e], m0, m1) : fy[e];
                const float g = (relu && !(out > 0.f)) ? 0.f : fg[e];
                a0 += g; a1 = fmaf(g, fx[e], a1);
            }
            if (++r == HW) {                                      // the next element starts the next channel's row
                atomicAdd(bins + c, a0); atomicAdd(bins + C + c, a1);
                a0 = a1 = 0.f; r = 0;
                if (++c == C) c = 0;
                if (MODE == 1 && relu == 2) bn_fwd_coef(fw, c, m0, m1);
            }
        }
        atomicAdd(bins + c, a0); atomicAdd(bins + C + c, a1);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * C; i += BN_THREADS) atomicAdd(sums + i, bins[i]);
}

template <typename T, int MODE>
__global__ void __launch_bounds__(BN_THREADS)
bn_apply_flat_kernel(const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ out, BnCoef coef,
                     size_t groups, int C, int HW, int relu, const T* __restrict__ res, T* __restrict__ dres, BnFwdParams fw) {
    bn_coef_outputs<MODE>(coef, C);
    for (size_t gi = (size_t)blockIdx.x * BN_THREADS + threadIdx.x; gi < groups; gi += (size_t)gridDim.x * BN_THREADS) {
        const size_t i0 = gi * 8;
        const size_t row = i0 / HW;
        int r = (int)(i0 - row * HW), c = (int)(row % C);
        float fx[8], fo[8], fg[8], fy[8], fr[8];
        VecIO<T, 8>::load(x + i0, fx);
        if (MODE == 0) { if (res) VecIO<T, 8>::load(res + i0, fr); }
        else {
            VecIO<T, 8>::load(dy + i0, fg);
            if (relu == 1) VecIO<T, 8>::load(y + i0, fy);
        }
        float k0, k1, k2, m0 = 0.f, m1 = 0.f;
        bn_coef<MODE>(coef, C, c, k0, k1, k2);
        if (MODE == 1 && relu == 2) bn_fwd_coef(fw, c, m0, m1);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            if (MODE == 0) {
                const float v = fmaf(fx[e], k0, k1) + (res ? fr[e] : 0.f);
                fo[e] = relu ? fmaxf(v, 0.f) : v;
            } else {
                const float o = relu == 2 ? fmaf(fx[e], m0, m1) : fy[e];
                const float g = (relu && !(o > 0.f)) ? 0.f : fg[e];
                fo[e] = fmaf(k0, g, fmaf(k1, fx[e], k2));
                fg[e] = g;
            }
            if (++r == HW) {
                r = 0;
                if (++c == C) c = 0;
                bn_coef<MODE>(coef, C, c, k0, k1, k2);
                if (MODE == 1 && relu == 2) bn_fwd_coef(fw, c, m0, m1);
            }
        }
        VecIO<T, 8>::store(out + i0, fo);
        if (MODE == 1 && dres) VecIO<T, 8>::store(dres + i0, fg);
    }
}

// 3x3 stride-2 pad-1 max pooling over rows of H x W elements (one row per (plane, channel)); the forward pass keeps the
// position of the maximum inside its window (0..8), the backward pass gathers: every input pixel looks at the at most four
// windows that contain it, so there are no atomics.
template <typename T>
__global__ void __launch_bounds__(BN_THREADS)
maxpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint8_t* __restrict__ arg, size_t rows, int H, int W, int HO, int WO) {
    const size_t total = rows * HO * WO;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int ow = (int)(idx % WO);
        const int oh = (int)((idx / WO) % HO);
        const size_t row = idx / ((size_t)WO * HO);
        const T* src = x + row * H * W;
        float best = -INFINITY;
        int where = 0;
#pragma unroll
        for (int kh = 0; kh < 3; ++kh) {
            const int ih = 2 * oh - 1 + kh;
#pragma unroll
            for (int kw = 0; kw < 3; ++kw) {
                const int iw = 2 * ow - 1 + kw;
                if ((unsigned)ih < (unsigned)H && (unsigned)iw < (unsigned)W) {
                    const float v = DType<T>::load(src + ih * W + iw);
                    if (v > best || (v != v)) { best = v; where = kh * 3 + kw; }
                }
            }
        }
        DType<T>::store(y + idx, best);
        arg[idx] = (uint8_t)where;
    }
}

// The same pooling for lines of a multiple of 8 pixels (and a multiple of 4 outputs): one thread makes 4 consecutive outputs from
// three 16-byte loads (the 8 input columns 2*ow0 .. 2*ow0 + 7 of each window line) and three single elements (column 2*ow0 - 1),
// and writes them with one 8-byte store and one 4-byte store of arg-max positions. Same scan order inside a window as above.
template <typename T>
__global__ void __launch_bounds__(BN_THREADS)
maxpool_fwd4_kernel(const T* __restrict__ x, T* __restrict__ y, uint8_t* __restrict__ arg, size_t rows, int H, int W, int HO, int WO) {
    const int groups = WO / 4;
    const size_t total = rows * HO * groups;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int g = (int)(idx % groups);
        const int oh = (int)((idx / groups) % HO);
        const size_t row = idx / ((size_t)groups * HO);
        const T* src = x + row * H * W;
        float best[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        int where[4] = {0, 0, 0, 0};
#pragma unroll
        for (int kh = 0; kh < 3; ++kh) {
            const int ih = 2 * oh - 1 + kh;
            if ((unsigned)ih >= (unsigned)H) continue;
            float f[8];
            VecIO<T, 8>::load(src + (size_t)ih * W + 8 * g, f);
            const float left = g > 0 ? DType<T>::load(src + (size_t)ih * W + 8 * g - 1) : 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
                for (int kw = 0; kw < 3; ++kw) {
                    const int rel = 2 * j - 1 + kw;                 // column relative to 8 * g
                    if (rel < 0 && g == 0) continue;                // left padding
                    const float v = rel < 0 ? left : f[rel];
                    if (v > best[j] || (v != v)) { best[j] = v; where[j] = kh * 3 + kw; }
                }
            }
        }
        const size_t o = (row * HO + oh) * WO + 4 * g;
        VecIO<T, 4>::store(y + o, best);
        *reinterpret_cast<uint32_t*>(arg + o) = (uint32_t)where[0] | ((uint32_t)where[1] << 8) | ((uint32_t)where[2] << 16) | ((uint32_t)where[3] << 24);
    }
}

// Backward for the same line shapes: one thread per 8 input pixels reads, for each of its one or two output lines, the arg-max
// bytes of windows 4g .. 4g + 3 as one 32-bit word and their gradients as one 8-byte load, plus window 4g + 4 on its own.
template <typename T>
__global__ void __launch_bounds__(BN_THREADS)
maxpool_bwd8_kernel(const T* __restrict__ dy, const uint8_t* __restrict__ arg, T* __restrict__ dx, size_t rows, int H, int W, int HO, int WO) {
    const int per_line = W / 8;
    const size_t total = rows * H * per_line;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int g = (int)(idx % per_line), iw0 = 8 * g;
        const int ih = (int)((idx / per_line) % H);
        const size_t row = idx / ((size_t)per_line * H);
        const size_t obase = row * HO * WO;
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        for (int oh = ih >> 1; oh <= (ih + 1) >> 1; ++oh) {
            if (oh >= HO) continue;
            const int kh = ih - (2 * oh - 1);
            const size_t o = obase + (size_t)oh * WO + 4 * g;
            const uint32_t a4 = __ldg(reinterpret_cast<const uint32_t*>(arg + o));
            float g4[4];
            VecIO<T, 4>::load(dy + o, g4);
#pragma unroll
            for (int j = 0; j < 5; ++j) {
                int a;
                float gr;
                if (j < 4) { a = (int)((a4 >> (8 * j)) & 0xffu); gr = g4[j]; }
                else {
                    if (4 * g + 4 >= WO) continue;
                    a = arg[o + 4]; gr = DType<T>::load(dy + o + 4);
                }
                // window 4g + j covers the columns 2j - 1 .. 2j + 1 relative to iw0; j is a constant of the unrolled loop
                const int akh = (a * 11) >> 5, akw = a - 3 * akh;     // a / 3 and a % 3 for a in 0..8
                const float m = akh == kh ? gr : 0.f;
                if (2 * j - 1 >= 0) acc[(2 * j - 1) & 7] += akw == 0 ? m : 0.f;
                if (2 * j < 8) acc[(2 * j) & 7] += akw == 1 ? m : 0.f;
                if (2 * j + 1 < 8) acc[(2 * j + 1) & 7] += akw == 2 ? m : 0.f;
            }
        }
        VecIO<T, 8>::store(dx + (row * H + ih) * W + iw0, acc);
    }
}

// One thread per (row, input line, V consecutive input pixels): the windows that can contain them are the V/2 + 1 output
// columns from iw0/2 on and the one or two output lines around ih; their arg-max bytes and gradients are read once.
template <typename T, int V>
__global__ void __launch_bounds__(BN_THREADS)
maxpool_bwd_kernel(const T* __restrict__ dy, const uint8_t* __restrict__ arg, T* __restrict__ dx, size_t rows, int H, int W, int HO, int WO) {
    const int per_line = W / V;
    const size_t total = rows * H * per_line;
    constexpr int NC = V == 1 ? 2 : V / 2 + 1;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int iw0 = (int)(idx % per_line) * V;
        const int ih = (int)((idx / per_line) % H);
        const size_t row = idx / ((size_t)per_line * H);
        const size_t obase = row * HO * WO;
        float acc[V];
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = 0.f;
        for (int oh = ih >> 1; oh <= (ih + 1) >> 1; ++oh) {
            if (oh >= HO) continue;
            const int kh = ih - (2 * oh - 1);
            const int ow0 = iw0 >> 1;                      // window ow covers input columns 2*ow - 1 .. 2*ow + 1
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                const int ow = ow0 + j;
                if (ow >= WO) continue;
                const size_t o = obase + (size_t)oh * WO + ow;
                const int a = arg[o];
                if (a / 3 != kh) continue;
                const int e = 2 * ow - 1 + a % 3 - iw0;    // position of the maximum relative to iw0
                const float g = DType<T>::load(dy + o);
#pragma unroll
                for (int q = 0; q < V; ++q) if (q == e) acc[q] += g;
            }
        }
        VecIO<T, V>::store(dx + (row * H + ih) * W + iw0, acc);
    }
}

// ---- batch-norm + ReLU + 3x3 stride-2 max pooling in one (the network's stem) ----------------------------------------------
// Forward: the pooled maximum of relu(x * k0 + k1) straight from x -- the normalised full-size tensor is never written.
// Lines of a multiple of 8 pixels, an even number of lines; same window scan order and arg-max encoding as maxpool_fwd4_kernel.
template <typename T>
__global__ void __launch_bounds__(BN_THREADS)
bn_relu_pool_fwd_kernel(const T* __restrict__ x, BnCoef coef, T* __restrict__ y, uint8_t* __restrict__ arg, size_t rows, int C,
                        int H, int W, int HO, int WO) {
    bn_coef_outputs<0>(coef, C);
    const int groups = WO / 4;
    const size_t total = rows * HO * groups;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int g = (int)(idx % groups);
        const int oh = (int)((idx / groups) % HO);
        const size_t row = idx / ((size_t)groups * HO);
        const int c = (int)(row % C);
        float k0, k1, k2;
        bn_coef<0>(coef, C, c, k0, k1, k2);
        const T* src = x + row * H * W;
        float best[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        int where[4] = {0, 0, 0, 0};
#pragma unroll
        for (int kh = 0; kh < 3; ++kh) {
            const int ih = 2 * oh - 1 + kh;
            if ((unsigned)ih >= (unsigned)H) continue;
            float f[8];
            VecIO<T, 8>::load(src + (size_t)ih * W + 8 * g, f);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = fmaxf(fmaf(f[e], k0, k1), 0.f);
            const float left = g > 0 ? fmaxf(fmaf(DType<T>::load(src + (size_t)ih * W + 8 * g - 1), k0, k1), 0.f) : 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
                for (int kw = 0; kw < 3; ++kw) {
                    const int rel = 2 * j - 1 + kw;
                    if (rel < 0 && g == 0) continue;
                    const float v = rel < 0 ? left : f[rel];
                    if (v > best[j] || (v != v)) { best[j] = v; where[j] = kh * 3 + kw; }
                }
            }
        }
        const size_t o = (row * HO + oh) * WO + 4 * g;
        VecIO<T, 4>::store(y + o, best);
        *reinterpret_cast<uint32_t*>(arg + o) = (uint32_t)where[0] | ((uint32_t)where[1] << 8) | ((uint32_t)where[2] << 16) | ((uint32_t)where[3] << 24);
    }
}

// Backward sums (g, g * x) per channel, g being the pooled gradient routed to its arg-max pixel and masked by
// relu'(x * m0 + m1). The sums run over the POOLED outputs: each contributes its gradient once, at the pixel its arg-max byte
// names (always inside the image: the forward pass only compares pixels that exist), so the pass reads the pooled gradient,
// the arg-max bytes and one element of x per output instead of gathering around every input pixel.
template <typename T>
__global__ void __launch_bounds__(BN_THREADS)
bn_pool_sums_kernel(const T* __restrict__ x, const T* __restrict__ dp, const uint8_t* __restrict__ arg, float* __restrict__ sums, int planes, int C,
                    int H, int W, int HO, int WO, BnFwdParams fw) {
    const int c = blockIdx.x, s = blockIdx.y, S = gridDim.y;
    float m0, m1;
    bn_fwd_coef(fw, c, m0, m1);
    const int per_line = WO / 4, per_plane = HO * per_line;
    const int my_planes = s < planes ? (planes - s + S - 1) / S : 0;
    float a0 = 0.f, a1 = 0.f;
    for (int j = threadIdx.x; j < my_planes * per_plane; j += BN_THREADS) {
        const int pi = j / per_plane, r = j - pi * per_plane, oh = r / per_line, g = r - oh * per_line;
        const size_t row = (size_t)(s + pi * S) * C + c;
        const size_t o = (row * HO + oh) * WO + 4 * g;
        const uint32_t a4 = __ldg(reinterpret_cast<const uint32_t*>(arg + o));
        float g4[4];
        VecIO<T, 4>::load(dp + o, g4);
        const T* xr = x + row * H * W;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int a = (int)((a4 >> (8 * jj)) & 0xffu);
            const int akh = (a * 11) >> 5, akw = a - 3 * akh;          // a / 3 and a % 3 for a in 0..8
            const int ih = 2 * oh - 1 + akh, iw = 2 * (4 * g + jj) - 1 + akw;
            const float xv = DType<T>::load(xr + (size_t)ih * W + iw);
            if (fmaf(xv, m0, m1) > 0.f) { a0 += g4[jj]; a1 = fmaf(g4[jj], xv, a1); }
        }
    }
    __shared__ float red[2][BN_THREADS / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { a0 += __shfl_xor_sync(0xffffffffu, a0, o); a1 += __shfl_xor_sync(0xffffffffu, a1, o); }
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = a0; red[1][threadIdx.x >> 5] = a1; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float t0 = 0.f, t1 = 0.f;
#pragma unroll
        for (int w = 0; w < BN_THREADS / 32; ++w) { t0 += red[0][w]; t1 += red[1][w]; }
        atomicAdd(sums + c, t0);
        atomicAdd(sums + C + c, t1);
    }
}

// The gradient that reaches the 2 x 8 input pixels of lines 2r and 2r + 1, columns 8g .. 8g + 7: window line r holds line 2r
// as its middle line (kh = 1) and line 2r + 1 as its last (kh = 2), window line r + 1 holds line 2r + 1 as its first (kh = 0).
// The arg-max bytes and gradients of the five windows per window line are read and decoded once for both input lines.
template <typename T>
__device__ __forceinline__ void pool_gather2x8(const T* __restrict__ dp, const uint8_t* __restrict__ arg, size_t obase, int r, int g, int HO, int WO,
                                               float (&even)[8], float (&odd)[8]) {
#pragma unroll
    for (int e = 0; e < 8; ++e) even[e] = odd[e] = 0.f;
#pragma unroll
    for (int line = 0; line < 2; ++line) {
        const int oh = r + line;
        if (oh >= HO) continue;
        const size_t o = obase + (size_t)oh * WO + 4 * g;
        const uint32_t a4 = __ldg(reinterpret_cast<const uint32_t*>(arg + o));
        float g4[4];
        VecIO<T, 4>::load(dp + o, g4);
#pragma unroll
        for (int j = 0; j < 5; ++j) {
            int a;
            float gr;
            if (j < 4) { a = (int)((a4 >> (8 * j)) & 0xffu); gr = g4[j]; }
            else {
                if (4 * g + 4 >= WO) continue;
                a = arg[o + 4]; gr = DType<T>::load(dp + o + 4);
            }
            const int akh = (a * 11) >> 5, akw = a - 3 * akh;          // a / 3 and a % 3 for a in 0..8
            // window line r: kh = 1 -> even input line, kh = 2 -> odd input line; window line r + 1: kh = 0 -> odd input line
            const float me = (line == 0 && akh == 1) ? gr : 0.f;
            const float mo = (line == 0 ? akh == 2 : akh == 0) ? gr : 0.f;
            if (2 * j - 1 >= 0) { even[(2 * j - 1) & 7] += akw == 0 ? me : 0.f; odd[(2 * j - 1) & 7] += akw == 0 ? mo : 0.f; }
            if (2 * j < 8) { even[(2 * j) & 7] += akw == 1 ? me : 0.f; odd[(2 * j) & 7] += akw == 1 ? mo : 0.f; }
            if (2 * j + 1 < 8) { even[(2 * j + 1) & 7] += akw == 2 ? me : 0.f; odd[(2 * j + 1) & 7] += akw == 2 ? mo : 0.f; }
        }
    }
}

// dx = coef0 * g + coef1 * x + coef2 with g gathered from the pooled gradient and masked by relu'(x * m0 + m1); one thread
// per 2 x 8 input pixels (H is even).
template <typename T>
__global__ void __launch_bounds__(BN_THREADS)
bn_pool_apply_kernel(const T* __restrict__ x, const T* __restrict__ dp, const uint8_t* __restrict__ arg, T* __restrict__ dx,
                     BnCoef coef, size_t rows, int C, int H, int W, int HO, int WO, BnFwdParams fw) {
    bn_coef_outputs<1>(coef, C);
    const int per_line = W / 8, pairs = H / 2;
    const size_t total = rows * pairs * per_line;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int g = (int)(idx % per_line);
        const int r = (int)((idx / per_line) % pairs);
        const size_t row = idx / ((size_t)per_line * pairs);
        const int c = (int)(row % C);
        float k0, k1, k2;
        bn_coef<1>(coef, C, c, k0, k1, k2);
        float m0, m1;
        bn_fwd_coef(fw, c, m0, m1);
        float ge[8], go[8];
        pool_gather2x8<T>(dp, arg, row * HO * WO, r, g, HO, WO, ge, go);
#pragma unroll
        for (int line = 0; line < 2; ++line) {
            float fx[8], fo[8];
            const size_t off = (row * H + 2 * r + line) * W + 8 * g;
            VecIO<T, 8>::load(x + off, fx);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float gv = line == 0 ? ge[e] : go[e];
                const float gg = fmaf(fx[e], m0, m1) > 0.f ? gv : 0.f;
                fo[e] = fmaf(k0, gg, fmaf(k1, fx[e], k2));
            }
            VecIO<T, 8>::store(dx + off, fo);
        }
    }
}

int blocks_for(size_t work) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t cap = (size_t)sms * 16, need = (work + BN_THREADS - 1) / BN_THREADS;
    return (int)(need < cap ? (need ? need : 1) : cap);
}

// Widest vector (8, 4 or 1 elements) that rows of HW elements starting at these pointers allow; BN_FLAT where the rows
// allow none but the tensor as a whole is a sequence of aligned 8-element groups (see bn_sums_flat_kernel).
constexpr int BN_FLAT = -8;
int vec_width(int HW, uintptr_t ptr_bits, size_t total = 0, int C = 0) {
    if (HW % 8 == 0 && ptr_bits % 16 == 0) return 8;
    if (HW % 4 == 0 && ptr_bits % 8 == 0) return 4;
    if (total && total % 8 == 0 && ptr_bits % 16 == 0 && HW >= 8 && C <= 4096) return BN_FLAT;
    return 1;
}

template <typename T, int MODE, int V>
void bn_launch(const T* x, const T* y, const T* dy, T* out, float* scratch, BnCoef coef, int planes, int C, int HW, int relu, bool sums,
               cudaStream_t stream, const T* res, T* dres, BnFwdParams fw) {
    if (sums) {
        int S = (8 * 148 + C - 1) / C;
        if (S > planes) S = planes;
        if (S < 1) S = 1;
        bn_sums_kernel<T, MODE, V><<<dim3(C, S), BN_THREADS, 0, stream>>>(x, y, dy, scratch, planes, C, HW, relu, fw);
    } else {
        const size_t rows = (size_t)planes * C;
        bn_apply_kernel<T, MODE, V><<<blocks_for(rows * (HW / V)), BN_THREADS, 0, stream>>>(x, y, dy, out, coef, rows, C, HW, relu, res, dres, fw);
    }
}

template <typename T, int MODE>
void bn_dispatch(int V, const T* x, const T* y, const T* dy, T* out, float* scratch, BnCoef coef, int planes, int C, int HW, int relu, bool sums,
                 cudaStream_t stream, const T* res = nullptr, T* dres = nullptr, BnFwdParams fw = BnFwdParams{nullptr, nullptr, nullptr, nullptr}) {
    if (V == BN_FLAT) {
        const size_t groups = (size_t)planes * C * HW / 8;
        if (sums) {
            const size_t want = (groups + BN_THREADS - 1) / BN_THREADS;
            const int blocks = (int)(want < 4 * 148 ? (want ? want : 1) : 4 * 148);
            bn_sums_flat_kernel<T, MODE><<<blocks, BN_THREADS, 2 * C * sizeof(float), stream>>>(x, y, dy, scratch, groups, C, HW, relu, fw);
        } else {
            bn_apply_flat_kernel<T, MODE><<<blocks_for(groups), BN_THREADS, 0, stream>>>(x, y, dy, out, coef, groups, C, HW, relu, res, dres, fw);
        }
    } else if (V == 8) bn_launch<T, MODE, 8>(x, y, dy, out, scratch, coef, planes, C, HW, relu, sums, stream, res, dres, fw);
    else if (V == 4) bn_launch<T, MODE, 4>(x, y, dy, out, scratch, coef, planes, C, HW, relu, sums, stream, res, dres, fw);
    else bn_launch<T, MODE, 1>(x, y, dy, out, scratch, coef, planes, C, HW, relu, sums, stream, res, dres, fw);
}

template <typename T>
int bn_fwd_typed(const T* x, const float* gamma, const float* beta, T* y, float* mean, float* invstd, float* scratch, int planes, int C, int HW,
                 float eps, int relu, cudaStream_t stream, const T* res = nullptr) {
    const int V = vec_width(HW, reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(res), (size_t)planes * C * HW, C);
    PCB_CUDA_TRY(cudaMemsetAsync(scratch, 0, 2 * C * sizeof(float), stream));
    const BnCoef coef = {scratch, gamma, beta, nullptr, nullptr, mean, invstd, (float)planes * HW, eps};
    bn_dispatch<T, 0>(V, x, nullptr, nullptr, nullptr, scratch, coef, planes, C, HW, 0, true, stream);
    bn_dispatch<T, 0>(V, x, nullptr, nullptr, y, scratch, coef, planes, C, HW, relu, false, stream, res, nullptr);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

template <typename T>
int bn_bwd_typed(const T* x, const T* y, const T* dy, const float* gamma, const float* mean, const float* invstd, T* dx, float* dgamma, float* dbeta,
                 float* scratch, int planes, int C, int HW, int relu, cudaStream_t stream, T* dres = nullptr, const float* beta = nullptr) {
    const int V = vec_width(HW, reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx) |
                                    reinterpret_cast<uintptr_t>(dres) | (relu == 1 ? reinterpret_cast<uintptr_t>(y) : 0), (size_t)planes * C * HW, C);
    const BnFwdParams fw = {gamma, beta, mean, invstd};
    PCB_CUDA_TRY(cudaMemsetAsync(scratch, 0, 2 * C * sizeof(float), stream));
    const BnCoef coef = {scratch, gamma, nullptr, mean, invstd, dgamma, dbeta, (float)planes * HW, 0.f};
    bn_dispatch<T, 1>(V, x, y, dy, nullptr, scratch, coef, planes, C, HW, relu, true, stream, nullptr, nullptr, fw);
    bn_dispatch<T, 1>(V, x, y, dy, dx, scratch, coef, planes, C, HW, relu, false, stream, nullptr, dres, fw);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

template <typename T>
int bn_pool_fwd_typed(const T* x, const float* gamma, const float* beta, T* y, uint8_t* arg, float* mean, float* invstd, float* scratch, int planes, int C,
                      int H, int W, float eps, cudaStream_t stream) {
    const int HW = H * W, HO = H / 2, WO = W / 2;
    PCB_CUDA_TRY(cudaMemsetAsync(scratch, 0, 2 * C * sizeof(float), stream));
    const BnCoef coef = {scratch, gamma, beta, nullptr, nullptr, mean, invstd, (float)planes * HW, eps};
    bn_dispatch<T, 0>(8, x, nullptr, nullptr, nullptr, scratch, coef, planes, C, HW, 0, true, stream);
    const size_t rows = (size_t)planes * C;
    bn_relu_pool_fwd_kernel<T><<<blocks_for(rows * HO * (WO / 4)), BN_THREADS, 0, stream>>>(x, coef, y, arg, rows, C, H, W, HO, WO);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

template <typename T>
int bn_pool_bwd_typed(const T* x, const T* dp, const uint8_t* arg, const float* gamma, const float* beta, const float* mean, const float* invstd, T* dx,
                      float* dgamma, float* dbeta, float* scratch, int planes, int C, int H, int W, cudaStream_t stream) {
    const int HO = H / 2, WO = W / 2;
    const BnFwdParams fw = {gamma, beta, mean, invstd};
    PCB_CUDA_TRY(cudaMemsetAsync(scratch, 0, 2 * C * sizeof(float), stream));
    const BnCoef coef = {scratch, gamma, nullptr, mean, invstd, dgamma, dbeta, (float)planes * H * W, 0.f};
    int S = (8 * 148 + C - 1) / C;
    if (S > planes) S = planes;
    if (S < 1) S = 1;
    bn_pool_sums_kernel<T><<<dim3(C, S), BN_THREADS, 0, stream>>>(x, dp, arg, scratch, planes, C, H, W, HO, WO, fw);
    const size_t rows = (size_t)planes * C;
    bn_pool_apply_kernel<T><<<blocks_for(rows * (H / 2) * (W / 8)), BN_THREADS, 0, stream>>>(x, dp, arg, dx, coef, rows, C, H, W, HO, WO, fw);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

}  // namespace
}  // namespace pcb

extern "C" {

// Shapes the fused batch-norm + ReLU + max-pool kernels take: lines of a multiple of 8 pixels, an even number of them, 16-byte aligned tensors.
static bool bn_pool_shape_ok(int h, int w, const void* a, const void* b, const void* c) {
    return h > 0 && w > 0 && h % 2 == 0 && w % 8 == 0 &&
           ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15u) == 0;
}

int pcb_aux_bn_relu_maxpool_fwd(int dtype, const void* x, const float* gamma, const float* beta, void* y, void* argmax, float* mean, float* invstd,
                                float* scratch, int planes, int channels, int h, int w, float eps, void* stream) {
    using namespace pcb;
    if (!x || !gamma || !beta || !y || !argmax || !mean || !invstd || !scratch || planes <= 0 || channels <= 0) {
        set_error("invalid batch-norm arguments");
        return PCB_ERR_INVALID_ARGUMENT;
    }
    if (!bn_pool_shape_ok(h, w, x, y, argmax)) { set_error("fused batch-norm + pooling: lines of a multiple of 8 pixels, an even number of lines, 16-byte aligned tensors"); return PCB_ERR_UNSUPPORTED; }
    if (dtype == PCB_F16) return bn_pool_fwd_typed<__half>((const __half*)x, gamma, beta, (__half*)y, (uint8_t*)argmax, mean, invstd, scratch, planes, channels, h, w, eps, (cudaStream_t)stream);
    if (dtype == PCB_BF16) return bn_pool_fwd_typed<__nv_bfloat16>((const __nv_bfloat16*)x, gamma, beta, (__nv_bfloat16*)y, (uint8_t*)argmax, mean, invstd, scratch, planes, channels, h, w, eps, (cudaStream_t)stream);
    set_error("batch-norm helper: 16-bit tensors only");
    return PCB_ERR_UNSUPPORTED;
}

int pcb_aux_bn_relu_maxpool_bwd(int dtype, const void* x, const void* dy, const void* argmax, const float* gamma, const float* beta, const float* mean,
                                const float* invstd, void* dx, float* dgamma, float* dbeta, float* scratch, int planes, int channels, int h, int w,
                                void* stream) {
    using namespace pcb;
    if (!x || !dy || !argmax || !gamma || !beta || !mean || !invstd || !dx || !dgamma || !dbeta || !scratch || planes <= 0 || channels <= 0) {
        set_error("invalid batch-norm arguments");
        return PCB_ERR_INVALID_ARGUMENT;
    }
    if (!bn_pool_shape_ok(h, w, x, dy, dx) || (reinterpret_cast<uintptr_t>(argmax) & 15u)) { set_error("fused batch-norm + pooling: lines of a multiple of 8 pixels, an even number of lines, 16-byte aligned tensors"); return PCB_ERR_UNSUPPORTED; }
    if (dtype == PCB_F16) return bn_pool_bwd_typed<__half>((const __half*)x, (const __half*)dy, (const uint8_t*)argmax, gamma, beta, mean, invstd, (__half*)dx, dgamma, dbeta, scratch, planes, channels, h, w, (cudaStream_t)stream);
    if (dtype == PCB_BF16) return bn_pool_bwd_typed<__nv_bfloat16>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (const uint8_t*)argmax, gamma, beta, mean, invstd, (__nv_bfloat16*)dx, dgamma, dbeta, scratch, planes, channels, h, w, (cudaStream_t)stream);
    set_error("batch-norm helper: 16-bit tensors only");
    return PCB_ERR_UNSUPPORTED;
}

int pcb_aux_bn_relu_fwd(int dtype, const void* x, const float* gamma, const float* beta, void* y, float* mean, float* invstd, float* scratch,
                        int planes, int channels, int hw, float eps, int relu, void* stream) {
    using namespace pcb;
    if (!x || !gamma || !beta || !y || !mean || !invstd || !scratch || planes <= 0 || channels <= 0 || hw <= 0) {
        set_error("invalid batch-norm arguments");
        return PCB_ERR_INVALID_ARGUMENT;
    }
    if (dtype == PCB_F16) return bn_fwd_typed<__half>((const __half*)x, gamma, beta, (__half*)y, mean, invstd, scratch, planes, channels, hw, eps, relu, (cudaStream_t)stream);
    if (dtype == PCB_BF16) return bn_fwd_typed<__nv_bfloat16>((const __nv_bfloat16*)x, gamma, beta, (__nv_bfloat16*)y, mean, invstd, scratch, planes, channels, hw, eps, relu, (cudaStream_t)stream);
    set_error("batch-norm helper: 16-bit tensors only");
    return PCB_ERR_UNSUPPORTED;
}

int pcb_aux_bn_relu_bwd(int dtype, const void* x, const void* y, const void* dy, const float* gamma, const float* mean, const float* invstd, void* dx,
                        float* dgamma, float* dbeta, float* scratch, int planes, int channels, int hw, int relu, void* stream) {
    using namespace pcb;
    if (!x || !dy || !gamma || !mean || !invstd || !dx || !dgamma || !dbeta || !scratch || (relu && !y) || planes <= 0 || channels <= 0 || hw <= 0) {
        set_error("invalid batch-norm arguments");
        return PCB_ERR_INVALID_ARGUMENT;
    }
    if (dtype == PCB_F16) return bn_bwd_typed<__half>((const __half*)x, (const __half*)y, (const __half*)dy, gamma, mean, invstd, (__half*)dx, dgamma, dbeta, scratch, planes, channels, hw, relu, (cudaStream_t)stream);
    if (dtype == PCB_BF16) return bn_bwd_typed<__nv_bfloat16>((const __nv_bfloat16*)x, (const __nv_bfloat16*)y, (const __nv_bfloat16*)dy, gamma, mean, invstd, (__nv_bfloat16*)dx, dgamma, dbeta, scratch, planes, channels, hw, relu, (cudaStream_t)stream);
    set_error("batch-norm helper: 16-bit tensors only");
    return PCB_ERR_UNSUPPORTED;
}

int pcb_aux_bn_relu_bwd_from_input(int dtype, const void* x, const void* dy, const float* gamma, const float* beta, const float* mean,
                                   const float* invstd, void* dx, float* dgamma, float* dbeta, float* scratch, int planes, int channels, int hw,
                                   void* stream) {
    using namespace pcb;
    if (!x || !dy || !gamma || !beta || !mean || !invstd || !dx || !dgamma || !dbeta || !scratch || planes <= 0 || channels <= 0 || hw <= 0) {
        set_error("invalid batch-norm arguments");
        return PCB_ERR_INVALID_ARGUMENT;
    }
    if (dtype == PCB_F16) return bn_bwd_typed<__half>((const __half*)x, nullptr, (const __half*)dy, gamma, mean, invstd, (__half*)dx, dgamma, dbeta, scratch, planes, channels, hw, 2, (cudaStream_t)stream, nullptr, beta);
    if (dtype == PCB_BF16) return bn_bwd_typed<__nv_bfloat16>((const __nv_bfloat16*)x, nullptr, (const __nv_bfloat16*)dy, gamma, mean, invstd, (__nv_bfloat16*)dx, dgamma, dbeta, scratch, planes, channels, hw, 2, (cudaStream_t)stream, nullptr, beta);
    set_error("batch-norm helper: 16-bit tensors only");
    return PCB_ERR_UNSUPPORTED;
}

int pcb_aux_bn_add_relu_fwd(int dtype, const void* x, const void* residual, const float* gamma, const float* beta, void* y, float* mean, float* invstd,
                            float* scratch, int planes, int channels, int hw, float eps, void* stream) {
    using namespace pcb;
    if (!x || !residual || !gamma || !beta || !y || !mean || !invstd || !scratch || planes <= 0 || channels <= 0 || hw <= 0) {
        set_error("invalid batch-norm arguments");
        return PCB_ERR_INVALID_ARGUMENT;
    }
    if (dtype == PCB_F16) return bn_fwd_typed<__half>((const __half*)x, gamma, beta, (__half*)y, mean, invstd, scratch, planes, channels, hw, eps, 1, (cudaStream_t)stream, (const __half*)residual);
    if (dtype == PCB_BF16) return bn_fwd_typed<__nv_bfloat16>((const __nv_bfloat16*)x, gamma, beta, (__nv_bfloat16*)y, mean, invstd, scratch, planes, channels, hw, eps, 1, (cudaStream_t)stream, (const __nv_bfloat16*)residual);
    set_error("batch-norm helper: 16-bit tensors only");
    return PCB_ERR_UNSUPPORTED;
}

int pcb_aux_bn_add_relu_bwd(int dtype, const void* x, const void* y, const void* dy, const float* gamma, const float* mean, const float* invstd, void* dx,
                            void* dresidual, float* dgamma, float* dbeta, float* scratch, int planes, int channels, int hw, void* stream) {
    using namespace pcb;
    if (!x || !y || !dy || !gamma || !mean || !invstd || !dx || !dresidual || !dgamma || !dbeta || !scratch || planes <= 0 || channels <= 0 || hw <= 0) {
        set_error("invalid batch-norm arguments");
        return PCB_ERR_INVALID_ARGUMENT;
    }
    if (dtype == PCB_F16) return bn_bwd_typed<__half>((const __half*)x, (const __half*)y, (const __half*)dy, gamma, mean, invstd, (__half*)dx, dgamma, dbeta, scratch, planes, channels, hw, 1, (cudaStream_t)stream, (__half*)dresidual);
    if (dtype == PCB_BF16) return bn_bwd_typed<__nv_bfloat16>((const __nv_bfloat16*)x, (const __nv_bfloat16*)y, (const __nv_bfloat16*)dy, gamma, mean, invstd, (__nv_bfloat16*)dx, dgamma, dbeta, scratch, planes, channels, hw, 1, (cudaStream_t)stream, (__nv_bfloat16*)dresidual);
    set_error("batch-norm helper: 16-bit tensors only");
    return PCB_ERR_UNSUPPORTED;
}

int pcb_aux_maxpool3x3s2_fwd(int dtype, const void* x, void* y, void* argmax, int rows, int h, int w, void* stream) {
    using namespace pcb;
    if (!x || !y || !argmax || rows <= 0 || h <= 0 || w <= 0) { set_error("invalid max-pool arguments"); return PCB_ERR_INVALID_ARGUMENT; }
    const int ho = (h - 1) / 2 + 1, wo = (w - 1) / 2 + 1;
    const bool lines8 = w % 8 == 0 && wo % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 8 == 0 &&
                        reinterpret_cast<uintptr_t>(argmax) % 4 == 0;
    if (lines8 && (dtype == PCB_F16 || dtype == PCB_BF16)) {
        const int b4 = blocks_for((size_t)rows * ho * (wo / 4));
        if (dtype == PCB_F16) maxpool_fwd4_kernel<__half><<<b4, BN_THREADS, 0, (cudaStream_t)stream>>>((const __half*)x, (__half*)y, (uint8_t*)argmax, rows, h, w, ho, wo);
        else maxpool_fwd4_kernel<__nv_bfloat16><<<b4, BN_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, (uint8_t*)argmax, rows, h, w, ho, wo);
        PCB_CUDA_TRY(cudaGetLastError());
        return PCB_OK;
    }
    const int blocks = blocks_for((size_t)rows * ho * wo);
    if (dtype == PCB_F16) maxpool_fwd_kernel<__half><<<blocks, BN_THREADS, 0, (cudaStream_t)stream>>>((const __half*)x, (__half*)y, (uint8_t*)argmax, rows, h, w, ho, wo);
    else if (dtype == PCB_BF16) maxpool_fwd_kernel<__nv_bfloat16><<<blocks, BN_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, (uint8_t*)argmax, rows, h, w, ho, wo);
    else { set_error("max-pool helper: 16-bit tensors only"); return PCB_ERR_UNSUPPORTED; }
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

int pcb_aux_maxpool3x3s2_bwd(int dtype, const void* dy, const void* argmax, void* dx, int rows, int h, int w, void* stream) {
    using namespace pcb;
    if (!dy || !dx || !argmax || rows <= 0 || h <= 0 || w <= 0) { set_error("invalid max-pool arguments"); return PCB_ERR_INVALID_ARGUMENT; }
    const int ho = (h - 1) / 2 + 1, wo = (w - 1) / 2 + 1;
    if (dtype != PCB_F16 && dtype != PCB_BF16) { set_error("max-pool helper: 16-bit tensors only"); return PCB_ERR_UNSUPPORTED; }
    const bool wide = w % 8 == 0 && reinterpret_cast<uintptr_t>(dx) % 16 == 0;
    const int blocks = blocks_for((size_t)rows * h * (wide ? w / 8 : w));
    cudaStream_t st = (cudaStream_t)stream;
    if (wide && wo % 4 == 0 && reinterpret_cast<uintptr_t>(dy) % 8 == 0 && reinterpret_cast<uintptr_t>(argmax) % 4 == 0) {
        if (dtype == PCB_F16) maxpool_bwd8_kernel<__half><<<blocks, BN_THREADS, 0, st>>>((const __half*)dy, (const uint8_t*)argmax, (__half*)dx, rows, h, w, ho, wo);
        else maxpool_bwd8_kernel<__nv_bfloat16><<<blocks, BN_THREADS, 0, st>>>((const __nv_bfloat16*)dy, (const uint8_t*)argmax, (__nv_bfloat16*)dx, rows, h, w, ho, wo);
        PCB_CUDA_TRY(cudaGetLastError());
        return PCB_OK;
    }
    if (dtype == PCB_F16) {
        if (wide) maxpool_bwd_kernel<__half, 8><<<blocks, BN_THREADS, 0, st>>>((const __half*)dy, (const uint8_t*)argmax, (__half*)dx, rows, h, w, ho, wo);
        else maxpool_bwd_kernel<__half, 1><<<blocks, BN_THREADS, 0, st>>>((const __half*)dy, (const uint8_t*)argmax, (__half*)dx, rows, h, w, ho, wo);
    } else {
        if (wide) maxpool_bwd_kernel<__nv_bfloat16, 8><<<blocks, BN_THREADS, 0, st>>>((const __nv_bfloat16*)dy, (const uint8_t*)argmax, (__nv_bfloat16*)dx, rows, h, w, ho, wo);
        else maxpool_bwd_kernel<__nv_bfloat16, 1><<<blocks, BN_THREADS, 0, st>>>((const __nv_bfloat16*)dy, (const uint8_t*)argmax, (__nv_bfloat16*)dx, rows, h, w, ho, wo);
    }
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

}  // extern "C"
