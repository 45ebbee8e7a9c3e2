// CUDA-core (fp32 FMA) quaternion implicit-GEMM kernels: the fp32-exact path of the backend and the
// family that covers every geometry (any stride, padding, dilation, channel count).
//
// Each pass is ONE real GEMM  C[M,N] = sum_K A[M,K] * B[K,N]  in which the quaternion structure lives in
// the index maps, so no per-component intermediate tensor is ever written:
//
//   forward          M = (d, co)   N = (img, oh, ow)   K = (tap, l, ci)
//                    A = sign(l,d) * w[l^d][co][ci][tap]        B = x[l][img][ci][oh*s-p+kh][ow*s-p+kw]
//   backward-data    M = (l, ci)   N = (img, ih, iw)   K = (tap, d, co)
//                    A = sign(l,d) * w[l^d][co][ci][tap]        B = dy[d][img][co][(ih+p-kh)/s][(iw+p-kw)/s]
//   backward-filter  M = (r, co)   N = (ci, tap)       K = (l, img, oh, ow)      (split over K)
//                    A = sign(l,l^r) * dy[l^r][img][co][oh][ow] B = x[l][img][ci][oh*s-p+kh][ow*s-p+kw]
//
// (reference arithmetic being replaced: the 16 scalar library calls plus 12/24 accumulate passes of
//  src/conv2d.hpp:237-275 and :522-562, and the CUDA-core 1x1 kernels of
//  src/backend/cudnn/quat_pointwise_conv2d.cu:33-607.)
//
// Index decoding is table driven: per CTA one table for its M rows and one for its N columns (built
// once), and per K step a small table for the K slice, so the inner gather is two shared-memory reads,
// a bounds test and one global load per element.
#include <mutex>

#include "common.cuh"

namespace pcb {
namespace {

constexpr int BK = 16;
constexpr int THREADS = 256;

struct SimtParams {
    Geom g;
    int M, N, K;
    int ck;             // quaternion components folded into K (see make_k_entry)
    int k_per_split;    // K range handled by one blockIdx.z
    int atomic_out;     // accumulate into fp32 `out32` with atomics (split-K)
};

__device__ __forceinline__ int pack16(int lo, int hi) { return (lo & 0xffff) | (hi << 16); }
__device__ __forceinline__ int unpack_lo(int v) { return (int)(short)(v & 0xffff); }
__device__ __forceinline__ int unpack_hi(int v) { return v >> 16; }

// ---- table builders ------------------------------------------------------------------------------
template <int PASS>
__device__ __forceinline__ int4 make_m_entry(const Geom& g, int m, int M) {
    if (m >= M) return make_int4(-1, 0, 0, 0);
    if (PASS == PASS_FWD) {
        const int d = m / g.Co, co = m - d * g.Co;
        return make_int4(d, co * g.wo, (d * g.Nb) * g.yp + co * g.yc, d * g.bias_ld + co);
    } else if (PASS == PASS_BWD_DATA) {
        const int l = m / g.Ci, ci = m - l * g.Ci;
        return make_int4(l, ci * g.wi, (l * g.Nb) * g.xp + ci * g.xc, 0);
    } else {
        const int r = m / g.Co, co = m - r * g.Co;
        return make_int4(r, co * g.yc, r * g.dr + co * g.dco, 0);
    }
}

template <int PASS>
__device__ __forceinline__ int4 make_n_entry(const Geom& g, int n, int N) {
    if (n >= N) return make_int4(0, -30000, -30000, -1);
    const int T = g.KH * g.KW;
    const int P = g.HO * g.WO;
    if (PASS == PASS_FWD) {
        const int img = n / P, p = n - img * P;
        const int oh = p / g.WO, ow = p - oh * g.WO;
        return make_int4(img * g.xp, oh * g.SH - g.PT, ow * g.SW - g.PL, img * g.yp + oh * g.yh + ow * g.yw);
    } else if (PASS == PASS_BWD_DATA) {
        const int HW = g.H * g.W;
        const int img = n / HW, p = n - img * HW;
        const int ih = p / g.W, iw = p - ih * g.W;
        return make_int4(img * g.yp, ih + g.PT, iw + g.PL, img * g.xp + ih * g.xh + iw * g.xw);
    } else {
        const int ci = n / T, tap = n - ci * T;
        const int kh = tap / g.KW, kw = tap - kh * g.KW;
        return make_int4(ci * g.xc, kh * g.DH, kw * g.DW, ci * g.dci + kh * g.dkh + kw * g.dkw);
    }
}

// ck = number of components folded into the K index (all of the algebra's, or 1 when only one component runs
// along K: real-valued inputs and the 8-product kernels).
template <int PASS>
__device__ __forceinline__ int4 make_k_entry(const Geom& g, int k, int kend, int ck) {
    if (k >= kend) return make_int4(-1, 0, 0, 0);
    const int P = g.HO * g.WO;
    if (PASS == PASS_FWD) {
        const int tap = k / (ck * g.Ci);
        const int rem = k - tap * (ck * g.Ci);
        const int l = rem / g.Ci, ci = rem - l * g.Ci;
        const int kh = tap / g.KW, kw = tap - kh * g.KW;
        return make_int4(l, (l * g.Nb) * g.xp + ci * g.xc, pack16(kh * g.DH, kw * g.DW), ci * g.wi + kh * g.wh + kw * g.ww);
    } else if (PASS == PASS_BWD_DATA) {
        const int tap = k / (ck * g.Co);
        const int rem = k - tap * (ck * g.Co);
        const int d = rem / g.Co, co = rem - d * g.Co;
        const int kh = tap / g.KW, kw = tap - kh * g.KW;
        return make_int4(d, (d * g.Nb) * g.yp + co * g.yc, pack16(kh * g.DH, kw * g.DW), co * g.wo + kh * g.wh + kw * g.ww);
    } else {
        const int NP = g.Nb * P;
        const int l = k / NP;
        const int rem = k - l * NP;
        const int img = rem / P, p = rem - img * P;
        const int oh = p / g.WO, ow = p - oh * g.WO;
        return make_int4(l, img * g.yp + oh * g.yh + ow * g.yw, pack16(oh * g.SH - g.PT, ow * g.SW - g.PL), (l * g.Nb + img) * g.xp);
    }
}

// ---- element gathers -----------------------------------------------------------------------------
template <int PASS, typename T>
__device__ __forceinline__ float gather_a(const Geom& g, const T* __restrict__ a, int4 me, int4 ke) {
    if (me.x < 0 || ke.x < 0) return 0.f;
    if (PASS == PASS_FWD) {
        const int d = me.x, l = ke.x;
        const float v = DType<T>::load(a + (size_t)alg_pair(g.ga, l, d) * g.wr + me.y + ke.w);
        return alg_negative(g.neg, l, d) ? -v : v;
    } else if (PASS == PASS_BWD_DATA) {
        const int l = me.x, d = ke.x;
        const float v = DType<T>::load(a + (size_t)alg_pair(g.ga, l, d) * g.wr + me.y + ke.w);
        return alg_negative(g.neg, l, d) ? -v : v;
    } else {
        const int r = me.x, l = ke.x, d = alg_pair(g.ga, l, r);
        const float v = DType<T>::load(a + (size_t)(d * g.Nb) * g.yp + me.y + ke.y);
        return alg_negative(g.neg, l, d) ? -v : v;
    }
}

template <int PASS, typename T>
__device__ __forceinline__ float gather_b(const Geom& g, const T* __restrict__ b, int4 ne, int4 ke) {
    if (ke.x < 0) return 0.f;
    if (PASS == PASS_FWD) {
        const int ih = ne.y + unpack_lo(ke.z), iw = ne.z + unpack_hi(ke.z);
        if ((unsigned)ih >= (unsigned)g.H || (unsigned)iw >= (unsigned)g.W) return 0.f;
        return DType<T>::load(b + (size_t)ke.y + ne.x + ih * g.xh + iw * g.xw);
    } else if (PASS == PASS_BWD_DATA) {
        const int th = ne.y - unpack_lo(ke.z), tw = ne.z - unpack_hi(ke.z);
        if (th < 0 || tw < 0) return 0.f;
        const int oh = th / g.SH, ow = tw / g.SW;
        if (oh * g.SH != th || ow * g.SW != tw || oh >= g.HO || ow >= g.WO) return 0.f;
        return DType<T>::load(b + (size_t)ke.y + ne.x + oh * g.yh + ow * g.yw);
    } else {
        if (ne.w < 0) return 0.f;
        const int ih = unpack_lo(ke.z) + ne.y, iw = unpack_hi(ke.z) + ne.z;
        if ((unsigned)ih >= (unsigned)g.H || (unsigned)iw >= (unsigned)g.W) return 0.f;
        return DType<T>::load(b + (size_t)ke.w + ne.x + ih * g.xh + iw * g.xw);
    }
}

// ---- the kernel ----------------------------------------------------------------------------------
// BM x BN output tile, BK-deep slices, 256 threads as a 16x16 grid; each thread owns (BM/16) x (BN/16)
// outputs arranged as groups of 4 consecutive rows / columns 64 apart (conflict-free float4 reads).
// A_KFAST / B_KFAST pick which index runs fastest across threads when gathering (the one that is
// contiguous in memory for the pass).
template <int PASS, typename T, int BM, int BN, bool A_KFAST, bool B_KFAST>
__global__ void __launch_bounds__(THREADS)
qgemm_simt_kernel(SimtParams p, const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ bias,
                  T* __restrict__ out, float* __restrict__ out32) {
    constexpr int TM = BM / 16, TN = BN / 16;
    constexpr int PADM = BM + 4, PADN = BN + 4;
    __shared__ __align__(16) float As[BK * PADM];
    __shared__ __align__(16) float Bs[BK * PADN];
    __shared__ int4 mtab[BM];
    __shared__ int4 ntab[BN];
    __shared__ int4 ktab[BK];

    const Geom& g = p.g;
    const int t = threadIdx.x;
    const int tx = t & 15, ty = t >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int kbeg = blockIdx.z * p.k_per_split;
    const int kend = min(p.K, kbeg + p.k_per_split);

    for (int i = t; i < BM; i += THREADS) mtab[i] = make_m_entry<PASS>(g, m0 + i, p.M);
    for (int i = t; i < BN; i += THREADS) ntab[i] = make_n_entry<PASS>(g, n0 + i, p.N);
    __syncthreads();

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = kbeg; k0 < kend; k0 += BK) {
        __syncthreads();   // previous slice fully consumed; tables of the first iteration visible below
        if (t < BK) ktab[t] = make_k_entry<PASS>(g, k0 + t, kend, p.ck);
        __syncthreads();

        // gather A: BM*BK elements
#pragma unroll
        for (int j = 0; j < (BM * BK) / THREADS; ++j) {
            int kk, mm;
            if (A_KFAST) { kk = t % BK; mm = t / BK + j * (THREADS / BK); }
            else         { mm = t % BM; kk = t / BM + j * (THREADS / BM); }
            As[kk * PADM + mm] = gather_a<PASS, T>(g, a, mtab[mm], ktab[kk]);
        }
#pragma unroll
        for (int j = 0; j < (BN * BK) / THREADS; ++j) {
            int kk, nn;
            if (B_KFAST) { kk = t % BK; nn = t / BK + j * (THREADS / BK); }
            else         { nn = t % BN; kk = t / BN + j * (THREADS / BN); }
            Bs[kk * PADN + nn] = gather_b<PASS, T>(g, b, ntab[nn], ktab[kk]);
        }
        __syncthreads();

#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[TM], bv[TN];
#pragma unroll
            for (int gi = 0; gi < TM / 4; ++gi) {
                const float4 v = *reinterpret_cast<const float4*>(&As[kk * PADM + gi * 64 + ty * 4]);
                av[gi * 4 + 0] = v.x; av[gi * 4 + 1] = v.y; av[gi * 4 + 2] = v.z; av[gi * 4 + 3] = v.w;
            }
#pragma unroll
            for (int gj = 0; gj < TN / 4; ++gj) {
                const float4 v = *reinterpret_cast<const float4*>(&Bs[kk * PADN + gj * 64 + tx * 4]);
                bv[gj * 4 + 0] = v.x; bv[gj * 4 + 1] = v.y; bv[gj * 4 + 2] = v.z; bv[gj * 4 + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }

    // epilogue: output offset = M part + N part for every pass
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int mm = (i / 4) * 64 + ty * 4 + (i & 3);
        const int4 me = mtab[mm];
        if (me.x < 0) continue;
        float badd = 0.f;
        if (PASS == PASS_FWD && g.has_bias) badd = DType<T>::load(bias + me.w);
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int nn = (j / 4) * 64 + tx * 4 + (j & 3);
            if (n0 + nn >= p.N) continue;
            const int4 ne = ntab[nn];
            const size_t off = (size_t)me.z + (size_t)ne.w;
            if (p.atomic_out) atomicAdd(out32 + off, acc[i][j]);
            else DType<T>::store(out + off, acc[i][j] + badd);
        }
    }
}

template <typename T>
__global__ void cast_from_f32_kernel(const float* __restrict__ src, T* __restrict__ dst, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) DType<T>::store(dst + i, src[i]);
}

int device_sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    return sms;
}

void problem_dims(Pass pass, const Geom& g, int& M, int& N, int& K) {
    const int T = g.KH * g.KW, P = g.HO * g.WO, LK = g.real_in ? 1 : g.nc;
    if (pass == PASS_FWD)           { M = g.nc * g.Co;  N = g.Nb * P;         K = T * LK * g.Ci; }
    else if (pass == PASS_BWD_DATA) { M = g.nc * g.Ci;  N = g.Nb * g.H * g.W; K = T * g.nc * g.Co; }
    else                            { M = g.nc * g.Co;  N = g.Ci * T;         K = LK * g.Nb * P; }
}

size_t filter_numel(const Geom& g) { return (size_t)g.nc * g.Co * g.Ci * g.KH * g.KW; }

template <int PASS, typename T, int BM, int BN, bool AK, bool BKF>
int launch_one(const SimtParams& p, int splits, const void* a, const void* b, const void* bias, void* out, float* out32,
               cudaStream_t stream) {
    dim3 grid((p.N + BN - 1) / BN, (p.M + BM - 1) / BM, splits);
    qgemm_simt_kernel<PASS, T, BM, BN, AK, BKF><<<grid, THREADS, 0, stream>>>(
        p, (const T*)a, (const T*)b, (const T*)bias, (T*)out, out32);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

template <int PASS, typename T, bool AK, bool BKF>
int launch_sized(bool small, const SimtParams& p, const void* a, const void* b, const void* bias, void* out, cudaStream_t stream) {
    return small ? launch_one<PASS, T, 64, 64, AK, BKF>(p, 1, a, b, bias, out, nullptr, stream)
                 : launch_one<PASS, T, 128, 128, AK, BKF>(p, 1, a, b, bias, out, nullptr, stream);
}

template <typename T>
int launch_typed(Pass pass, const Geom& g, const void* a, const void* b, const void* bias, void* out, float* scratch,
                 cudaStream_t stream) {
    SimtParams p;
    p.g = g;
    problem_dims(pass, g, p.M, p.N, p.K);
    p.ck = (pass == PASS_BWD_DATA || !g.real_in) ? g.nc : 1;
    p.k_per_split = p.K;
    p.atomic_out = 0;
    if (p.M == 0 || p.N == 0) return PCB_OK;
    const bool small = ((long long)((p.M + 127) / 128) * ((p.N + 127) / 128)) < device_sm_count();

    // Gather order per operand: the index that is contiguous in memory runs fastest across threads.
    //   weights [r][co][ci][tap] (OIHW/OI): forward K=(ci,tap) contiguous; backward-data M=ci (stride taps)
    //   weights [r][ci][co] (IO):           forward M=co contiguous;       backward-data K=co contiguous
    //   activations: pixels contiguous (N) for images; for dense layers (1x1 images) channels (K) are.
    const bool dense_like = (g.H * g.W == 1) && (g.HO * g.WO == 1);
    if (pass == PASS_FWD) {
        const bool ak = !g.w_io;
        if (ak && dense_like)  return launch_sized<PASS_FWD, T, true, true>(small, p, a, b, bias, out, stream);
        if (ak && !dense_like) return launch_sized<PASS_FWD, T, true, false>(small, p, a, b, bias, out, stream);
        if (dense_like)        return launch_sized<PASS_FWD, T, false, true>(small, p, a, b, bias, out, stream);
        return launch_sized<PASS_FWD, T, false, false>(small, p, a, b, bias, out, stream);
    }
    if (pass == PASS_BWD_DATA) {
        const bool ak = g.w_io;
        if (ak && dense_like)  return launch_sized<PASS_BWD_DATA, T, true, true>(small, p, a, b, bias, out, stream);
        if (ak && !dense_like) return launch_sized<PASS_BWD_DATA, T, true, false>(small, p, a, b, bias, out, stream);
        if (dense_like)        return launch_sized<PASS_BWD_DATA, T, false, true>(small, p, a, b, bias, out, stream);
        return launch_sized<PASS_BWD_DATA, T, false, false>(small, p, a, b, bias, out, stream);
    }
    // backward-filter: tiny M x N, huge K -> split K over the grid and accumulate with fp32 atomics
    const int tiles = ((p.M + 63) / 64) * ((p.N + 63) / 64);
    int splits = (2 * device_sm_count() + tiles - 1) / tiles;
    const int max_splits = (p.K + 8 * BK - 1) / (8 * BK);
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    int kps = (p.K + splits - 1) / splits;
    kps = (kps + BK - 1) / BK * BK;
    splits = (p.K + kps - 1) / kps;
    p.k_per_split = kps;
    const size_t numel = filter_numel(g);
    if (splits == 1) return launch_one<PASS_BWD_FILTER, T, 64, 64, true, true>(p, 1, a, b, bias, out, nullptr, stream);
    p.atomic_out = 1;
    float* acc32 = sizeof(T) == 4 ? (float*)out : scratch;
    if (acc32 == nullptr) { set_error("backward-filter needs fp32 scratch for 16-bit outputs"); return PCB_ERR_WORKSPACE; }
    PCB_CUDA_TRY(cudaMemsetAsync(acc32, 0, numel * sizeof(float), stream));
    int rc = launch_one<PASS_BWD_FILTER, T, 64, 64, true, true>(p, splits, a, b, bias, out, acc32, stream);
    if (rc != PCB_OK) return rc;
    if (sizeof(T) != 4) {
        const int blocks = (int)((numel + 255) / 256 < 1184 ? (numel + 255) / 256 : 1184);
        cast_from_f32_kernel<T><<<blocks, 256, 0, stream>>>(acc32, (T*)out, numel);
        PCB_CUDA_TRY(cudaGetLastError());
    }
    return PCB_OK;
}


// ===================================================================================================
// 8-product (factorised) variant. The reference forms 8 "lane" tensors from the 4 components of each
// operand, runs 8 real convolutions and recombines (src/conv2d.hpp:167-234, :433-519; lane formulas
// src/backend/onednn/tensor.hpp:62-170). Here the lane sums are formed in registers while gathering, the
// 8 lane products accumulate side by side in one thread, and the recombination happens in the epilogue:
// a batched GEMM over lanes  C_i[M,N] = sum_K A_i[M,K] * B_i[K,N]  with
//   forward          M = co, N = (img,oh,ow), K = (tap,ci):   A_i = Wl_i(w),  B_i = Xl_i(x)
//   backward-data    M = ci, N = (img,ih,iw), K = (tap,co):   A_i = Wl_i(w),  B_i = Gl_i(dy)
//   backward-filter  M = co, N = (ci,tap),    K = (img,oh,ow): A_i = Gl_i(dy), B_i = Xl_i(x)
// ===================================================================================================
constexpr int BK8 = 8, BM8 = 32, BN8 = 128;

__device__ __forceinline__ void lanes_x(const float x[4], float o[8]) {
    o[0] = x[3] + x[1]; o[1] = x[0] - x[2]; o[2] = x[0] + x[2]; o[3] = x[3] - x[1];
    o[4] = x[3] - x[2]; o[5] = x[1] + x[0]; o[6] = x[0] - x[1]; o[7] = x[3] + x[2];
}
__device__ __forceinline__ void lanes_w(const float w[4], float o[8]) {
    o[0] = w[1] + w[2]; o[1] = w[0] + w[3]; o[2] = w[0] - w[3]; o[3] = w[1] - w[2];
    o[4] = w[2] - w[3]; o[5] = w[1] + w[0]; o[6] = w[2] + w[3]; o[7] = w[0] - w[1];
}
__device__ __forceinline__ void lanes_g(const float g[4], float o[8]) {
    const float t1 = g[0] + g[1], t3 = g[0] - g[1], t2 = g[2] + g[3], t4 = g[2] - g[3];
    o[0] = 0.5f * (t2 - t1); o[1] = 0.5f * (t3 - t4); o[2] = 0.5f * (t3 + t4); o[3] = 0.5f * (t1 + t2);
    o[4] = g[0]; o[5] = g[1]; o[6] = g[2]; o[7] = g[3];
}

template <int PASS, typename T>
__global__ void __launch_bounds__(THREADS)
qgemm8_simt_kernel(SimtParams p, const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ bias,
                   T* __restrict__ out, float* __restrict__ out32) {
    __shared__ __align__(16) float As[8 * BK8 * BM8];
    __shared__ __align__(16) float Bs[8 * BK8 * BN8];
    __shared__ int4 mtab[BM8];
    __shared__ int4 ntab[BN8];
    __shared__ int4 ktab[BK8];

    const Geom& g = p.g;
    const int t = threadIdx.x;
    const int tx = t & 31, ty = t >> 5;
    const int m0 = blockIdx.y * BM8, n0 = blockIdx.x * BN8;
    const int kbeg = blockIdx.z * p.k_per_split;
    const int kend = min(p.K, kbeg + p.k_per_split);
    const size_t w_comp = (size_t)g.wr;                    // one component of the filters
    const size_t x_comp = (size_t)g.Nb * g.xp;             // one component of the input
    const size_t y_comp = (size_t)g.Nb * g.yp;             // one component of the output

    for (int i = t; i < BM8; i += THREADS) mtab[i] = make_m_entry<PASS>(g, m0 + i, p.M);
    for (int i = t; i < BN8; i += THREADS) ntab[i] = make_n_entry<PASS>(g, n0 + i, p.N);
    __syncthreads();

    float acc[8][4][4];
#pragma unroll
    for (int l = 0; l < 8; ++l)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[l][i][j] = 0.f;

    for (int k0 = kbeg; k0 < kend; k0 += BK8) {
        __syncthreads();
        if (t < BK8) ktab[t] = make_k_entry<PASS>(g, k0 + t, kend, 1);
        __syncthreads();

        {   // A operand: BM8*BK8 = 256 elements, one per thread
            int kk, mm;
            if (PASS == PASS_BWD_DATA) { mm = t % BM8; kk = t / BM8; }     // ci contiguous
            else                       { kk = t % BK8; mm = t / BK8; }     // (ci,tap) resp. pixels contiguous
            const int4 me = mtab[mm], ke = ktab[kk];
            float c[4] = {0.f, 0.f, 0.f, 0.f}, lanes[8];
            if (me.x >= 0 && ke.x >= 0) {
                if (PASS == PASS_BWD_FILTER) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) c[q] = DType<T>::load(a + q * y_comp + me.y + ke.y);
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q) c[q] = DType<T>::load(a + q * w_comp + me.y + ke.w);
                }
            }
            if (PASS == PASS_BWD_FILTER) lanes_g(c, lanes); else lanes_w(c, lanes);
#pragma unroll
            for (int l = 0; l < 8; ++l) As[(l * BK8 + kk) * BM8 + mm] = lanes[l];
        }
#pragma unroll
        for (int j = 0; j < (BN8 * BK8) / THREADS; ++j) {   // B operand: 4 elements per thread
            int kk, nn;
            if (PASS == PASS_BWD_FILTER) { kk = t % BK8; nn = t / BK8 + j * (THREADS / BK8); }
            else                         { nn = t % BN8; kk = t / BN8 + j * (THREADS / BN8); }
            const int4 ne = ntab[nn], ke = ktab[kk];
            float c[4] = {0.f, 0.f, 0.f, 0.f}, lanes[8];
            if (ke.x >= 0 && ne.w >= 0) {
                if (PASS == PASS_FWD) {
                    const int ih = ne.y + unpack_lo(ke.z), iw = ne.z + unpack_hi(ke.z);
                    if ((unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W) {
                        const T* src = b + (size_t)ke.y + ne.x + ih * g.xh + iw * g.xw;
#pragma unroll
                        for (int q = 0; q < 4; ++q) c[q] = DType<T>::load(src + q * x_comp);
                    }
                } else if (PASS == PASS_BWD_DATA) {
                    const int th = ne.y - unpack_lo(ke.z), tw = ne.z - unpack_hi(ke.z);
                    const int oh = th / g.SH, ow = tw / g.SW;
                    if (th >= 0 && tw >= 0 && oh * g.SH == th && ow * g.SW == tw && oh < g.HO && ow < g.WO) {
                        const T* src = b + (size_t)ke.y + ne.x + oh * g.yh + ow * g.yw;
#pragma unroll
                        for (int q = 0; q < 4; ++q) c[q] = DType<T>::load(src + q * y_comp);
                    }
                } else {
                    const int ih = unpack_lo(ke.z) + ne.y, iw = unpack_hi(ke.z) + ne.z;
                    if ((unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W) {
                        const T* src = b + (size_t)ke.w + ne.x + ih * g.xh + iw * g.xw;
#pragma unroll
                        for (int q = 0; q < 4; ++q) c[q] = DType<T>::load(src + q * x_comp);
                    }
                }
            }
            if (PASS == PASS_BWD_DATA) lanes_g(c, lanes); else lanes_x(c, lanes);
#pragma unroll
            for (int l = 0; l < 8; ++l) Bs[(l * BK8 + kk) * BN8 + nn] = lanes[l];
        }
        __syncthreads();

#pragma unroll
        for (int kk = 0; kk < BK8; ++kk)
#pragma unroll
            for (int l = 0; l < 8; ++l) {
                const float4 av = *reinterpret_cast<const float4*>(&As[(l * BK8 + kk) * BM8 + ty * 4]);
                const float4 bv = *reinterpret_cast<const float4*>(&Bs[(l * BK8 + kk) * BN8 + tx * 4]);
                const float aa[4] = {av.x, av.y, av.z, av.w}, bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[l][i][j] = fmaf(aa[i], bb[j], acc[l][i][j]);
            }
    }

    // epilogue: recombine the 8 lanes into the 4 components and write them
    const size_t out_comp = PASS == PASS_FWD ? y_comp : (PASS == PASS_BWD_DATA ? x_comp : (size_t)g.dr);   // the gradient has its own component stride
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int4 me = mtab[ty * 4 + i];
        if (me.x < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int nn = tx * 4 + j;
            if (n0 + nn >= p.N) continue;
            const int4 ne = ntab[nn];
            float L[8], o[4];
#pragma unroll
            for (int l = 0; l < 8; ++l) L[l] = acc[l][i][j];
            if (PASS == PASS_FWD) {             // src/backend/onednn/tensor.hpp:131-136
                const float a2 = L[0] + L[1] + L[2];
                const float a5 = 0.5f * (a2 + L[3]);
                o[0] = a5 - L[0] + L[4]; o[1] = a5 - a2 + L[5]; o[2] = a5 - L[1] + L[6]; o[3] = a5 - L[2] + L[7];
                if (g.has_bias) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) o[q] += DType<T>::load(bias + q * g.bias_ld + me.w);
                }
            } else if (PASS == PASS_BWD_DATA) { // src/backend/onednn/tensor.hpp:150-153
                o[0] = L[1] + L[2] + L[5] + L[6]; o[1] = L[0] - L[3] + L[5] - L[6];
                o[2] = L[2] - L[1] - L[4] + L[7]; o[3] = L[0] + L[3] + L[4] + L[7];
            } else {                            // src/backend/onednn/tensor.hpp:164-167
                o[0] = L[1] + L[2] + L[5] + L[7]; o[1] = L[0] + L[3] + L[5] - L[7];
                o[2] = L[0] - L[3] + L[4] + L[6]; o[3] = L[1] - L[2] - L[4] + L[6];
            }
            const size_t off = (size_t)me.z + (size_t)ne.w;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if (p.atomic_out) atomicAdd(out32 + q * out_comp + off, o[q]);
                else DType<T>::store(out + q * out_comp + off, o[q]);
            }
        }
    }
}

template <int PASS, typename T>
int launch8_one(const SimtParams& p, int splits, const void* a, const void* b, const void* bias, void* out, float* out32,
                cudaStream_t stream) {
    dim3 grid((p.N + BN8 - 1) / BN8, (p.M + BM8 - 1) / BM8, splits);
    qgemm8_simt_kernel<PASS, T><<<grid, THREADS, 0, stream>>>(p, (const T*)a, (const T*)b, (const T*)bias, (T*)out, out32);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

template <typename T>
int launch8_typed(Pass pass, const Geom& g, const void* a, const void* b, const void* bias, void* out, float* scratch,
                  cudaStream_t stream) {
    SimtParams p;
    p.g = g;
    const int TAPS = g.KH * g.KW, P = g.HO * g.WO;
    if (pass == PASS_FWD)           { p.M = g.Co; p.N = g.Nb * P;         p.K = TAPS * g.Ci; }
    else if (pass == PASS_BWD_DATA) { p.M = g.Ci; p.N = g.Nb * g.H * g.W; p.K = TAPS * g.Co; }
    else                            { p.M = g.Co; p.N = g.Ci * TAPS;      p.K = g.Nb * P; }
    p.ck = 1;
    p.k_per_split = p.K;
    p.atomic_out = 0;
    if (p.M == 0 || p.N == 0) return PCB_OK;
    if (pass == PASS_FWD) return launch8_one<PASS_FWD, T>(p, 1, a, b, bias, out, nullptr, stream);
    if (pass == PASS_BWD_DATA) return launch8_one<PASS_BWD_DATA, T>(p, 1, a, b, bias, out, nullptr, stream);
    const int tiles = ((p.M + BM8 - 1) / BM8) * ((p.N + BN8 - 1) / BN8);
    int splits = (2 * device_sm_count() + tiles - 1) / tiles;
    const int max_splits = (p.K + 16 * BK8 - 1) / (16 * BK8);
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    int kps = (p.K + splits - 1) / splits;
    kps = (kps + BK8 - 1) / BK8 * BK8;
    splits = (p.K + kps - 1) / kps;
    p.k_per_split = kps;
    const size_t numel = filter_numel(g);
    if (splits == 1) return launch8_one<PASS_BWD_FILTER, T>(p, 1, a, b, bias, out, nullptr, stream);
    p.atomic_out = 1;
    float* acc32 = sizeof(T) == 4 ? (float*)out : scratch;
    if (acc32 == nullptr) { set_error("backward-filter needs fp32 scratch for 16-bit outputs"); return PCB_ERR_WORKSPACE; }
    PCB_CUDA_TRY(cudaMemsetAsync(acc32, 0, numel * sizeof(float), stream));
    int rc = launch8_one<PASS_BWD_FILTER, T>(p, splits, a, b, bias, out, acc32, stream);
    if (rc != PCB_OK) return rc;
    if (sizeof(T) != 4) {
        const int blocks = (int)((numel + 255) / 256 < 1184 ? (numel + 255) / 256 : 1184);
        cast_from_f32_kernel<T><<<blocks, 256, 0, stream>>>(acc32, (T*)out, numel);
        PCB_CUDA_TRY(cudaGetLastError());
    }
    return PCB_OK;
}

int simt8_launch(Pass pass, int dtype, const Geom& g, const void* a, const void* b, const void* bias, void* out,
                 float* scratch, cudaStream_t stream) {
    switch (dtype) {
        case PCB_F32: return launch8_typed<float>(pass, g, a, b, bias, out, scratch, stream);
        case PCB_F16: return launch8_typed<__half>(pass, g, a, b, bias, out, scratch, stream);
        case PCB_BF16: return launch8_typed<__nv_bfloat16>(pass, g, a, b, bias, out, scratch, stream);
    }
    set_error("unknown dtype %d", dtype);
    return PCB_ERR_INVALID_ARGUMENT;
}

}  // namespace

size_t simt_scratch_bytes(Pass pass, int dtype, int /*variant*/, const Geom& g) {
    if (pass == PASS_BWD_FILTER && dtype != PCB_F32) return filter_numel(g) * sizeof(float);
    return 0;
}

int simt_launch(Pass pass, int dtype, int variant, const Geom& g, const void* a, const void* b, const void* bias,
                void* out, float* scratch, cudaStream_t stream) {
    if (variant == PCB_VARIANT_8_PRODUCT && !g.real_in) return simt8_launch(pass, dtype, g, a, b, bias, out, scratch, stream);
    switch (dtype) {
        case PCB_F32: return launch_typed<float>(pass, g, a, b, bias, out, scratch, stream);
        case PCB_F16: return launch_typed<__half>(pass, g, a, b, bias, out, scratch, stream);
        case PCB_BF16: return launch_typed<__nv_bfloat16>(pass, g, a, b, bias, out, scratch, stream);
    }
    set_error("unknown dtype %d", dtype);
    return PCB_ERR_INVALID_ARGUMENT;
}

// ---------------------------------------------------------------------------------------------------
// Backward-filter without any caller- or library-allocated scratch.
//
// Some hosts of this library may not allocate device memory at all once they are running: a plugin that
// lives inside a framework which has handed the whole device heap to its own arena and forbids
// cudaMalloc from operator callbacks, or a deployment whose memory plan is frozen at start-up. For them
// the split-K accumulator of the filter gradient (needed when the tensors are fp16 / bf16) lives in a
// fixed array in the library's own device image instead of a workspace. The array costs
// STATIC_SCRATCH_FLOATS * 4 bytes on every GPU that loads the library, for the life of the process.
//
// The array's name is only a host-side handle; the device address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and cached. All calls on a device share the one
// array and it keeps whatever the previous call left, so every call zeroes the part it accumulates
// into first; two calls that overlap on the GPU (different streams) would race on it.
// ---------------------------------------------------------------------------------------------------
constexpr size_t STATIC_SCRATCH_FLOATS = size_t(4) << 20;     // 4 Mi floats = 16 MiB: up to 4*Co*Ci*kh*kw = 4,194,304
static __device__ __align__(256) float g_static_scratch[STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_static_scratch_addr[MAX_DEVICES] = {};
std::mutex g_static_scratch_mutex;
}  // namespace

size_t simt_static_scratch_capacity() { return STATIC_SCRATCH_FLOATS; }

int simt_bwd_filter_static(int dtype, int variant, const Geom& g, const void* dy, const void* x, void* dw, cudaStream_t stream) {
    const size_t need = filter_numel(g);
    if (need > STATIC_SCRATCH_FLOATS) {
        set_error("filter gradient of %zu elements exceeds the built-in scratch of %zu elements", need, (size_t)STATIC_SCRATCH_FLOATS);
        return PCB_ERR_TOO_LARGE;
    }
    int dev = -1;
    PCB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) { set_error("device index %d out of range", dev); return PCB_ERR_INVALID_ARGUMENT; }
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        if (g_static_scratch_addr[dev] == nullptr) {
            // first call on this device: resolve the device address of the array (do this before any stream capture)
            float* addr = nullptr;
            PCB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_static_scratch));
            g_static_scratch_addr[dev] = addr;
        }
        scratch = g_static_scratch_addr[dev];
    }
    return simt_launch(PASS_BWD_FILTER, dtype, variant, g, dy, x, nullptr, dw, scratch, stream);
}

}  // namespace pcb
