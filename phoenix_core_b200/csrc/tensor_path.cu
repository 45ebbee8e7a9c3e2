// tcgen05 / TMEM kernels for the quaternion operators with 16-bit operands (fp16 or bf16, fp32
// accumulation in tensor memory).
//
// Pointwise (1x1, stride 1, no padding) quaternion convolution, all three passes, as ONE real GEMM per
// pass whose M x K operand carries the quaternion structure:
//
//   forward          D[(d,co), (img,p)] = sum_{(l,ci)}   s(l,d) w[l^d][co][ci]      * x[l][img][ci][p]
//   backward-data    D[(l,ci), (img,p)] = sum_{(d,co)}   s(l,d) w[l^d][co][ci]      * dy[d][img][co][p]
//   backward-filter  D[(r,co), ci]      = sum_{(l,img,p)} s(l,l^r) dy[l^r][img][co][p] * x[l][img][ci][p]
//
// The 4x4 signed / permuted weight block (reference sign table src/algebras.cc:28-49) is never stored in
// global memory: producer warps read the four component tiles and write their signed copies straight into
// the shared-memory operand tile in the tcgen05 canonical layout (sign = one XOR on the fp16/bf16 sign
// bits, so it is exact). For the filter gradient the same is done to the dy operand. Replaces the
// CUDA-core 1x1 kernels of src/backend/cudnn/quat_pointwise_conv2d.cu:33-607 and, for 1x1 shapes, the 16
// cuDNN calls of src/conv2d.hpp:237-275 / :522-562.
//
// CTA = 5 warps. Warps 0-3 produce operand tiles (global -> registers -> swizzled shared memory) through a
// 3-stage ring of mbarriers, then become the epilogue (TMEM -> registers -> global). Warp 4 allocates
// tensor memory and its lane 0 issues tcgen05.mma. Tile 128 (M) x 128 (N) x 64 (K per stage); two CTAs
// fit on an SM (96 KB shared memory and 128 TMEM columns each), so one CTA's epilogue overlaps the
// other's main loop. Every barrier wait is bounded; on expiry a status word is set and the CTA runs to its
// normal teardown (TMEM is always released).
#include "tensor_path.cuh"
#include "umma.cuh"

namespace pcb {
extern int g_sm_margin;
namespace {

using namespace umma;

constexpr int TBM = 128, TBN = 128, TBK = 64, STAGES = 3;
constexpr int PRODUCER_THREADS = 128, TC_THREADS = 160;
constexpr uint32_t A_STAGE_BYTES = TBM * TBK * 2, B_STAGE_BYTES = TBN * TBK * 2;
constexpr uint32_t MN_BLOCK_BYTES = 64 * 128;          // one 64-element M/N block of an MN-major tile (64 K rows)
constexpr uint32_t TMEM_COLS = 128;
constexpr size_t TC_SMEM_BYTES = 1024 /*alignment slack*/ + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) +
                                 STAGES * 64 * sizeof(int4) + 512;

// status codes OR-ed into the workspace status word when a bounded wait expires
constexpr int ST_PRODUCER_TIMEOUT = 1, ST_MMA_TIMEOUT = 2, ST_EPILOGUE_TIMEOUT = 4;

struct TcParams {
    Geom g;
    int pass;
    int fmt;            // 0 = f16, 1 = bf16
    int M, N, K;
    int k_per_split;    // multiple of TBK
    int atomic_out;     // backward-filter: accumulate into fp32 scratch with atomics
};

__device__ __forceinline__ uint4 ld_chunk(const uint16_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void st_chunk(uint8_t* tile, uint32_t off, uint4 v) { *reinterpret_cast<uint4*>(tile + off) = v; }
__device__ __forceinline__ uint4 negate16(uint4 v) {
    v.x ^= 0x80008000u; v.y ^= 0x80008000u; v.z ^= 0x80008000u; v.w ^= 0x80008000u;
    return v;
}

// Row / column ("MN") part of an operand address: component selector `aux` (-1: out of range -> zeros)
// and element offset.
struct MnInfo { int aux; int off; };

template <int PASS>
__device__ __forceinline__ MnInfo a_mn_info(const Geom& g, int m, int M) {
    if (m >= M) return {-1, 0};
    const int HW = g.H * g.W;
    if (PASS == PASS_FWD) { const int d = m / g.Co, co = m - d * g.Co; return {d, co * g.Ci}; }
    if (PASS == PASS_BWD_DATA) { const int l = m / g.Ci, ci = m - l * g.Ci; return {l, ci}; }
    const int r = m / g.Co, co = m - r * g.Co;
    return {r, co * HW};
}
template <int PASS>
__device__ __forceinline__ MnInfo b_mn_info(const Geom& g, int n, int N) {
    if (n >= N) return {-1, 0};
    const int HW = g.H * g.W;
    if (PASS == PASS_BWD_FILTER) return {0, n * HW};                       // n = ci
    const int img = n / HW, p = n - img * HW;
    return {0, img * (PASS == PASS_FWD ? g.Ci : g.Co) * HW + p};
}
// K part: x = component selector (-1: beyond K), y = offset into the A operand, z = offset into B.
template <int PASS>
__device__ __forceinline__ int4 k_info(const Geom& g, int k, int kend) {
    if (k >= kend) return make_int4(-1, 0, 0, 0);
    const int HW = g.H * g.W;
    if (PASS == PASS_FWD) { const int l = k / g.Ci, ci = k - l * g.Ci; return make_int4(l, ci, ci * HW, 0); }
    if (PASS == PASS_BWD_DATA) { const int d = k / g.Co, co = k - d * g.Co; return make_int4(d, co * g.Ci, co * HW, 0); }
    const int NP = g.Nb * HW;
    const int l = k / NP, rem = k - l * NP;
    const int img = rem / HW, p = rem - img * HW;
    return make_int4(l, img * g.Co * HW + p, img * g.Ci * HW + p, 0);
}

// A operand is MN-major only for backward-data (ci is the contiguous index of the filters);
// B operand is K-major only for backward-filter (pixels are the contiguous index of x).
template <int PASS> struct Layout {
    static constexpr bool A_MN = (PASS == PASS_BWD_DATA);
    static constexpr bool B_MN = (PASS != PASS_BWD_FILTER);
};

template <int PASS>
__global__ void __launch_bounds__(TC_THREADS)
qgemm_tc_kernel(TcParams p, const uint16_t* __restrict__ a, const uint16_t* __restrict__ b, const uint16_t* __restrict__ bias,
                uint16_t* __restrict__ out, float* __restrict__ out32, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const Geom& g = p.g;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int HW = g.H * g.W;

    // carve shared memory: operand ring (1024-byte aligned), K tables, barriers, TMEM slot
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* a_tiles = base;
    uint8_t* b_tiles = base + STAGES * A_STAGE_BYTES;
    int4* ktab = reinterpret_cast<int4*>(b_tiles + STAGES * B_STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(ktab + STAGES * 64);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * STAGES + 1);
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + STAGES), ktab_bar = smem_u32(bars + 2 * STAGES),
                   accum_bar = smem_u32(bars + 3 * STAGES);

    const int m0 = blockIdx.y * TBM, n0 = blockIdx.x * TBN;
    const int kbeg = blockIdx.z * p.k_per_split;
    const int kend = min(p.K, kbeg + p.k_per_split);
    const int num_it = (kend - kbeg + TBK - 1) / TBK;

    if (t == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, PRODUCER_THREADS);
            mbar_init(empty_bar + 8 * s, 1);
            mbar_init(ktab_bar + 8 * s, 64);
        }
        mbar_init(accum_bar, 1);
        fence_barrier_init();
    }
    if (warp == 4) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
        // ------------------------------------------------------------------ producers
        // component strides of the two operands
        const int a_comp = PASS == PASS_BWD_FILTER ? g.Nb * g.Co * HW : g.Co * g.Ci;
        const int b_comp = PASS == PASS_BWD_DATA ? g.Nb * g.Co * HW : g.Nb * g.Ci * HW;
        // stage-invariant part of this thread's chunk coordinates
        MnInfo a_info[8], b_info[8];
        if (Layout<PASS>::A_MN) {
            a_info[0] = a_mn_info<PASS>(g, m0 + 8 * (t & 15), p.M);             // chunk column t%16 of an MN-major tile
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) a_info[j] = a_mn_info<PASS>(g, m0 + (t >> 3) + 16 * j, p.M);   // rows of a K-major tile
        }
        if (Layout<PASS>::B_MN) {
            b_info[0] = b_mn_info<PASS>(g, n0 + 8 * (t & 15), p.N);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) b_info[j] = b_mn_info<PASS>(g, n0 + (t >> 3) + 16 * j, p.N);
        }

        bool ok = true;
        for (int it = 0; it < num_it && ok; ++it) {
            const int s = it % STAGES;
            const uint32_t parity = ((it / STAGES) & 1) ^ 1;
            ok = mbar_wait_bounded(empty_bar + 8 * s, parity, status, ST_PRODUCER_TIMEOUT);
            if (!ok) break;
            const int k0 = kbeg + it * TBK;
            int4* kt = ktab + s * 64;
            if (t < 64) {
                kt[t] = k_info<PASS>(g, k0 + t, kend);
                mbar_arrive(ktab_bar + 8 * s);
            }
            ok = mbar_wait_bounded(ktab_bar + 8 * s, parity ^ 1, status, ST_PRODUCER_TIMEOUT);
            if (!ok) break;

            uint8_t* a_tile = a_tiles + s * A_STAGE_BYTES;
            uint8_t* b_tile = b_tiles + s * B_STAGE_BYTES;
            // ---- A operand: signed copies of the component tiles
            if (Layout<PASS>::A_MN) {
                const int c = t & 15;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int kr = (t >> 4) + 8 * j;
                    const int4 ke = kt[kr];
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (a_info[0].aux >= 0 && ke.x >= 0) {
                        const int l = a_info[0].aux, d = ke.x;                   // backward-data: rows carry l, K carries d
                        v = ld_chunk(a + (size_t)(l ^ d) * a_comp + a_info[0].off + ke.y);
                        if (quat_negative(l, d)) v = negate16(v);
                    }
                    st_chunk(a_tile, mnmajor_sw128_offset(kr, c, MN_BLOCK_BYTES), v);
                }
            } else {
                const int kc = t & 7;
                const int4 ke = kt[8 * kc];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int row = (t >> 3) + 16 * j;
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (a_info[j].aux >= 0 && ke.x >= 0) {
                        int l, d;
                        if (PASS == PASS_FWD) { d = a_info[j].aux; l = ke.x; }
                        else { l = ke.x; d = l ^ a_info[j].aux; }                 // backward-filter: rows carry r
                        v = ld_chunk(a + (size_t)(PASS == PASS_FWD ? (l ^ d) : d) * a_comp + a_info[j].off + ke.y);
                        if (quat_negative(l, d)) v = negate16(v);
                    }
                    st_chunk(a_tile, kmajor_sw128_offset(row, kc), v);
                }
            }
            // ---- B operand: activations, copied as they are
            if (Layout<PASS>::B_MN) {
                const int c = t & 15;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int kr = (t >> 4) + 8 * j;
                    const int4 ke = kt[kr];
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (b_info[0].aux >= 0 && ke.x >= 0) v = ld_chunk(b + (size_t)ke.x * b_comp + b_info[0].off + ke.z);
                    st_chunk(b_tile, mnmajor_sw128_offset(kr, c, MN_BLOCK_BYTES), v);
                }
            } else {
                const int kc = t & 7;
                const int4 ke = kt[8 * kc];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int row = (t >> 3) + 16 * j;
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (b_info[j].aux >= 0 && ke.x >= 0) v = ld_chunk(b + (size_t)ke.x * b_comp + b_info[j].off + ke.z);
                    st_chunk(b_tile, kmajor_sw128_offset(row, kc), v);
                }
            }
            fence_proxy_async_smem();
            mbar_arrive(full_bar + 8 * s);
        }

        // ------------------------------------------------------------------ epilogue
        if (ok) ok = mbar_wait_bounded(accum_bar, 0, status, ST_EPILOGUE_TIMEOUT);
        // one decision per warp (tcgen05.ld is warp-collective); nothing is written once any wait has expired
        ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
        tc_fence_after_sync();
        if (ok && num_it > 0) {
            const int m = m0 + warp * 32 + lane;                                 // TMEM lane == tile row
            const MnInfo mi = a_mn_info<PASS>(g, m, p.M);
            size_t row_off = 0;
            float badd = 0.f;
            if (mi.aux >= 0) {
                if (PASS == PASS_FWD) {
                    const int d = mi.aux, co = m - d * g.Co;
                    row_off = ((size_t)d * g.Nb * g.Co + co) * HW;
                    if (g.has_bias) {
                        const uint16_t raw = bias[d * g.Co + co];
                        badd = p.fmt == 0 ? __half2float(__ushort_as_half(raw)) : __bfloat162float(__ushort_as_bfloat16(raw));
                    }
                } else if (PASS == PASS_BWD_DATA) {
                    const int l = mi.aux, ci = m - l * g.Ci;
                    row_off = ((size_t)l * g.Nb * g.Ci + ci) * HW;
                } else {
                    row_off = (size_t)m * g.Ci;                                  // dw[r][co][ci], m = r*Co + co
                }
            }
#pragma unroll 1
            for (int cb = 0; cb < TBN / 32; ++cb) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(warp * 32) << 16) + cb * 32, v);
                tmem_ld_wait();
                if (mi.aux < 0) continue;
                if (PASS == PASS_BWD_FILTER) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int n = n0 + cb * 32 + c;
                        if (n < p.N) {
                            if (p.atomic_out) atomicAdd(out32 + row_off + n, __uint_as_float(v[c]));
                            else out32[row_off + n] = __uint_as_float(v[c]);
                        }
                    }
                } else {
                    const int out_c = PASS == PASS_FWD ? g.Co : g.Ci;
#pragma unroll
                    for (int c8 = 0; c8 < 4; ++c8) {
                        const int n = n0 + cb * 32 + c8 * 8;
                        if (n >= p.N) continue;
                        const int img = n / HW, px = n - img * HW;
                        uint32_t packed[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float f0 = __uint_as_float(v[c8 * 8 + 2 * q]) + badd;
                            const float f1 = __uint_as_float(v[c8 * 8 + 2 * q + 1]) + badd;
                            if (p.fmt == 0) {
                                const __half2 h = __floats2half2_rn(f0, f1);
                                packed[q] = *reinterpret_cast<const uint32_t*>(&h);
                            } else {
                                const __nv_bfloat162 h = __floats2bfloat162_rn(f0, f1);
                                packed[q] = *reinterpret_cast<const uint32_t*>(&h);
                            }
                        }
                        uint16_t* dst = out + row_off + (size_t)img * out_c * HW + px;
                        *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ MMA issuer (warp 4)
        const uint32_t idesc = make_idesc_f16(p.fmt, TBM, TBN, Layout<PASS>::A_MN, Layout<PASS>::B_MN);
        bool ok = true;
        for (int it = 0; it < num_it && ok; ++it) {
            const int s = it % STAGES;
            const uint32_t parity = (it / STAGES) & 1;
            ok = mbar_wait_bounded(full_bar + 8 * s, parity, status, ST_MMA_TIMEOUT);
            if (!ok) break;
            tc_fence_after_sync();
            if (lane == 0) {
                const uint32_t a_addr = smem_u32(a_tiles + s * A_STAGE_BYTES);
                const uint32_t b_addr = smem_u32(b_tiles + s * B_STAGE_BYTES);
#pragma unroll
                for (int j = 0; j < TBK / 16; ++j) {
                    // 16 K-elements per instruction: 32 bytes along a K-major row, 16 K-rows (2048 bytes) of an MN-major tile
                    const uint64_t ad = Layout<PASS>::A_MN ? make_desc_mnmajor(a_addr + j * 2048, MN_BLOCK_BYTES)
                                                           : make_desc_kmajor(a_addr + j * 32);
                    const uint64_t bd = Layout<PASS>::B_MN ? make_desc_mnmajor(b_addr + j * 2048, MN_BLOCK_BYTES)
                                                           : make_desc_kmajor(b_addr + j * 32);
                    mma_f16_ss(tmem_base, ad, bd, idesc, (it > 0 || j > 0) ? 1u : 0u);
                }
                mma_commit(empty_bar + 8 * s);          // frees the stage once these MMAs have read it
            }
            __syncwarp();
        }
        if (lane == 0 && num_it > 0 && ok) mma_commit(accum_bar);
        if (lane == 0 && (num_it == 0 || !ok)) mbar_arrive(accum_bar);   // never leave the epilogue waiting
        __syncwarp();
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 4) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <typename T>
__global__ void cast_f32_to_16_kernel(const float* __restrict__ src, T* __restrict__ dst, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) DType<T>::store(dst + i, src[i]);
}

int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    const int left = sms - g_sm_margin;      // see pcb_set_sm_margin
    return left < 2 ? 2 : left;
}

template <int PASS>
int launch_tc(const TcParams& p, int splits, const void* a, const void* b, const void* bias, void* out, float* out32,
              int* status, cudaStream_t stream) {
    PCB_CUDA_TRY(cudaFuncSetAttribute(qgemm_tc_kernel<PASS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_BYTES));
    dim3 grid((p.N + TBN - 1) / TBN, (p.M + TBM - 1) / TBM, splits);
    qgemm_tc_kernel<PASS><<<grid, TC_THREADS, TC_SMEM_BYTES, stream>>>(
        p, (const uint16_t*)a, (const uint16_t*)b, (const uint16_t*)bias, (uint16_t*)out, out32, status);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

bool pointwise(const Geom& g) {
    return g.KH == 1 && g.KW == 1 && g.SH == 1 && g.SW == 1 && g.PT == 0 && g.PL == 0 && g.HO == g.H && g.WO == g.W &&
           g.DH == 1 && g.DW == 1;
}


// ---------------------------------------------------------------------------------------------------
// Pointwise (1x1) layers with a stride touch only every SH-th row and SW-th column of the input: they run as
// stride-1 pointwise layers on a compact copy of those pixels (forward, filter gradient), or produce the compact
// input gradient and scatter it between zeros (backward-data). Without this the strided layers went through the
// general kernel, which staged the whole input and, backward, convolved a zero-inserted dy at full resolution.
// (reference: the same layers are ordinary strided cuDNN / oneDNN convolutions, src/backend/cudnn/conv2d.hpp:181-310)
// ---------------------------------------------------------------------------------------------------
template <int BYTES> struct VecBytes;
template <> struct VecBytes<2> { typedef uint16_t type; };
template <> struct VecBytes<4> { typedef uint32_t type; };
template <> struct VecBytes<8> { typedef uint2 type; };
template <> struct VecBytes<16> { typedef uint4 type; };

// dst[plane][oh][ow] = src[plane][oh*SH - PT][ow*SW - PL] (zero outside); planes = components * images * channels.
// V = 0: any stride and padding, one output per thread. V >= 1: V outputs per thread from one load of 2 V inputs;
// requires SW == 2, PL == 0, WO % V == 0, W % (2 V) == 0 and 16-byte aligned bases. Indices are 32-bit: tensors hold
// fewer than 2^31 elements.
template <typename E, int V>
__global__ void subsample_kernel(const E* __restrict__ src, E* __restrict__ dst, unsigned planes, int H, int W, int HO, int WO,
                                 int SH, int SW, int PT, int PL) {
    constexpr int VV = V > 0 ? V : 1;
    const unsigned wq = WO / VV;
    const unsigned total = planes * HO * wq;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const unsigned q = idx % wq, rest = idx / wq;
        const unsigned oh = rest % HO, plane = rest / HO;
        const int ih = (int)oh * SH - PT;
        alignas(16) E out[VV];
        if (V == 0) {
            const int iw = (int)q * SW - PL;
            out[0] = (ih >= 0 && ih < H && iw >= 0 && iw < W) ? src[((size_t)plane * H + ih) * W + iw] : E(0);
        } else {
            alignas(16) E in[2 * VV];
            typedef typename VecBytes<2 * VV * sizeof(E)>::type In;
            if (ih >= 0 && ih < H) *reinterpret_cast<In*>(in) = __ldg(reinterpret_cast<const In*>(src + ((size_t)plane * H + ih) * W + 2 * VV * q));
            else *reinterpret_cast<In*>(in) = In();
#pragma unroll
            for (int e = 0; e < VV; ++e) out[e] = in[2 * e];
        }
        typedef typename VecBytes<VV * sizeof(E)>::type Out;
        *reinterpret_cast<Out*>(dst + ((size_t)plane * HO + oh) * WO + (size_t)VV * q) = *reinterpret_cast<const Out*>(out);
    }
}

// dst[plane][ih][iw] = src[plane][oh][ow] where ih = oh*SH - PT, iw = ow*SW - PL, zero everywhere else.
// V = 0: any stride and padding, one destination element per thread. V >= 1: V source elements (2 V destination elements)
// per thread; requires SW == 2, PL == 0, W == 2 WO, W % (2 V) == 0 and 16-byte aligned bases.
template <typename E, int V>
__global__ void scatter_strided_kernel(const E* __restrict__ src, E* __restrict__ dst, unsigned planes, int H, int W, int HO, int WO,
                                       int SH, int SW, int PT, int PL) {
    constexpr int VV = V > 0 ? V : 1;
    const unsigned wq = V == 0 ? W : W / (2 * VV);
    const unsigned total = planes * H * wq;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const unsigned q = idx % wq, rest = idx / wq;
        const unsigned ih = rest % H, plane = rest / H;
        const int th = (int)ih + PT, oh = th / SH;
        const bool row = (th % SH == 0) && oh < HO;
        if (V == 0) {
            const int tw = (int)q + PL, ow = tw / SW;
            dst[((size_t)plane * H + ih) * W + q] = (row && tw % SW == 0 && ow < WO) ? src[((size_t)plane * HO + oh) * WO + ow] : E(0);
        } else {
            alignas(16) E in[VV], out[2 * VV];
            typedef typename VecBytes<VV * sizeof(E)>::type In;
            typedef typename VecBytes<2 * VV * sizeof(E)>::type Out;
            if (row) *reinterpret_cast<In*>(in) = __ldg(reinterpret_cast<const In*>(src + ((size_t)plane * HO + oh) * WO + (size_t)VV * q));
#pragma unroll
            for (int e = 0; e < VV; ++e) { out[2 * e] = row ? in[e] : E(0); out[2 * e + 1] = E(0); }
            *reinterpret_cast<Out*>(dst + ((size_t)plane * H + ih) * W + (size_t)2 * VV * q) = *reinterpret_cast<const Out*>(out);
        }
    }
}


// ---------------------------------------------------------------------------------------------------
// Backward-data of a strided layer with taps. dx[ih] collects only the taps kh with (ih + PT - kh) divisible by the
// stride, so the input pixels fall into SH x SW classes by (ih mod SH, iw mod SW), and the gradient of one class is the
// backward-data pass of a STRIDE-1 layer over the same dy whose filters are every SH-th / SW-th tap:
//     dx[SH i + a] = sum_k' dy[i + c - k'] w[r + SH k'],   r = (a + PT) mod SH,  c = (a + PT) div SH
// -- a layer with ceil((KH - r) / SH) taps and padding c before. Each class runs through the stride-1 kernels into a
// compact tensor and one kernel interleaves the classes into dx. The classes together execute the FLOPs of the layer;
// convolving a zero-inserted dy at full resolution, the route this replaces, executed SH x SW times as many.
// ---------------------------------------------------------------------------------------------------
struct StrideClass {
    int a, b;            // class: input row and column modulo the strides
    int rh, rw;          // first tap of the class
    Geom g;              // the stride-1 layer (g.KH == 0 or g.KW == 0: the class receives no tap, its pixels are zero)
    size_t dx_off, w_off;   // byte offsets of the compact gradient / the class's filters in the scratch area
};

// Taken from 512 gradient rows (128 quaternion channels) up: each class pays its own staging pass and launch, and below that
// width those cost more than the zero-insertion route's extra MMAs (measured at batch 128: 0.47 -> 0.38 ms at 128
// channels and 28 x 28, 0.51 -> 0.34 ms at 256 and 14 x 14, but 0.12 -> 0.27 ms at 64 -> 128 channels and 14 x 14).
// From 256 rows (64 quaternion channels) the classes also win when the gradient is large (at least ~200k pixels per component).
bool strided_taps(const Geom& g) {
    const bool wide = g.nc * g.Ci >= 512 || (g.nc * g.Ci >= 256 && (long long)g.Nb * g.H * g.W >= 200000);
    return (g.KH > 1 || g.KW > 1) && (g.SH > 1 || g.SW > 1) && g.SH <= 2 && g.SW <= 2 && g.DH == 1 && g.DW == 1 && g.plain && !g.w_io &&
           !g.dw_io && !g.real_in && wide;
}

// Fills the classes; returns their number. `bytes` receives the scratch the classes' tensors take.
int stride_classes(const Geom& g, int dtype, StrideClass* cls, size_t* bytes) {
    const size_t es = dtype_size(dtype);
    size_t off = 0;
    int n = 0;
    for (int a = 0; a < g.SH; ++a)
        for (int b = 0; b < g.SW; ++b) {
            StrideClass& c = cls[n++];
            c.a = a; c.b = b;
            c.rh = (a + g.PT) % g.SH; c.rw = (b + g.PL) % g.SW;
            Geom s = g;
            s.H = (g.H - a + g.SH - 1) / g.SH; s.W = (g.W - b + g.SW - 1) / g.SW;
            s.KH = c.rh < g.KH ? (g.KH - c.rh + g.SH - 1) / g.SH : 0;
            s.KW = c.rw < g.KW ? (g.KW - c.rw + g.SW - 1) / g.SW : 0;
            s.SH = s.SW = 1; s.PT = (a + g.PT) / g.SH; s.PL = (b + g.PL) / g.SW;
            s.xp = g.Ci * s.H * s.W; s.xc = s.H * s.W; s.xh = s.W; s.xw = 1;
            s.wr = g.Co * g.Ci * s.KH * s.KW; s.wo = g.Ci * s.KH * s.KW; s.wi = s.KH * s.KW; s.wh = s.KW; s.ww = 1;
            s.dr = s.wr; s.dco = s.wo; s.dci = s.wi; s.dkh = s.wh; s.dkw = s.ww;
            c.g = s;
            c.dx_off = off;
            off += ((size_t)g.nc * g.Nb * g.Ci * s.H * s.W * es + 1023) / 1024 * 1024;
            c.w_off = off;
            off += ((size_t)g.nc * g.Co * g.Ci * s.KH * s.KW * es + 1023) / 1024 * 1024;
        }
    *bytes = off;
    return n;
}

bool strided_classes_supported(int dtype, int variant, const Geom& g) {
    if (!strided_taps(g)) return false;
    StrideClass cls[4];
    size_t bytes;
    const int n = stride_classes(g, dtype, cls, &bytes);
    for (int i = 0; i < n; ++i) {
        const Geom& s = cls[i].g;
        if (s.H <= 0 || s.W <= 0) return false;
        if (s.KH == 0 || s.KW == 0) continue;
        if (!tensor_path_supported(PASS_BWD_DATA, dtype, variant, s)) return false;
    }
    return true;
}

// w_sub[r][co][ci][u][v] = w[r][co][ci][rh + SH u][rw + SW v]
template <typename E>
__global__ void gather_taps_kernel(const E* __restrict__ w, E* __restrict__ sub, unsigned rows /*components * Co * Ci*/, int KH, int KW,
                                   int KHs, int KWs, int rh, int rw, int SH, int SW) {
    const unsigned total = rows * KHs * KWs;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const unsigned v = idx % KWs, rest = idx / KWs;
        const unsigned u = rest % KHs, row = rest / KHs;
        sub[idx] = w[((size_t)row * KH + rh + SH * u) * KW + rw + SW * v];
    }
}

struct ClassPtrs { const void* p[4]; int H[4], W[4], live[4]; };

// dx[plane][ih][iw] = class (ih mod SH, iw mod SW) [plane][ih div SH][iw div SW], zero for a class without taps.
template <typename E>
__global__ void interleave_classes_kernel(ClassPtrs c, E* __restrict__ dx, unsigned planes, int H, int W, int SH, int SW) {
    const unsigned total = planes * H * W;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const unsigned iw = idx % W, rest = idx / W;
        const unsigned ih = rest % H, plane = rest / H;
        const int k = (ih % SH) * SW + (iw % SW);
        dx[idx] = c.live[k] ? static_cast<const E*>(c.p[k])[((size_t)plane * c.H[k] + ih / SH) * c.W[k] + iw / SW] : E(0);
    }
}
// The same for SH == SW == 2, 16-bit elements and W a multiple of 2 V: one thread writes 2 V pixels of a row from V + V
// pixels of the two classes of that row (V = 4, 2 or 1: stores of 16, 8 or 4 bytes).
template <int V>
__global__ void interleave_classes_2x2_kernel(ClassPtrs c, uint16_t* __restrict__ dx, unsigned planes, int H, int W) {
    typedef typename VecBytes<2 * V>::type In;
    typedef typename VecBytes<4 * V>::type Out;
    const unsigned wq = W / (2 * V), total = planes * H * wq;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const unsigned q = idx % wq, rest = idx / wq;
        const unsigned ih = rest % H, plane = rest / H;
        const int k0 = (ih & 1) * 2;
        alignas(8) uint16_t even[V], odd[V];
        alignas(16) uint16_t o[2 * V];
        if (c.live[k0])
            *reinterpret_cast<In*>(even) = __ldg(reinterpret_cast<const In*>(static_cast<const uint16_t*>(c.p[k0]) + ((size_t)plane * c.H[k0] + (ih >> 1)) * c.W[k0] + V * q));
        if (c.live[k0 + 1])
            *reinterpret_cast<In*>(odd) = __ldg(reinterpret_cast<const In*>(static_cast<const uint16_t*>(c.p[k0 + 1]) + ((size_t)plane * c.H[k0 + 1] + (ih >> 1)) * c.W[k0 + 1] + V * q));
#pragma unroll
        for (int e = 0; e < V; ++e) { o[2 * e] = c.live[k0] ? even[e] : (uint16_t)0; o[2 * e + 1] = c.live[k0 + 1] ? odd[e] : (uint16_t)0; }
        *reinterpret_cast<Out*>(dx + ((size_t)plane * H + ih) * W + 2 * V * q) = *reinterpret_cast<const Out*>(o);
    }
}

bool strided_pointwise(const Geom& g) {
    return g.KH == 1 && g.KW == 1 && (g.SH > 1 || g.SW > 1) && g.plain && !g.w_io && !g.dw_io;
}

// The stride-1 pointwise layer on the compact copy: input plane = output plane.
Geom compact_geom(const Geom& g) {
    Geom s = g;
    s.H = g.HO; s.W = g.WO; s.SH = s.SW = 1; s.PT = s.PL = 0;
    s.xp = g.Ci * s.H * s.W; s.xc = s.H * s.W; s.xh = s.W; s.xw = 1;
    return s;
}

size_t compact_bytes(Pass pass, int dtype, const Geom& g) {
    const size_t comps = (pass != PASS_BWD_DATA && g.real_in) ? 1 : g.nc;
    return (comps * g.Nb * g.Ci * g.HO * g.WO * dtype_size(dtype) + 1023) / 1024 * 1024;
}

template <typename E>
int launch_subsample(const void* src, void* dst, size_t planes, const Geom& g, cudaStream_t stream) {
    const bool al = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    const bool v = g.SW == 2 && g.PL == 0 && al && g.W >= 2 * g.WO;
    int V = 0;                                            // outputs per thread; loads of up to 16 bytes
    if (v && sizeof(E) == 2 && g.WO % 4 == 0 && g.W % 8 == 0) V = 4;
    else if (v && g.WO % 2 == 0 && g.W % 4 == 0) V = 2;
    else if (v && g.W % 2 == 0) V = 1;
    const size_t total = planes * g.HO * (g.WO / (V ? V : 1));
    const size_t want = (total + 255) / 256, cap = (size_t)sm_count() * 16;
    const int blocks = (int)(want < cap ? (want ? want : 1) : cap);
    const E* s = static_cast<const E*>(src); E* d = static_cast<E*>(dst);
    const unsigned pl = (unsigned)planes;
    if (V == 4) subsample_kernel<E, (sizeof(E) == 2 ? 4 : 2)><<<blocks, 256, 0, stream>>>(s, d, pl, g.H, g.W, g.HO, g.WO, g.SH, g.SW, g.PT, g.PL);
    else if (V == 2) subsample_kernel<E, 2><<<blocks, 256, 0, stream>>>(s, d, pl, g.H, g.W, g.HO, g.WO, g.SH, g.SW, g.PT, g.PL);
    else if (V == 1) subsample_kernel<E, 1><<<blocks, 256, 0, stream>>>(s, d, pl, g.H, g.W, g.HO, g.WO, g.SH, g.SW, g.PT, g.PL);
    else subsample_kernel<E, 0><<<blocks, 256, 0, stream>>>(s, d, pl, g.H, g.W, g.HO, g.WO, g.SH, g.SW, g.PT, g.PL);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

template <typename E>
int launch_scatter(const void* src, void* dst, size_t planes, const Geom& g, cudaStream_t stream) {
    const bool al = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    const bool v = g.SW == 2 && g.PL == 0 && al && g.W == 2 * g.WO;
    int V = 0;                                            // source elements per thread; stores of up to 16 bytes
    if (v && sizeof(E) == 2 && g.W % 8 == 0) V = 4;
    else if (v && g.W % 4 == 0) V = 2;
    else if (v) V = 1;
    const size_t total = planes * g.H * (V == 0 ? g.W : g.W / (2 * V));
    const size_t want = (total + 255) / 256, cap = (size_t)sm_count() * 16;
    const int blocks = (int)(want < cap ? (want ? want : 1) : cap);
    const E* s = static_cast<const E*>(src); E* d = static_cast<E*>(dst);
    const unsigned pl = (unsigned)planes;
    if (V == 4) scatter_strided_kernel<E, (sizeof(E) == 2 ? 4 : 2)><<<blocks, 256, 0, stream>>>(s, d, pl, g.H, g.W, g.HO, g.WO, g.SH, g.SW, g.PT, g.PL);
    else if (V == 2) scatter_strided_kernel<E, 2><<<blocks, 256, 0, stream>>>(s, d, pl, g.H, g.W, g.HO, g.WO, g.SH, g.SW, g.PT, g.PL);
    else if (V == 1) scatter_strided_kernel<E, 1><<<blocks, 256, 0, stream>>>(s, d, pl, g.H, g.W, g.HO, g.WO, g.SH, g.SW, g.PT, g.PL);
    else scatter_strided_kernel<E, 0><<<blocks, 256, 0, stream>>>(s, d, pl, g.H, g.W, g.HO, g.WO, g.SH, g.SW, g.PT, g.PL);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

}  // namespace

namespace {
// The first tensor-core kernels of this backend (producer warps copy operand chunks): still used for the
// filter gradient of narrow pointwise layers.
bool legacy_supported(int dtype, int variant, const Geom& g) {
    if (dtype != PCB_F16 && dtype != PCB_BF16) return false;
    if (variant != PCB_VARIANT_16_PRODUCT) return false;
    if (g.nc != 4 || g.real_in || g.w_io || g.dw_io) return false;     // quaternion-only kernel
    if (!pointwise(g)) return false;
    // 16-byte operand chunks must not straddle a component, an image or a channel row
    return (g.Ci % 8 == 0) && (g.Co % 8 == 0) && ((g.H * g.W) % 8 == 0);
}
}  // namespace

bool tensor_path_supported(Pass pass, int dtype, int variant, const Geom& g) {
    // a literal 8-product request: the factorised kernels exist for pointwise quaternion layers
    if (variant == PCB_VARIANT_8_PRODUCT) return pointwise8_tc_supported(pass, dtype, variant, g);
    // channels-last activations, OHWI / HWIO filters, one group of a grouped layer: the general 16-bit kernels address
    // every tensor through element strides (and read channels-last activations in place)
    if (!g.plain)
        return dtype != PCB_F32 && (pass == PASS_BWD_FILTER ? conv_filter_tc_supported(dtype, variant, g) : conv_tc_supported(pass, dtype, variant, g));
    if (strided_pointwise(g) && tensor_path_supported(pass, dtype, variant, compact_geom(g))) return true;
    if (pass == PASS_BWD_DATA && strided_classes_supported(dtype, variant, g)) return true;
    if (dtype == PCB_F32) return conv_tf32_supported(pass, dtype, variant, g);
    if (pass == PASS_BWD_FILTER)
        return pointwise_filter_tc_supported(dtype, variant, g) || narrow_filter_tc_supported(dtype, variant, g) ||
               conv_filter_tc_supported(dtype, variant, g) || legacy_supported(dtype, variant, g);
    return pointwise_tc_supported(pass, dtype, variant, g) || narrow_tc_supported(pass, dtype, variant, g) ||
           conv_tc_supported(pass, dtype, variant, g) || legacy_supported(dtype, variant, g);
}

size_t tensor_scratch_bytes(Pass pass, int dtype, int variant, int engine, const Geom& g) {
    if (engine == PCB_ENGINE_SIMT || !tensor_path_supported(pass, dtype, variant, g)) return 0;
    if (variant == PCB_VARIANT_8_PRODUCT) return pointwise8_tc_scratch_bytes(pass, g);
    if (!g.plain) return pass == PASS_BWD_FILTER ? conv_filter_tc_scratch_bytes(g) : conv_tc_scratch_bytes(pass, g);
    if (strided_pointwise(g) && tensor_path_supported(pass, dtype, variant, compact_geom(g)))
        return compact_bytes(pass, dtype, g) + tensor_scratch_bytes(pass, dtype, variant, engine, compact_geom(g));
    if (pass == PASS_BWD_DATA && strided_classes_supported(dtype, variant, g)) {
        StrideClass cls[4];
        size_t bytes, inner = 0;
        const int n = stride_classes(g, dtype, cls, &bytes);
        for (int i = 0; i < n; ++i)
            if (cls[i].g.KH > 0 && cls[i].g.KW > 0) {
                const size_t t = tensor_scratch_bytes(pass, dtype, variant, engine, cls[i].g);
                if (t > inner) inner = t;
            }
        return bytes + inner;
    }
    if (dtype == PCB_F32) return conv_tf32_scratch_bytes(pass, g);
    if (pass == PASS_BWD_FILTER) {
        if (pointwise_filter_tc_supported(dtype, variant, g)) return (size_t)g.nc * g.Co * g.Ci * g.KH * g.KW * sizeof(float);
        if (narrow_filter_tc_supported(dtype, variant, g)) return narrow_filter_tc_scratch_bytes(g);
        if (conv_filter_tc_supported(dtype, variant, g)) return conv_filter_tc_scratch_bytes(g);
        return (size_t)g.nc * g.Co * g.Ci * g.KH * g.KW * sizeof(float);
    }
    if (pointwise_tc_supported(pass, dtype, variant, g)) return 0;
    if (narrow_tc_supported(pass, dtype, variant, g)) return narrow_tc_scratch_bytes(pass, g);
    if (conv_tc_supported(pass, dtype, variant, g)) return conv_tc_scratch_bytes(pass, g);
    return 0;
}

bool forward_keeps_staged_input(int dtype, int variant, const Geom& g) {
    if ((dtype != PCB_F16 && dtype != PCB_BF16) || variant != PCB_VARIANT_16_PRODUCT || !g.plain || g.groups != 1) return false;
    if (g.KH * g.KW == 1) return false;             // pointwise layers read x in place (or a compacted copy of their own)
    // the same order of preference as tensor_launch
    if (pointwise_pair_tc_supported(PASS_FWD, dtype, variant, g) || pointwise_tc_supported(PASS_FWD, dtype, variant, g)) return false;
    if (pointwise_filter_tc_supported(dtype, variant, g)) return false;
    const bool narrow_fwd = narrow_tc_supported(PASS_FWD, dtype, variant, g), narrow_flt = narrow_filter_tc_supported(dtype, variant, g);
    if (narrow_fwd || narrow_flt) return narrow_fwd && narrow_flt;
    return conv_tc_supported(PASS_FWD, dtype, variant, g) && conv_filter_tc_supported(dtype, variant, g) && conv_filter_tc_stages_like_forward(g);
}

bool backward_shares_staged_dy(int dtype, int variant, const Geom& g, StagedView* view, size_t* bytes) {
    if ((dtype != PCB_F16 && dtype != PCB_BF16) || variant != PCB_VARIANT_16_PRODUCT || !g.plain || g.groups != 1 || g.real_in) return false;
    if (g.KH * g.KW == 1 || g.SH != 1 || g.SW != 1) return false;
    // the same order of preference as tensor_launch, for both passes
    if (pointwise_filter_tc_supported(dtype, variant, g)) return false;
    const bool narrow_dat = narrow_tc_supported(PASS_BWD_DATA, dtype, variant, g), narrow_flt = narrow_filter_tc_supported(dtype, variant, g);
    if (narrow_dat || narrow_flt) return narrow_dat && narrow_flt && narrow_tc_staged_dy_view(g, view, bytes);
    return conv_tc_supported(PASS_BWD_DATA, dtype, variant, g) && conv_filter_tc_supported(dtype, variant, g) && conv_tc_staged_dy_view(g, view, bytes);
}

int tensor_launch(Pass pass, int dtype, int variant, const Geom& g, const void* a, const void* b, const void* bias,
                  void* out, float* scratch, int* status, cudaStream_t stream, const PassExtras* extras) {
    const void* kept_x = extras ? extras->kept_x : nullptr;
    const StagedView* kept_dy = (extras && extras->dy.base) ? &extras->dy : nullptr;
    if (kept_x && !(pass == PASS_BWD_FILTER && forward_keeps_staged_input(dtype, variant, g))) kept_x = nullptr;
    if (kept_dy) {
        StagedView v;
        size_t bytes;
        if (!(pass == PASS_BWD_FILTER && backward_shares_staged_dy(dtype, variant, g, &v, &bytes))) kept_dy = nullptr;
    }
    if (variant == PCB_VARIANT_8_PRODUCT) return pointwise8_tc_launch(pass, dtype, g, a, b, bias, out, scratch, status, stream);
    if (!g.plain) {
        if (pass == PASS_BWD_FILTER) return conv_filter_tc_launch(dtype, g, a, b, out, scratch, status, stream);
        return conv_tc_launch(pass, dtype, g, a, b, bias, out, scratch, status, stream);
    }
    if (strided_pointwise(g) && tensor_path_supported(pass, dtype, variant, compact_geom(g))) {
        const Geom s = compact_geom(g);
        void* compact = scratch;
        float* rest = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + compact_bytes(pass, dtype, g));
        const size_t planes = (size_t)((pass != PASS_BWD_DATA && g.real_in) ? 1 : g.nc) * g.Nb * g.Ci;
        if (pass == PASS_BWD_DATA) {
            const int rc = tensor_launch(pass, dtype, variant, s, a, b, bias, compact, rest, status, stream);
            if (rc != PCB_OK) return rc;
            return dtype == PCB_F32 ? launch_scatter<uint32_t>(compact, out, planes, g, stream) : launch_scatter<uint16_t>(compact, out, planes, g, stream);
        }
        const int rc = dtype == PCB_F32 ? launch_subsample<uint32_t>(b, compact, planes, g, stream) : launch_subsample<uint16_t>(b, compact, planes, g, stream);
        if (rc != PCB_OK) return rc;
        return tensor_launch(pass, dtype, variant, s, a, compact, bias, out, rest, status, stream);
    }
    if (pass == PASS_BWD_DATA && strided_classes_supported(dtype, variant, g)) {
        StrideClass cls[4];
        size_t bytes;
        const int n = stride_classes(g, dtype, cls, &bytes);
        char* area = reinterpret_cast<char*>(scratch);
        float* rest = reinterpret_cast<float*>(area + bytes);
        ClassPtrs ptrs;
        for (int i = 0; i < 4; ++i) { ptrs.p[i] = nullptr; ptrs.H[i] = ptrs.W[i] = 1; ptrs.live[i] = 0; }
        const unsigned rows = (unsigned)g.nc * g.Co * g.Ci;
        for (int i = 0; i < n; ++i) {
            const Geom& s = cls[i].g;
            const int slot = cls[i].a * g.SW + cls[i].b;
            ptrs.p[slot] = area + cls[i].dx_off; ptrs.H[slot] = s.H; ptrs.W[slot] = s.W;
            if (s.KH == 0 || s.KW == 0) continue;
            ptrs.live[slot] = 1;
            void* w_sub = area + cls[i].w_off;
            const unsigned total = rows * s.KH * s.KW;
            const int blocks = (int)((total + 255) / 256 < (unsigned)sm_count() * 8 ? (total + 255) / 256 : (unsigned)sm_count() * 8);
            if (dtype == PCB_F32)
                gather_taps_kernel<uint32_t><<<blocks, 256, 0, stream>>>((const uint32_t*)a, (uint32_t*)w_sub, rows, g.KH, g.KW, s.KH, s.KW, cls[i].rh, cls[i].rw, g.SH, g.SW);
            else
                gather_taps_kernel<uint16_t><<<blocks, 256, 0, stream>>>((const uint16_t*)a, (uint16_t*)w_sub, rows, g.KH, g.KW, s.KH, s.KW, cls[i].rh, cls[i].rw, g.SH, g.SW);
            PCB_CUDA_TRY(cudaGetLastError());
            const int rc = tensor_launch(pass, dtype, variant, s, w_sub, b, nullptr, area + cls[i].dx_off, rest, status, stream);
            if (rc != PCB_OK) return rc;
        }
        const unsigned planes = (unsigned)g.nc * g.Nb * g.Ci;
        int V = 0;                                   // pixels per class and thread of the vector form
        if (dtype != PCB_F32 && g.SH == 2 && g.SW == 2 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0)
            V = g.W % 8 == 0 ? 4 : (g.W % 4 == 0 ? 2 : (g.W % 2 == 0 ? 1 : 0));
        const size_t items = V ? (size_t)planes * g.H * (g.W / (2 * V)) : (size_t)planes * g.H * g.W;
        const size_t want = (items + 255) / 256, cap = (size_t)sm_count() * 16;
        const int blocks = (int)(want < cap ? (want ? want : 1) : cap);
        if (V == 4) interleave_classes_2x2_kernel<4><<<blocks, 256, 0, stream>>>(ptrs, (uint16_t*)out, planes, g.H, g.W);
        else if (V == 2) interleave_classes_2x2_kernel<2><<<blocks, 256, 0, stream>>>(ptrs, (uint16_t*)out, planes, g.H, g.W);
        else if (V == 1) interleave_classes_2x2_kernel<1><<<blocks, 256, 0, stream>>>(ptrs, (uint16_t*)out, planes, g.H, g.W);
        else if (dtype == PCB_F32) interleave_classes_kernel<uint32_t><<<blocks, 256, 0, stream>>>(ptrs, (uint32_t*)out, planes, g.H, g.W, g.SH, g.SW);
        else interleave_classes_kernel<uint16_t><<<blocks, 256, 0, stream>>>(ptrs, (uint16_t*)out, planes, g.H, g.W, g.SH, g.SW);
        PCB_CUDA_TRY(cudaGetLastError());
        return PCB_OK;
    }
    // the status word is cleared once per API call by the caller of this function; the kernels only OR into it
    if (dtype == PCB_F32) return conv_tf32_launch(pass, g, a, b, bias, out, scratch, status, stream);
    TcParams p;
    p.g = g;
    p.pass = pass;
    p.fmt = dtype == PCB_F16 ? 0 : 1;
    const int HW = g.H * g.W;
    if (pass == PASS_FWD)           { p.M = 4 * g.Co; p.N = g.Nb * HW; p.K = 4 * g.Ci; }
    else if (pass == PASS_BWD_DATA) { p.M = 4 * g.Ci; p.N = g.Nb * HW; p.K = 4 * g.Co; }
    else                            { p.M = 4 * g.Co; p.N = g.Ci;      p.K = 4 * g.Nb * HW; }
    p.k_per_split = (p.K + TBK - 1) / TBK * TBK;
    p.atomic_out = 0;
    if (pointwise_pair_tc_supported(pass, dtype, PCB_VARIANT_16_PRODUCT, g)) return pointwise_pair_tc_launch(dtype, g, a, b, bias, out, status, stream);
    if (pointwise_tc_supported(pass, dtype, PCB_VARIANT_16_PRODUCT, g)) return pointwise_tc_launch(pass, dtype, g, a, b, bias, out, status, stream);
    if (pass != PASS_BWD_FILTER && narrow_tc_supported(pass, dtype, PCB_VARIANT_16_PRODUCT, g))
        return narrow_tc_launch(pass, dtype, g, a, b, bias, out, scratch, status, stream);
    if (pass != PASS_BWD_FILTER && conv_tc_supported(pass, dtype, PCB_VARIANT_16_PRODUCT, g))
        return conv_tc_launch(pass, dtype, g, a, b, bias, out, scratch, status, stream);
    if (pass == PASS_FWD) return launch_tc<PASS_FWD>(p, 1, a, b, bias, out, nullptr, status, stream);
    if (pass == PASS_BWD_DATA) return launch_tc<PASS_BWD_DATA>(p, 1, a, b, bias, out, nullptr, status, stream);

    // backward-filter: the output is tiny and K is the whole batch of pixels -> split K across the grid,
    // accumulate in fp32 scratch, then cast once.
    if (scratch == nullptr) { set_error("backward-filter needs fp32 scratch"); return PCB_ERR_WORKSPACE; }
    if (pointwise_filter_tc_supported(dtype, PCB_VARIANT_16_PRODUCT, g)) return pointwise_filter_tc_launch(dtype, g, a, b, out, scratch, status, stream);
    if (narrow_filter_tc_supported(dtype, PCB_VARIANT_16_PRODUCT, g)) return narrow_filter_tc_launch(dtype, g, a, b, out, scratch, status, stream, kept_x, kept_dy);
    if (conv_filter_tc_supported(dtype, PCB_VARIANT_16_PRODUCT, g)) return conv_filter_tc_launch(dtype, g, a, b, out, scratch, status, stream, kept_x, kept_dy);
    const int tiles = ((p.M + TBM - 1) / TBM) * ((p.N + TBN - 1) / TBN);
    int splits = (2 * sm_count() + tiles - 1) / tiles;
    const int max_splits = (p.K + 4 * TBK - 1) / (4 * TBK);
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    int kps = (p.K + splits - 1) / splits;
    kps = (kps + TBK - 1) / TBK * TBK;
    splits = (p.K + kps - 1) / kps;
    p.k_per_split = kps;
    p.atomic_out = splits > 1 ? 1 : 0;
    const size_t numel = (size_t)4 * g.Co * g.Ci;
    if (p.atomic_out) PCB_CUDA_TRY(cudaMemsetAsync(scratch, 0, numel * sizeof(float), stream));
    int rc = launch_tc<PASS_BWD_FILTER>(p, splits, a, b, bias, out, scratch, status, stream);
    if (rc != PCB_OK) return rc;
    const int blocks = (int)((numel + 255) / 256 < 1184 ? (numel + 255) / 256 : 1184);
    if (dtype == PCB_F16) cast_f32_to_16_kernel<__half><<<blocks, 256, 0, stream>>>(scratch, (__half*)out, numel);
    else cast_f32_to_16_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(scratch, (__nv_bfloat16*)out, numel);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

}  // namespace pcb
