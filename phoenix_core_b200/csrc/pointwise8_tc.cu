// The factorised 8-product form of the pointwise (1x1, stride 1) quaternion convolution on the tensor cores:
// forward, backward-data and backward-filter, fp16 / bf16 tensors, fp32 accumulation in tensor memory.
//
// The reference's default path computes a quaternion convolution from 8 real convolutions of "lane" tensors
// (src/conv2d.hpp:167-234 forward, :433-519 backward): lanes of the input, A_i(x), and of the filters, B_i(w), are sums
// and differences of two components each (src/backend/onednn/tensor.hpp:72-97; output-gradient lanes G_i(dy) with
// a factor 1/2, :109-120), the 8 lane products are recombined linearly (:131-136 forward, :150-153 input gradient,
// :164-167 filter gradient), and the lanes and lane products are tensors in memory (2(X+W+Y) bytes of temporaries,
// src/conv2d.hpp:176-207). Here nothing of that leaves the SM:
//
//   prologue   TMA brings the four raw component tiles of both operands into shared memory; eight "worker" warps
//              form the eight lane tiles of each operand there (16-byte chunks: 4 loads, 32 packed half2 / bfloat162
//              adds, 8 stores). A lane tile has exactly the layout of a component tile, so the transform is the
//              same code for K-major and MN-major, swizzled operands: chunk offset in, same chunk offset out.
//   main loop  one tcgen05.mma per lane and K step: D_i += A_i * B_i, eight accumulators of 128 x 64 fp32 = all 512
//              columns of tensor memory. Half as many multiply-adds as the 16-product form.
//   epilogue   the same warps read the eight accumulators, recombine them in registers (bias added on the way,
//              forward) and store the four output components -- through a swizzled staging tile and TMA stores
//              (forward, backward-data), or as vector reductions into the fp32 split-K scratch (backward-filter).
//
// Tensor memory holds eight accumulators only at 64 columns each, so an MMA is 128 x 64 x 16 and reads 6 KB of
// operands from shared memory for 32 cycles of tensor work, and every operand byte is written twice more (raw by
// TMA, lane by the workers): the kernel is bound by shared-memory bandwidth, not by the halved tensor work. It is
// the literal implementation of the factorised form (PCB_ENGINE_TENSOR with an 8-product request); the automatic
// engine keeps the 16-product kernels of pointwise_tc.cu, which are faster on this hardware.
//
// CTA: warp 0 = TMA producer, warp 1 = tensor-memory owner + MMA issuer, warps 2-9 = workers (lane transform, then
// epilogue). Raw stages: 2 x (32 KB + 16 KB), 32 K elements each; lane buffer: 64 KB + 32 KB, filled and consumed in
// two halves of 16 K elements (one MMA K step), so the transform of one half overlaps the MMAs of the other.
// Every mbarrier wait is bounded; an expired wait sets the status word and the CTA leaves through the common teardown.
#include "tc_common.cuh"
#include "tensor_path.cuh"

namespace pcb {
namespace {

using namespace umma;
using namespace tc;

enum { M_FWD = 0, M_BWD_DATA = 1, M_BWD_FILTER = 2 };

constexpr int E_MT = 128;                                  // MMA M: rows of the A operand per tile
constexpr int E_NT = 64;                                   // MMA N: columns per lane accumulator
constexpr int E_KS = 32;                                   // K elements per raw stage = two MMA K steps
constexpr int E_RAW_STAGES = 2;
constexpr uint32_t E_A_RAW = 4 * E_MT * E_KS * 2;          // 32 KB: four components of the A operand
constexpr uint32_t E_B_RAW = 4 * E_NT * E_KS * 2;          // 16 KB
constexpr uint32_t E_RAW_STAGE = E_A_RAW + E_B_RAW;
constexpr uint32_t E_A_LANES = 2 * E_A_RAW;                // 64 KB: eight lanes
constexpr uint32_t E_B_LANES = 2 * E_B_RAW;                // 32 KB
constexpr uint32_t E_A_COMP = E_MT * E_KS * 2;             // 8 KB: one component (or lane) of A
constexpr uint32_t E_B_COMP = E_NT * E_KS * 2;             // 4 KB
constexpr uint32_t E_OUT_BYTES = E_MT * 64 * 2;            // 16 KB: one output component of a tile, [128 channels][64 pixels]
constexpr int E_THREADS = 320;
constexpr size_t E_SMEM_BYTES = 1024 + E_RAW_STAGES * E_RAW_STAGE + E_A_LANES + E_B_LANES + E_OUT_BYTES + 256;
constexpr int ST_E_PRODUCER = 0x1000, ST_E_MMA = 0x2000, ST_E_WORKER = 0x4000;

constexpr uint64_t DESC_SWIZZLE_64B = 4ull << 61;
// K-major tile with 64-byte rows (32 16-bit K elements), 64-byte swizzle: 8-row groups are 512 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor_sw64(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(512 >> 4) << 32) | DESC_VERSION_SM100 | DESC_SWIZZLE_64B;
}

struct EParams {
    int Nb, HW, fmt, has_bias;
    // forward / backward-data: output channels (rows), reduced channels (K), 64-pixel blocks
    int Cout, Cred, blocks_per_image, n_c_tiles, n_tiles;
    // backward-filter: 32-pixel steps split over the grid
    int Co, Ci, n_co_tiles, n_ci_tiles, steps_total, steps_per_split;
};

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

// Packed pair arithmetic on the raw 32-bit words of either 16-bit type.
template <typename T2> __device__ __forceinline__ uint32_t padd(uint32_t a, uint32_t b) {
    const T2 r = __hadd2(*reinterpret_cast<const T2*>(&a), *reinterpret_cast<const T2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
template <typename T2> __device__ __forceinline__ uint32_t psub(uint32_t a, uint32_t b) {
    const T2 r = __hsub2(*reinterpret_cast<const T2*>(&a), *reinterpret_cast<const T2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
template <typename T2> __device__ __forceinline__ uint32_t phalf(uint32_t a);
template <> __device__ __forceinline__ uint32_t phalf<__half2>(uint32_t a) {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), __float2half2_rn(0.5f));
    return *reinterpret_cast<const uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t phalf<__nv_bfloat162>(uint32_t a) {
    const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a), __float2bfloat162_rn(0.5f));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// Which lane formulas an operand takes (src/backend/onednn/tensor.hpp:72-79 input, :90-97 filters, :109-120 output gradient).
enum { L_INPUT = 0, L_FILTER = 1, L_GRAD = 2 };

// One 32-bit word (two elements) of each of the four components -> the same word of each of the eight lanes.
template <int KIND, typename T2>
__device__ __forceinline__ void lane_words(const uint32_t c[4], uint32_t l[8]) {
    if (KIND == L_INPUT) {
        l[0] = padd<T2>(c[3], c[1]); l[1] = psub<T2>(c[0], c[2]); l[2] = padd<T2>(c[0], c[2]); l[3] = psub<T2>(c[3], c[1]);
        l[4] = psub<T2>(c[3], c[2]); l[5] = padd<T2>(c[1], c[0]); l[6] = psub<T2>(c[0], c[1]); l[7] = padd<T2>(c[3], c[2]);
    } else if (KIND == L_FILTER) {
        l[0] = padd<T2>(c[1], c[2]); l[1] = padd<T2>(c[0], c[3]); l[2] = psub<T2>(c[0], c[3]); l[3] = psub<T2>(c[1], c[2]);
        l[4] = psub<T2>(c[2], c[3]); l[5] = padd<T2>(c[1], c[0]); l[6] = padd<T2>(c[2], c[3]); l[7] = psub<T2>(c[0], c[1]);
    } else {
        const uint32_t t1 = padd<T2>(c[0], c[1]), t3 = psub<T2>(c[0], c[1]), t2 = padd<T2>(c[2], c[3]), t4 = psub<T2>(c[2], c[3]);
        l[0] = phalf<T2>(psub<T2>(t2, t1)); l[1] = phalf<T2>(psub<T2>(t3, t4)); l[2] = phalf<T2>(padd<T2>(t3, t4)); l[3] = phalf<T2>(padd<T2>(t1, t2));
        l[4] = c[0]; l[5] = c[1]; l[6] = c[2]; l[7] = c[3];
    }
}

// One 16-byte chunk of each component (at raw + q * comp_stride) -> the same chunk of each lane (at lanes + i * lane_stride).
template <int KIND, typename T2>
__device__ __forceinline__ void lane_chunk(uint32_t raw, uint32_t comp_stride, uint32_t lanes, uint32_t lane_stride) {
    uint4 c[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) c[q] = ld_shared_v4(raw + q * comp_stride);
    uint32_t o[4][8];
    {
        const uint32_t w0[4] = {c[0].x, c[1].x, c[2].x, c[3].x}, w1[4] = {c[0].y, c[1].y, c[2].y, c[3].y};
        const uint32_t w2[4] = {c[0].z, c[1].z, c[2].z, c[3].z}, w3[4] = {c[0].w, c[1].w, c[2].w, c[3].w};
        lane_words<KIND, T2>(w0, o[0]); lane_words<KIND, T2>(w1, o[1]); lane_words<KIND, T2>(w2, o[2]); lane_words<KIND, T2>(w3, o[3]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) st_shared_v4(lanes + i * lane_stride, o[0][i], o[1][i], o[2][i], o[3][i]);
}

// Byte offset, inside one component of a K-major tile with 64-byte rows and 64-byte swizzle, of chunk slot `t` of the K
// half `h` (16 K elements = two 16-byte chunks per row; chunk c of row r sits at position c ^ ((r / 2) % 4)).
// Slots are handed out so that eight consecutive threads touch eight different 16-byte bank groups: the two chunks of
// rows {0, 1, 4, 5} of an 8-row group (rows 0 and 2 would share their bank groups, rows 0 and 4 do not), the next
// eight threads rows {2, 3, 6, 7}.
__device__ __forceinline__ uint32_t kmajor_half_offset(int t, int h) {
    const int v = t & 7, sub = (t >> 3) & 1, grp = t >> 4;
    const int sel = v >> 1;
    const int row = grp * 8 + 2 * sub + (sel & 1) + 4 * (sel >> 1), c = 2 * h + (v & 1);
    return (uint32_t)row * 64u + (uint32_t)((c ^ ((row >> 1) & 3)) << 4);
}

// Linear recombination of the eight lane products into the four components of the result.
template <int MODE>
__device__ __forceinline__ void recombine(const float L[8], float o[4]) {
    if (MODE == M_FWD) {                 // src/backend/onednn/tensor.hpp:131-136
        const float a2 = L[0] + L[1] + L[2], a5 = 0.5f * (a2 + L[3]);
        o[0] = a5 - L[0] + L[4]; o[1] = a5 - a2 + L[5]; o[2] = a5 - L[1] + L[6]; o[3] = a5 - L[2] + L[7];
    } else if (MODE == M_BWD_DATA) {     // :150-153
        o[0] = L[1] + L[2] + L[5] + L[6]; o[1] = L[0] - L[3] + L[5] - L[6];
        o[2] = L[2] - L[1] - L[4] + L[7]; o[3] = L[0] + L[3] + L[4] + L[7];
    } else {                             // :164-167
        o[0] = L[1] + L[2] + L[5] + L[7]; o[1] = L[0] + L[3] + L[5] - L[7];
        o[2] = L[0] - L[3] + L[4] + L[6]; o[3] = L[1] - L[2] - L[4] + L[6];
    }
}

template <int MODE>
__global__ void __launch_bounds__(E_THREADS, 1)
qconv_pointwise8_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const __grid_constant__ CUtensorMap map_out, EParams p, const uint16_t* __restrict__ bias,
                           float* __restrict__ dw32, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t raw_addr = smem_u32(base);
    const uint32_t a_lanes = raw_addr + E_RAW_STAGES * E_RAW_STAGE, b_lanes = a_lanes + E_A_LANES;
    const uint32_t out_addr = b_lanes + E_B_LANES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + E_RAW_STAGES * E_RAW_STAGE + E_A_LANES + E_B_LANES + E_OUT_BYTES);
    const uint32_t raw_full = smem_u32(bars), raw_empty = smem_u32(bars + 2);
    const uint32_t lane_full = smem_u32(bars + 4), lane_empty = smem_u32(bars + 6);
    const uint32_t tmem_full = smem_u32(bars + 8), tmem_empty = smem_u32(bars + 9), epi_bar = smem_u32(bars + 10);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);

    // The work of this CTA: `n_jobs` accumulator tiles of `steps` raw stages each.
    int n_jobs, steps, f_co0 = 0, f_ci0 = 0, f_step_beg = 0;
    if (MODE == M_BWD_FILTER) {
        const int n_out_tiles = p.n_co_tiles * p.n_ci_tiles;
        const int out_tile = blockIdx.x % n_out_tiles, split = blockIdx.x / n_out_tiles;
        f_co0 = (out_tile / p.n_ci_tiles) * E_MT; f_ci0 = (out_tile % p.n_ci_tiles) * E_NT;
        f_step_beg = split * p.steps_per_split;
        steps = max(0, min(p.steps_total, f_step_beg + p.steps_per_split) - f_step_beg);
        n_jobs = steps > 0 ? 1 : 0;
    } else {
        steps = (p.Cred + E_KS - 1) / E_KS;
        n_jobs = blockIdx.x < p.n_tiles ? (p.n_tiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    }

    if (t == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(raw_full + 8 * s, 1); mbar_init(raw_empty + 8 * s, 8);
            mbar_init(lane_full + 8 * s, 8); mbar_init(lane_empty + 8 * s, 1);
        }
        mbar_init(tmem_full, 1); mbar_init(tmem_empty, 8); mbar_init(epi_bar, 8);
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int job = 0; job < n_jobs && ok; ++job) {
                const int tile = blockIdx.x + job * gridDim.x;
                int c0 = 0, img = 0, pix = 0;
                if (MODE != M_BWD_FILTER) {
                    const int blk = tile / p.n_c_tiles;
                    c0 = (tile - blk * p.n_c_tiles) * E_MT;
                    img = blk / p.blocks_per_image; pix = (blk - img * p.blocks_per_image) * 64;
                }
                for (int k = 0; k < steps && ok; ++k, ++it) {
                    const int s = it & 1;
                    ok = mbar_wait_bounded(raw_empty + 8 * s, ((it >> 1) & 1) ^ 1, status, ST_E_PRODUCER);
                    if (!ok) break;
                    const uint32_t a_dst = raw_addr + s * E_RAW_STAGE, b_dst = a_dst + E_A_RAW, bar = raw_full + 8 * s;
                    mbar_arrive_expect_tx(bar, E_RAW_STAGE);
                    if (MODE == M_FWD) {
                        tma_load_3d(a_dst, &map_a, k * E_KS, c0, 0, bar);                     // filters [r][128 co][32 ci]
                        tma_load_4d(b_dst, &map_b, pix, k * E_KS, img, 0, bar);               // x [comp][32 ci][64 px]
                    } else if (MODE == M_BWD_DATA) {
                        tma_load_3d(a_dst, &map_a, c0, k * E_KS, 0, bar);                     // filters [r][32 co][64 ci], two ci blocks
                        tma_load_3d(a_dst + E_A_RAW / 2, &map_a, c0 + 64, k * E_KS, 0, bar);
                        tma_load_4d(b_dst, &map_b, pix, k * E_KS, img, 0, bar);               // dy [comp][32 co][64 px]
                    } else {
                        const int step = f_step_beg + k;
                        const int fimg = step / p.blocks_per_image, px0 = (step - fimg * p.blocks_per_image) * E_KS;
                        tma_load_4d(a_dst, &map_a, px0, f_co0, fimg, 0, bar);                 // dy [comp][128 co][32 px]
                        tma_load_4d(b_dst, &map_b, px0, f_ci0, fimg, 0, bar);                 // x [comp][64 ci][32 px]
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        int it = 0;
        bool ok = true;
        const uint32_t idesc = make_idesc_f16(p.fmt, E_MT, E_NT, MODE == M_BWD_DATA, MODE != M_BWD_FILTER);
        for (int job = 0; job < n_jobs && ok; ++job) {
            for (int k = 0; k < steps && ok; ++k, ++it) {
#pragma unroll 1
                for (int h = 0; h < 2 && ok; ++h) {
                    ok = mbar_wait_bounded(lane_full + 8 * h, it & 1, status, ST_E_MMA);
                    if (ok && k == 0 && h == 0 && job > 0) ok = mbar_wait_bounded(tmem_empty, (job - 1) & 1, status, ST_E_MMA);
                    if (!ok) break;
                    tc_fence_after_sync();
                    if (lane == 0) {
                        const uint32_t acc = (k > 0 || h > 0) ? 1u : 0u;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            uint64_t ad, bd;
                            if (MODE == M_BWD_DATA) ad = make_desc_mnmajor(a_lanes + i * (E_KS * 128) + h * 2048, E_A_LANES / 2);
                            else ad = desc_kmajor_sw64(a_lanes + i * E_A_COMP + h * 32);
                            if (MODE == M_BWD_FILTER) bd = desc_kmajor_sw64(b_lanes + i * E_B_COMP + h * 32);
                            else bd = make_desc_mnmajor(b_lanes + i * E_B_COMP + h * 2048, E_B_COMP);
                            mma_f16_ss(tmem_base + i * E_NT, ad, bd, idesc, acc);
                        }
                        mma_commit(lane_empty + 8 * h);
                        if (k == steps - 1 && h == 1) mma_commit(tmem_full);
                    }
                    __syncwarp();
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- workers: lane transform, then epilogue
        const int wt = t - 64;                      // 0..255
        const int q = warp & 3;                     // tensor-memory lane quadrant this warp may read
        const int chalf = (warp - 2) >> 2;          // which 32 accumulator columns of each lane
        const int row = q * 32 + lane;              // accumulator row = output row of the tile
        const bool issuer = warp == 2 && lane == 0;
        int it = 0, epi_phase = 0;
        bool ok = true;
        auto epi_sync = [&]() {                     // the eight worker warps meet; bounded like every other wait
            __syncwarp();
            if (lane == 0) mbar_arrive(epi_bar);
            const bool done = mbar_wait_bounded(epi_bar, epi_phase & 1, status, ST_E_WORKER);
            ++epi_phase;
            return __all_sync(0xffffffffu, done);
        };
        // chunk slots of this thread inside one component, per K half (see kmajor_half_offset; MN-major halves are
        // 2 KB contiguous per 64-element block)
        for (int job = 0; job < n_jobs && ok; ++job) {
            for (int k = 0; k < steps && ok; ++k, ++it) {
                const int s = it & 1;
                ok = mbar_wait_bounded(raw_full + 8 * s, (it >> 1) & 1, status, ST_E_WORKER);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint32_t a_raw = raw_addr + s * E_RAW_STAGE, b_raw = a_raw + E_A_RAW;
#pragma unroll 1
                for (int h = 0; h < 2; ++h) {
                    ok = mbar_wait_bounded(lane_empty + 8 * h, (it & 1) ^ 1, status, ST_E_WORKER);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after_sync();
                    // A operand: 256 chunk slots per component and half, one per worker thread
                    if (MODE == M_FWD) {
                        const uint32_t off = kmajor_half_offset(wt, h);
                        if (p.fmt == 0) lane_chunk<L_FILTER, __half2>(a_raw + off, E_A_COMP, a_lanes + off, E_A_COMP);
                        else lane_chunk<L_FILTER, __nv_bfloat162>(a_raw + off, E_A_COMP, a_lanes + off, E_A_COMP);
                    } else if (MODE == M_BWD_DATA) {
                        const int blk = wt >> 7;
                        const uint32_t off = (uint32_t)h * 2048u + (uint32_t)(wt & 127) * 16u;
                        const uint32_t src = a_raw + blk * (E_A_RAW / 2) + off, dst = a_lanes + blk * (E_A_LANES / 2) + off;
                        if (p.fmt == 0) lane_chunk<L_FILTER, __half2>(src, E_KS * 128, dst, E_KS * 128);
                        else lane_chunk<L_FILTER, __nv_bfloat162>(src, E_KS * 128, dst, E_KS * 128);
                    } else {
                        const uint32_t off = kmajor_half_offset(wt, h);
                        if (p.fmt == 0) lane_chunk<L_GRAD, __half2>(a_raw + off, E_A_COMP, a_lanes + off, E_A_COMP);
                        else lane_chunk<L_GRAD, __nv_bfloat162>(a_raw + off, E_A_COMP, a_lanes + off, E_A_COMP);
                    }
                    // B operand: 128 chunk slots per component and half (the first four worker warps)
                    if (wt < 128) {
                        if (MODE == M_BWD_FILTER) {
                            const uint32_t off = kmajor_half_offset(wt, h);
                            if (p.fmt == 0) lane_chunk<L_INPUT, __half2>(b_raw + off, E_B_COMP, b_lanes + off, E_B_COMP);
                            else lane_chunk<L_INPUT, __nv_bfloat162>(b_raw + off, E_B_COMP, b_lanes + off, E_B_COMP);
                        } else {
                            const uint32_t off = (uint32_t)h * 2048u + (uint32_t)wt * 16u;
                            constexpr int KIND = MODE == M_FWD ? L_INPUT : L_GRAD;
                            if (p.fmt == 0) lane_chunk<KIND, __half2>(b_raw + off, E_B_COMP, b_lanes + off, E_B_COMP);
                            else lane_chunk<KIND, __nv_bfloat162>(b_raw + off, E_B_COMP, b_lanes + off, E_B_COMP);
                        }
                    }
                    fence_proxy_async_smem();       // the lane tiles are read by the tensor cores (async proxy)
                    __syncwarp();
                    if (lane == 0) mbar_arrive(lane_full + 8 * h);
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(raw_empty + 8 * s);     // this warp has read all it needs of the raw stage
            }
            if (!ok) break;

            // ------------------------------------------------------------ epilogue of the job
            ok = mbar_wait_bounded(tmem_full, job & 1, status, ST_E_WORKER);
            ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + chalf * 32;
            if (MODE == M_BWD_FILTER) {
                const int co = f_co0 + row;
#pragma unroll 1
                for (int half = 0; half < 2; ++half) {
                    uint32_t v[8][16];
#pragma unroll
                    for (int i = 0; i < 8; ++i) tmem_ld_32x32b_x16(lane_addr + i * E_NT + half * 16, v[i]);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 8; ++i) tmem_regs_ready(v[i]);
                    if (co < p.Co) {
#pragma unroll
                        for (int g4 = 0; g4 < 4; ++g4) {
                            const int ci = f_ci0 + chalf * 32 + half * 16 + g4 * 4;
                            if (ci >= p.Ci) continue;
                            float o[4][4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float L[8], r4[4];
#pragma unroll
                                for (int i = 0; i < 8; ++i) L[i] = __uint_as_float(v[i][g4 * 4 + e]);
                                recombine<M_BWD_FILTER>(L, r4);
#pragma unroll
                                for (int r = 0; r < 4; ++r) o[r][e] = r4[r];
                            }
#pragma unroll
                            for (int r = 0; r < 4; ++r)
                                red_add_f32x4(dw32 + ((size_t)r * p.Co + co) * p.Ci + ci, o[r][0], o[r][1], o[r][2], o[r][3]);
                        }
                    }
                }
            } else {
                const int tile = blockIdx.x + job * gridDim.x;
                const int blk = tile / p.n_c_tiles, c_tile = tile - blk * p.n_c_tiles;
                const int img = blk / p.blocks_per_image, pix = (blk - img * p.blocks_per_image) * 64;
                const int c = c_tile * E_MT + row;
                float badd[4] = {0.f, 0.f, 0.f, 0.f};
                if (MODE == M_FWD && p.has_bias && c < p.Cout) {
#pragma unroll
                    for (int o = 0; o < 4; ++o) {
                        const uint16_t raw = bias[o * p.Cout + c];
                        badd[o] = p.fmt == 0 ? __half2float(__ushort_as_half(raw)) : __bfloat162float(__ushort_as_bfloat16(raw));
                    }
                }
                uint32_t packed[4][16];             // this thread's 32 pixels of each output component, as 16-bit pairs
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t v[8][16];
#pragma unroll
                    for (int i = 0; i < 8; ++i) tmem_ld_32x32b_x16(lane_addr + i * E_NT + half * 16, v[i]);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 8; ++i) tmem_regs_ready(v[i]);
#pragma unroll
                    for (int e2 = 0; e2 < 8; ++e2) {
                        float lo[4], hi[4], L[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) L[i] = __uint_as_float(v[i][2 * e2]);
                        recombine<MODE>(L, lo);
#pragma unroll
                        for (int i = 0; i < 8; ++i) L[i] = __uint_as_float(v[i][2 * e2 + 1]);
                        recombine<MODE>(L, hi);
#pragma unroll
                        for (int o = 0; o < 4; ++o) {
                            const float f0 = lo[o] + badd[o], f1 = hi[o] + badd[o];
                            if (p.fmt == 0) { const __half2 hh = __floats2half2_rn(f0, f1); packed[o][half * 8 + e2] = *reinterpret_cast<const uint32_t*>(&hh); }
                            else { const __nv_bfloat162 hh = __floats2bfloat162_rn(f0, f1); packed[o][half * 8 + e2] = *reinterpret_cast<const uint32_t*>(&hh); }
                        }
                    }
                }
                // the accumulators are free for the next tile
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_empty);
                // the tile leaves component by component through a 128-byte-swizzled [128 channels][64 pixels] box and a TMA
                // store: chunk j (8 pixels) of row r sits at position j ^ (r % 8); out-of-range rows / pixels are clipped
#pragma unroll
                for (int o = 0; o < 4 && ok; ++o) {
                    if (issuer) bulk_wait_read_all();          // the previous component has left the staging buffer
                    ok = epi_sync();
                    if (!ok) break;
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch)
                        st_shared_v4(out_addr + row * 128 + (((chalf * 4 + ch) ^ (row & 7)) << 4), packed[o][4 * ch], packed[o][4 * ch + 1],
                                     packed[o][4 * ch + 2], packed[o][4 * ch + 3]);
                    fence_proxy_async_smem();
                    ok = epi_sync();
                    if (!ok) break;
                    if (issuer) {
                        tma_store_4d(&map_out, out_addr, pix, c_tile * E_MT, img, o);
                        bulk_commit_group();
                    }
                }
            }
            if (MODE == M_BWD_FILTER) {             // one job per CTA: nothing waits for the accumulators again
                tc_fence_before_sync();
            }
        }
        if (issuer && MODE != M_BWD_FILTER) bulk_wait_read_all();   // shared memory must outlive the last bulk store's reads
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

template <typename T>
__global__ void cast8_f32_kernel(const float* __restrict__ src, T* __restrict__ dst, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) DType<T>::store(dst + i, src[i]);
}

int make_map8(CUtensorMap* map, int fmt, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
              const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
    return make_tensor_map(map, fmt == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ptr, rank, dims, strides_bytes,
                           box, nullptr, swizzle, "8-product pointwise operand");
}

bool pointwise_1x1(const Geom& g) {
    return g.KH == 1 && g.KW == 1 && g.SH == 1 && g.SW == 1 && g.PT == 0 && g.PL == 0 && g.HO == g.H && g.WO == g.W;
}

}  // namespace

bool pointwise8_tc_supported(Pass /*pass*/, int dtype, int variant, const Geom& g) {
    if (variant != PCB_VARIANT_8_PRODUCT) return false;
    if (dtype != PCB_F16 && dtype != PCB_BF16) return false;
    if (g.nc != 4 || g.real_in || g.w_io || g.dw_io || !g.plain) return false;   // quaternions only; NCHW / OIHW tensors
    if (!pointwise_1x1(g)) return false;
    // TMA: every global stride a multiple of 16 bytes
    return (g.Ci % 8 == 0) && (g.Co % 8 == 0) && ((g.H * g.W) % 8 == 0);
}

size_t pointwise8_tc_scratch_bytes(Pass pass, const Geom& g) {
    return pass == PASS_BWD_FILTER ? (size_t)4 * g.Co * g.Ci * sizeof(float) : 0;
}

int pointwise8_tc_launch(Pass pass, int dtype, const Geom& g, const void* a, const void* b, const void* bias, void* out,
                         float* scratch, int* status, cudaStream_t stream) {
    const int fmt = dtype == PCB_F16 ? 0 : 1;
    const int HW = g.H * g.W;
    EParams p = {};
    p.Nb = g.Nb; p.HW = HW; p.fmt = fmt;
    alignas(64) CUtensorMap map_a, map_b, map_out;
    if (pass == PASS_BWD_FILTER) {          // a = dy, b = x, out = dw
        p.Co = g.Co; p.Ci = g.Ci;
        p.blocks_per_image = (HW + E_KS - 1) / E_KS;
        p.n_co_tiles = (g.Co + E_MT - 1) / E_MT;
        p.n_ci_tiles = (g.Ci + E_NT - 1) / E_NT;
        p.steps_total = g.Nb * p.blocks_per_image;
        const int n_out_tiles = p.n_co_tiles * p.n_ci_tiles;
        int splits = sm_count() / n_out_tiles;
        if (splits < 1) splits = 1;
        if (splits > p.steps_total) splits = p.steps_total;
        p.steps_per_split = (p.steps_total + splits - 1) / splits;
        splits = (p.steps_total + p.steps_per_split - 1) / p.steps_per_split;
        {
            const cuuint64_t dims[4] = {(cuuint64_t)HW, (cuuint64_t)g.Co, (cuuint64_t)g.Nb, 4};
            const cuuint64_t strides[3] = {(cuuint64_t)HW * 2, (cuuint64_t)g.Co * HW * 2, (cuuint64_t)g.Nb * g.Co * HW * 2};
            const cuuint32_t box[4] = {E_KS, E_MT, 1, 4};
            const int rc = make_map8(&map_a, fmt, a, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
            if (rc != PCB_OK) return rc;
        }
        {
            const cuuint64_t dims[4] = {(cuuint64_t)HW, (cuuint64_t)g.Ci, (cuuint64_t)g.Nb, 4};
            const cuuint64_t strides[3] = {(cuuint64_t)HW * 2, (cuuint64_t)g.Ci * HW * 2, (cuuint64_t)g.Nb * g.Ci * HW * 2};
            const cuuint32_t box[4] = {E_KS, E_NT, 1, 4};
            const int rc = make_map8(&map_b, fmt, b, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
            if (rc != PCB_OK) return rc;
        }
        map_out = map_b;                    // not used by this mode
        if (scratch == nullptr) { set_error("backward-filter needs fp32 scratch"); return PCB_ERR_WORKSPACE; }
        const size_t numel = (size_t)4 * g.Co * g.Ci;
        PCB_CUDA_TRY(cudaMemsetAsync(scratch, 0, numel * sizeof(float), stream));
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_pointwise8_tc_kernel<M_BWD_FILTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)E_SMEM_BYTES));
        qconv_pointwise8_tc_kernel<M_BWD_FILTER><<<n_out_tiles * splits, E_THREADS, E_SMEM_BYTES, stream>>>(map_a, map_b, map_out, p, nullptr, scratch, status);
        PCB_CUDA_TRY(cudaGetLastError());
        const int blocks = (int)((numel + 255) / 256 < 1184 ? (numel + 255) / 256 : 1184);
        if (dtype == PCB_F16) cast8_f32_kernel<__half><<<blocks, 256, 0, stream>>>(scratch, (__half*)out, numel);
        else cast8_f32_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(scratch, (__nv_bfloat16*)out, numel);
        PCB_CUDA_TRY(cudaGetLastError());
        return PCB_OK;
    }

    const bool bwd = pass == PASS_BWD_DATA;  // a = filters, b = x (forward) or dy (backward-data), out = y or dx
    p.has_bias = (!bwd && g.has_bias) ? 1 : 0;
    p.Cout = bwd ? g.Ci : g.Co;
    p.Cred = bwd ? g.Co : g.Ci;
    p.blocks_per_image = (HW + 63) / 64;
    p.n_c_tiles = (p.Cout + E_MT - 1) / E_MT;
    p.n_tiles = g.Nb * p.blocks_per_image * p.n_c_tiles;
    {   // filters [4][Co][Ci]: (ci, co, r)
        const cuuint64_t dims[3] = {(cuuint64_t)g.Ci, (cuuint64_t)g.Co, 4};
        const cuuint64_t strides[2] = {(cuuint64_t)g.Ci * 2, (cuuint64_t)g.Co * g.Ci * 2};
        int rc;
        if (!bwd) { const cuuint32_t box[3] = {E_KS, E_MT, 4}; rc = make_map8(&map_a, fmt, a, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B); }
        else      { const cuuint32_t box[3] = {64, E_KS, 4}; rc = make_map8(&map_a, fmt, a, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B); }
        if (rc != PCB_OK) return rc;
    }
    {   // activations [4][Nb][C][HW]: (px, channel, image, component)
        const int C = p.Cred;
        const cuuint64_t dims[4] = {(cuuint64_t)HW, (cuuint64_t)C, (cuuint64_t)g.Nb, 4};
        const cuuint64_t strides[3] = {(cuuint64_t)HW * 2, (cuuint64_t)C * HW * 2, (cuuint64_t)g.Nb * C * HW * 2};
        const cuuint32_t box[4] = {64, E_KS, 1, 4};
        const int rc = make_map8(&map_b, fmt, b, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != PCB_OK) return rc;
    }
    {   // output [4][Nb][Cout][HW]; the epilogue stores [128 channels][64 pixels] boxes
        const cuuint64_t dims[4] = {(cuuint64_t)HW, (cuuint64_t)p.Cout, (cuuint64_t)g.Nb, 4};
        const cuuint64_t strides[3] = {(cuuint64_t)HW * 2, (cuuint64_t)p.Cout * HW * 2, (cuuint64_t)g.Nb * p.Cout * HW * 2};
        const cuuint32_t box[4] = {64, E_MT, 1, 1};
        const int rc = make_map8(&map_out, fmt, out, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != PCB_OK) return rc;
    }
    const int grid = p.n_tiles < sm_count() ? p.n_tiles : sm_count();
    if (!bwd) {
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_pointwise8_tc_kernel<M_FWD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)E_SMEM_BYTES));
        qconv_pointwise8_tc_kernel<M_FWD><<<grid, E_THREADS, E_SMEM_BYTES, stream>>>(map_a, map_b, map_out, p, (const uint16_t*)bias, nullptr, status);
    } else {
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_pointwise8_tc_kernel<M_BWD_DATA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)E_SMEM_BYTES));
        qconv_pointwise8_tc_kernel<M_BWD_DATA><<<grid, E_THREADS, E_SMEM_BYTES, stream>>>(map_a, map_b, map_out, p, nullptr, nullptr, status);
    }
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

}  // namespace pcb
