// Persistent TMA-fed tcgen05 kernel for the pointwise (1x1, stride 1) quaternion convolution, forward and
// backward-data, for layers with >= 96 output rows per component (the channel tile is 128 wide).
//
// The 4x4 signed weight block is not materialised at all here: the four output components live in four
// TMEM accumulators and each of the 16 (input component, output component) pairs is one tcgen05.mma whose
// A operand is the raw weight tile w[l^d] and whose sign s(l,d) is the instruction's negate-A flag:
//
//   forward        D_d[co, px] += s(l,d) * w[l^d][co, ci-slice] * x_l [ci-slice, px]        d, l = 0..3
//   backward-data  D_l[ci, px] += s(l,d) * w[l^d][co-slice, ci]^T * dy_d[co-slice, px]
//
// (reference sign table src/algebras.cc:28-49; this replaces the CUDA-core 1x1 kernels of
//  src/backend/cudnn/quat_pointwise_conv2d.cu:33-303.) Every weight tile is read once per stage and used
// by 4 MMAs, every activation tile by 4 MMAs, so shared-memory traffic from L2 is 1/4 of what an expanded
// 4Co x 4Ci GEMM would need and no thread ever touches an operand: both come by TMA
// (cp.async.bulk.tensor, 128B / 64B swizzle) straight into the tcgen05 canonical layouts.
//
// CTA (persistent, one per SM): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2-9 =
// epilogue (two warps per TMEM lane quadrant, one per 64-pixel half). Tile = 128 channels x 128 pixels x 4
// components (all 512 TMEM columns); K slice per stage = 32 channels per component (A 32 KB + B 32 KB), 3
// stages, or the weight slices resident (forward, <= 128 reduced channels) beside 2 activation stages.
// The accumulators are drained component by component into packed registers and released one at a time, so the
// next tile's first MMAs overlap the drain; the tile then leaves through a 32 KB shared-memory staging buffer and
// TMA stores (measured: ordinary global stores from the epilogue warps, 32 scattered segments per instruction,
// delayed the MMA warp's own instruction issue by ~4000 cycles per tile; the bulk stores do not).
// Every mbarrier wait is bounded; an expired wait sets the status word and the CTA leaves through the common
// teardown.
#include "tc_common.cuh"
#include "tensor_path.cuh"

namespace pcb {
namespace {

using namespace umma;
using namespace tc;

constexpr int CT = 128;             // channel tile (MMA M)
constexpr int PT = 128;             // pixel tile (MMA N): two TMA boxes of 64 pixels
constexpr int KS = 32;              // channels per component per stage
static_assert(KS / 16 == 2, "the MMA issuer handles the first and the last K step of a slice separately");
constexpr int U_STAGES = 3;
constexpr uint32_t A_BYTES = 4 * CT * KS * 2;      // 32 KB: 4 weight components
constexpr uint32_t B_BYTES = 2 * 4 * KS * 64 * 2;  // 32 KB: 2 pixel boxes x 4 activation components
constexpr uint32_t B_BOX_BYTES = 4 * KS * 64 * 2;  // 16 KB
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int U_THREADS = 320;
constexpr int MAX_RESIDENT_K = 4;                  // weight K slices that may stay in shared memory (4 x 32 KB)
constexpr int RB_STAGES = 2;                       // activation stages beside resident weights
constexpr uint32_t OPERAND_BYTES = U_STAGES * STAGE_BYTES;       // 192 KB, also MAX_RESIDENT_K * A_BYTES + RB_STAGES * B_BYTES
constexpr uint32_t OUT_HALF_BYTES = 64 * CT * 2;   // 16 KB: one component of a 64-pixel block, [128 channels][64 pixels]
constexpr uint32_t OUT_BYTES = 2 * OUT_HALF_BYTES; // output staging for the TMA store: one component of a tile
static_assert(MAX_RESIDENT_K * A_BYTES + RB_STAGES * B_BYTES <= OPERAND_BYTES, "resident plan must fit the operand region");
constexpr size_t U_SMEM_BYTES = 1024 + OPERAND_BYTES + OUT_BYTES + 256;
constexpr int ST_U_PRODUCER = 0x10, ST_U_MMA = 0x20, ST_U_EPILOGUE = 0x40;

struct UParams {
    int Nb, Cout, Cred;      // quaternion batch, output channels of the pass, reduced channels of the pass
    int HW;
    int blocks_per_image;    // ceil(HW / 64)
    int n_px_tiles, n_c_tiles;
    int fmt;                 // 0 f16, 1 bf16
    int has_bias;
    int bwd;                 // 0 forward, 1 backward-data
    int a_resident;          // forward: the CTA's weight slices are loaded once and stay in shared memory
};

constexpr uint64_t DESC_SWIZZLE_64B = 4ull << 61;
// K-major tile with 64-byte rows (32 16-bit K elements), 64-byte swizzle: 8-row groups are 512 bytes apart.
__device__ __forceinline__ uint64_t make_desc_kmajor_sw64(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(512 >> 4) << 32) | DESC_VERSION_SM100 | DESC_SWIZZLE_64B;
}

template <bool BWD>
__global__ void __launch_bounds__(U_THREADS, 1)
qconv_pointwise_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_act,
                          const __grid_constant__ CUtensorMap map_out, UParams p, const uint16_t* __restrict__ bias, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + OPERAND_BYTES + OUT_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * U_STAGES + 8);
    const uint32_t tiles_addr = smem_u32(base);
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + U_STAGES);
    const uint32_t a_full = smem_u32(bars + 2 * U_STAGES + 5);
    const uint32_t out_addr = tiles_addr + OPERAND_BYTES;         // staging for the TMA store
    // one "accumulator drained" barrier per component, so the next tile's MMAs can start on component 0 while
    // the epilogue is still reading components 1..3; one "accumulators complete" barrier per PAIR of components
    // (0,1 and 2,3), so the epilogue drains the first pair while the last MMAs of the tile still run on the second
    const uint32_t tmem_empty = smem_u32(bars + 2 * U_STAGES + 1);
    const uint32_t tmem_full0 = smem_u32(bars + 2 * U_STAGES), tmem_full1 = smem_u32(bars + 2 * U_STAGES + 7);

    const int n_tiles = p.n_px_tiles * p.n_c_tiles;
    const int n_k = (p.Cred + KS - 1) / KS;
    // shared-memory plan: either a ring of [A|B] stages, or all weight slices resident followed by a ring of B stages
    const bool resident = !BWD && p.a_resident;
    const int n_stages = resident ? RB_STAGES : U_STAGES;
    auto a_slot = [&](int k, int s) { return resident ? tiles_addr + k * A_BYTES : tiles_addr + s * STAGE_BYTES; };
    auto b_slot = [&](int s) { return resident ? tiles_addr + n_k * A_BYTES + s * B_BYTES : tiles_addr + s * STAGE_BYTES + A_BYTES; };

    if (t == 0) {
        for (int s = 0; s < U_STAGES; ++s) { mbar_init(full_bar + 8 * s, 1); mbar_init(empty_bar + 8 * s, 1); }
        mbar_init(tmem_full0, 1);
        mbar_init(tmem_full1, 1);
        mbar_init(a_full, 1);
        for (int o = 0; o < 4; ++o) mbar_init(tmem_empty + 8 * o, 8);
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
            if (resident && blockIdx.x < n_tiles) {
                // the grid is a multiple of the channel tiles, so this CTA keeps one channel tile for all its pixel tiles
                mbar_arrive_expect_tx(a_full, n_k * A_BYTES);
                for (int k = 0; k < n_k; ++k) tma_load_3d(a_slot(k, 0), &map_w, k * KS, (blockIdx.x % p.n_c_tiles) * CT, 0, a_full);
            }
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int px_tile = tile / p.n_c_tiles, c_tile = tile - px_tile * p.n_c_tiles;
                const int c0 = c_tile * CT;
                int img[2], pix[2];
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const int blk = 2 * px_tile + b;
                    img[b] = blk / p.blocks_per_image;          // == Nb for a block past the end: fully out of range -> zeros
                    pix[b] = (blk - img[b] * p.blocks_per_image) * 64;
                }
                for (int k = 0; k < n_k && ok; ++k, ++it) {
                    const int s = it % n_stages;
                    ok = mbar_wait_bounded(empty_bar + 8 * s, ((it / n_stages) & 1) ^ 1, status, ST_U_PRODUCER);
                    if (!ok) break;
                    const uint32_t a_dst = a_slot(k, s), b_dst = b_slot(s);
                    const uint32_t bar = full_bar + 8 * s;
                    mbar_arrive_expect_tx(bar, resident ? B_BYTES : STAGE_BYTES);
                    if (!BWD) {
                        if (!resident) tma_load_3d(a_dst, &map_w, k * KS, c0, 0, bar);  // [r][128 co][32 ci]
                    } else {
                        tma_load_3d(a_dst, &map_w, c0, k * KS, 0, bar);                 // [r][32 co][64 ci] x 2 ci blocks
                        tma_load_3d(a_dst + A_BYTES / 2, &map_w, c0 + 64, k * KS, 0, bar);
                    }
                    tma_load_4d(b_dst, &map_act, pix[0], k * KS, img[0], 0, bar);       // [comp][32 ch][64 px]
                    tma_load_4d(b_dst + B_BOX_BYTES, &map_act, pix[1], k * KS, img[1], 0, bar);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        // ONE thread runs this whole loop: waits, descriptor arithmetic and tcgen05.mma / commit. What that thread executes
        // between two MMAs is time the tensor pipe idles (its queue is shallow), so the loop carries no division, no warp
        // synchronisation and no descriptor construction: the two 64-bit shared-memory descriptors of a stage are built
        // once, and an MMA's descriptors are those with a constant added to the address field of the low word (addresses
        // are 16-byte units below 2^14, so the addition never carries into the neighbouring field).
        if (lane == 0) {
            int s = 0, local_tile = 0;
            uint32_t par = 0;                                    // phase parity of stage s
            bool ok = true;
            const uint32_t idesc_pos = make_idesc_f16(p.fmt, CT, PT, BWD, true, false, false);
            const uint32_t idesc_neg = make_idesc_f16(p.fmt, CT, PT, BWD, true, true, false);
            uint32_t a_lo = 0, a_hi = 0, b_lo = 0, b_hi = 0;
            auto issue = [&](int j, int i, int o, uint32_t accumulate) {
                const int r = i ^ o;
                const bool neg = BWD ? quat_negative(o, i) : quat_negative(i, o);
                const uint32_t a_off = BWD ? (uint32_t)(r * (KS * 128) + j * 2048) >> 4 : (uint32_t)(r * (CT * KS * 2) + j * 32) >> 4;
                const uint32_t b_off = (uint32_t)(i * (KS * 128) + j * 2048) >> 4;
                mma_f16_ss_words(tmem_base + o * PT, a_lo + a_off, a_hi, b_lo + b_off, b_hi, neg ? idesc_neg : idesc_pos, accumulate);
            };
            if (resident && blockIdx.x < n_tiles) ok = mbar_wait_bounded(a_full, 0, status, ST_U_MMA);
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++local_tile) {
                for (int k = 0; k < n_k && ok; ++k) {
                    ok = mbar_wait_bounded(full_bar + 8 * s, par, status, ST_U_MMA);
                    if (!ok) break;
                    tc_fence_after_sync();
                    {
                        const uint64_t ad = BWD ? make_desc_mnmajor(a_slot(k, s), A_BYTES / 2) : make_desc_kmajor_sw64(a_slot(k, s));
                        const uint64_t bd = make_desc_mnmajor(b_slot(s), B_BOX_BYTES);
                        a_lo = (uint32_t)ad; a_hi = (uint32_t)(ad >> 32); b_lo = (uint32_t)bd; b_hi = (uint32_t)(bd >> 32);
                    }
                    // A tile's MMAs go round the four accumulators (i = streamed component, o = accumulator component), except at
                    // its two ends, where they are issued pair-wise (accumulators 0,1 then 2,3):
                    //  - the first K step of the first slice: each pair starts as soon as the epilogue of the previous tile has
                    //    drained it;
                    //  - the last K step of the last slice: the first pair is complete (and signalled) while the second still
                    //    computes, so its drain overlaps those MMAs.
                    // Inside a pair the MMAs alternate between the two accumulators (back-to-back MMAs into one accumulator run at
                    // two thirds of the rate of independent ones).
                    constexpr int J = KS / 16;
                    const bool first = k == 0, last = k == n_k - 1;
                    if (first) {
#pragma unroll
                        for (int pair = 0; pair < 2; ++pair) {
                            if (local_tile > 0) {
                                ok = ok && mbar_wait_bounded(tmem_empty + 8 * (2 * pair), (local_tile - 1) & 1, status, ST_U_MMA) &&
                                     mbar_wait_bounded(tmem_empty + 8 * (2 * pair + 1), (local_tile - 1) & 1, status, ST_U_MMA);
                                tc_fence_after_sync();
                            }
                            if (ok) {
#pragma unroll
                                for (int i = 0; i < 4; ++i)
#pragma unroll
                                    for (int oo = 0; oo < 2; ++oo) issue(0, i, 2 * pair + oo, i > 0 ? 1u : 0u);
                            }
                        }
                        if (!ok) break;
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
#pragma unroll
                            for (int o = 0; o < 4; ++o) issue(0, i, o, 1u);
                    }
#pragma unroll
                    for (int j = 1; j < J - 1; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i)
#pragma unroll
                            for (int o = 0; o < 4; ++o) issue(j, i, o, 1u);
                    if (last) {
#pragma unroll
                        for (int pair = 0; pair < 2; ++pair) {
#pragma unroll
                            for (int i = 0; i < 4; ++i)
#pragma unroll
                                for (int oo = 0; oo < 2; ++oo) issue(J - 1, i, 2 * pair + oo, 1u);
                            mma_commit(pair == 0 ? tmem_full0 : tmem_full1);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
#pragma unroll
                            for (int o = 0; o < 4; ++o) issue(J - 1, i, o, 1u);
                    }
                    mma_commit(empty_bar + 8 * s);
                    if (++s == n_stages) { s = 0; par ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9)
        // Ordinary global stores from here cost more than their bandwidth: every lane owns another channel row, so
        // a warp store scatters 32 segments, and while those queue up the MMA warp's own instructions wait behind
        // them. The tile therefore leaves through shared memory and TMA stores: each thread writes its row of one
        // component into a 128-byte-swizzled [128 channels][64 pixels] box (conflict-free 16-byte stores). Every warp owns the
        // 4 KB of that box that hold its 32 rows and stores them itself ([32 channels][64 pixels] per bulk store), so the eight
        // warps never wait for one another: a warp only waits for its own previous store to have read its 4 KB. Out-of-range rows
        // and pixels are clipped by the tensor map.
        const int q = warp & 3;                   // TMEM lane quadrant this warp may read
        const int chalf = (warp - 2) >> 2;        // which 64-pixel block of the tile (64 accumulator columns)
        const int row = q * 32 + lane;
        const uint32_t warp_out = out_addr + chalf * OUT_HALF_BYTES + q * (32 * 128);   // this warp's 32 rows of 128 bytes
        const uint32_t my_out = warp_out + lane * 128;
        int local_tile = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++local_tile) {
            const int px_tile = tile / p.n_c_tiles, c_tile = tile - px_tile * p.n_c_tiles;
            const int c = c_tile * CT + row;
            // Drain: all eight warps read component 0 (a 64-column half each) and release it, then 1, 2, 3, so the MMA
            // warp starts the next tile on component 0 while the others are still being read. Components 0 and 1 are
            // complete before 2 and 3 (see the MMA warp). The values wait as packed 16-bit pairs in registers; nothing
            // slow sits between two releases.
            uint32_t packed[4][32];
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + chalf * 64;
#pragma unroll
            for (int o = 0; o < 4; ++o) {
                if ((o & 1) == 0) {
                    ok = mbar_wait_bounded(o == 0 ? tmem_full0 : tmem_full1, local_tile & 1, status, ST_U_EPILOGUE);
                    ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
                    if (!ok) break;
                    tc_fence_after_sync();
                }
                float badd = 0.f;
                if (!BWD && p.has_bias && c < p.Cout) {
                    const uint16_t raw = bias[o * p.Cout + c];
                    badd = p.fmt == 0 ? __half2float(__ushort_as_half(raw)) : __bfloat162float(__ushort_as_bfloat16(raw));
                }
                uint32_t v[64];
                tmem_ld_32x32b_x64(lane_addr + o * PT, v);
                tmem_ld_wait();
                tmem_regs_ready(v);
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_empty + 8 * o);
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const float f0 = __uint_as_float(v[2 * e]) + badd, f1 = __uint_as_float(v[2 * e + 1]) + badd;
                    if (p.fmt == 0) { const __half2 h = __floats2half2_rn(f0, f1); packed[o][e] = *reinterpret_cast<const uint32_t*>(&h); }
                    else { const __nv_bfloat162 h = __floats2bfloat162_rn(f0, f1); packed[o][e] = *reinterpret_cast<const uint32_t*>(&h); }
                }
            }
            if (!ok) break;
            const int blk = 2 * px_tile + chalf;
            const int img = blk / p.blocks_per_image;
            const int pix = (blk - img * p.blocks_per_image) * 64;
#pragma unroll
            for (int o = 0; o < 4; ++o) {
                if (lane == 0) bulk_wait_read_all();       // this warp's previous store has read its rows
                __syncwarp();
#pragma unroll
                for (int ch = 0; ch < 8; ++ch)              // 16-byte chunk ch of this row sits at position ch ^ (row % 8)
                    st_shared_v4(my_out + ((ch ^ (row & 7)) << 4), packed[o][4 * ch], packed[o][4 * ch + 1], packed[o][4 * ch + 2], packed[o][4 * ch + 3]);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (img < p.Nb) tma_store_4d(&map_out, warp_out, pix, c_tile * CT + q * 32, img, o);
                    bulk_commit_group();
                }
            }
        }
        if (lane == 0) bulk_wait_read_all();                // shared memory must outlive the last bulk store's reads
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}


// ===================================================================================================
// Backward-filter of the pointwise convolution, same idea: one accumulator per filter component r,
//   D_r[co, ci] += s(l, l^r) * dy_{l^r}[co, px-slice] * x_l[ci, px-slice]^T          l, r = 0..3
// Both operands are K-major here (pixels are contiguous in memory), 32 pixels per stage and component
// (64-byte rows, 64-byte swizzle). K = all pixels of all images, split across the grid; every CTA adds its
// 4 x 128 x 128 partial sums into the fp32 scratch with vector reductions and a last pass casts to the
// tensor type (replaces src/backend/cudnn/quat_pointwise_conv2d.cu:331-607).
// ===================================================================================================
constexpr int FKP = 32;                                  // pixels per stage
constexpr uint32_t F_OP_BYTES = 4 * 128 * FKP * 2;       // 32 KB per operand per stage
constexpr uint32_t F_STAGE_BYTES = 2 * F_OP_BYTES;
constexpr size_t F_SMEM_BYTES = 1024 + U_STAGES * F_STAGE_BYTES + 256;

struct FParams {
    int Nb, Co, Ci, HW;
    int blocks_per_image;     // ceil(HW / 32)
    int n_co_tiles, n_ci_tiles;
    int steps_total;          // Nb * blocks_per_image
    int steps_per_split;
    int fmt;
};

__global__ void __launch_bounds__(U_THREADS, 1)
qconv_pointwise_filter_tc_kernel(const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_x, FParams p,
                                 float* __restrict__ dw32, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + U_STAGES * F_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * U_STAGES + 1);
    const uint32_t tiles_addr = smem_u32(base);
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + U_STAGES), tmem_full = smem_u32(bars + 2 * U_STAGES);

    const int n_out_tiles = p.n_co_tiles * p.n_ci_tiles;
    const int out_tile = blockIdx.x % n_out_tiles, split = blockIdx.x / n_out_tiles;
    const int co0 = (out_tile / p.n_ci_tiles) * 128, ci0 = (out_tile % p.n_ci_tiles) * 128;
    const int step_beg = split * p.steps_per_split;
    const int step_end = min(p.steps_total, step_beg + p.steps_per_split);
    const int n_steps = max(0, step_end - step_beg);

    if (t == 0) {
        for (int s = 0; s < U_STAGES; ++s) { mbar_init(full_bar + 8 * s, 1); mbar_init(empty_bar + 8 * s, 1); }
        mbar_init(tmem_full, 1);
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            for (int it = 0; it < n_steps && ok; ++it) {
                const int s = it % U_STAGES;
                ok = mbar_wait_bounded(empty_bar + 8 * s, ((it / U_STAGES) & 1) ^ 1, status, ST_U_PRODUCER);
                if (!ok) break;
                const int step = step_beg + it;
                const int img = step / p.blocks_per_image, px0 = (step - img * p.blocks_per_image) * FKP;
                const uint32_t a_dst = tiles_addr + s * F_STAGE_BYTES, bar = full_bar + 8 * s;
                mbar_arrive_expect_tx(bar, F_STAGE_BYTES);
                tma_load_4d(a_dst, &map_dy, px0, co0, img, 0, bar);                 // [d][128 co][32 px]
                tma_load_4d(a_dst + F_OP_BYTES, &map_x, px0, ci0, img, 0, bar);     // [l][128 ci][32 px]
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {                       // one thread: waits, stepped descriptors, MMAs (see the forward kernel)
            bool ok = true;
            int s = 0;
            uint32_t par = 0;
            const uint32_t idesc_pos = make_idesc_f16(p.fmt, 128, 128, false, false, false, false);
            const uint32_t idesc_neg = make_idesc_f16(p.fmt, 128, 128, false, false, true, false);
            for (int it = 0; it < n_steps && ok; ++it) {
                ok = mbar_wait_bounded(full_bar + 8 * s, par, status, ST_U_MMA);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t ad = make_desc_kmajor_sw64(tiles_addr + s * F_STAGE_BYTES);
                const uint64_t bd = make_desc_kmajor_sw64(tiles_addr + s * F_STAGE_BYTES + F_OP_BYTES);
                const uint32_t a_lo = (uint32_t)ad, a_hi = (uint32_t)(ad >> 32), b_lo = (uint32_t)bd, b_hi = (uint32_t)(bd >> 32);
#pragma unroll
                for (int j = 0; j < FKP / 16; ++j) {
#pragma unroll
                    for (int l = 0; l < 4; ++l) {
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            const int d = l ^ r;
                            const uint32_t a_off = (uint32_t)(d * (128 * FKP * 2) + j * 32) >> 4, b_off = (uint32_t)(l * (128 * FKP * 2) + j * 32) >> 4;
                            mma_f16_ss_words(tmem_base + r * 128, a_lo + a_off, a_hi, b_lo + b_off, b_hi, quat_negative(l, d) ? idesc_neg : idesc_pos,
                                             (it > 0 || j > 0 || l > 0) ? 1u : 0u);
                        }
                    }
                }
                mma_commit(empty_bar + 8 * s);
                if (it == n_steps - 1) mma_commit(tmem_full);
                if (++s == U_STAGES) { s = 0; par ^= 1u; }
            }
            if (n_steps == 0) mbar_arrive(tmem_full);
        }
        __syncwarp();
    } else {
        const int q = warp & 3, half = (warp - 2) >> 2;
        bool ok = mbar_wait_bounded(tmem_full, 0, status, ST_U_EPILOGUE);
        ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
        tc_fence_after_sync();
        if (ok && n_steps > 0) {
            const int co = co0 + q * 32 + lane;
#pragma unroll 1
            for (int rr = 0; rr < 2; ++rr) {
                const int r = 2 * half + rr;
#pragma unroll 1
                for (int cb = 0; cb < 4; ++cb) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + r * 128 + cb * 32, v);
                    tmem_ld_wait();
                    if (co >= p.Co) continue;
                    float* dst = dw32 + ((size_t)r * p.Co + co) * p.Ci + ci0 + cb * 32;
#pragma unroll
                    for (int g4 = 0; g4 < 8; ++g4) {
                        if (ci0 + cb * 32 + g4 * 4 < p.Ci)
                            red_add_f32x4(dst + g4 * 4, __uint_as_float(v[4 * g4]), __uint_as_float(v[4 * g4 + 1]),
                                       __uint_as_float(v[4 * g4 + 2]), __uint_as_float(v[4 * g4 + 3]));
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

template <typename T>
__global__ void cast_f32_kernel(const float* __restrict__ src, T* __restrict__ dst, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) DType<T>::store(dst + i, src[i]);
}

int make_map(CUtensorMap* map, int fmt, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
             const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
    return make_tensor_map(map, fmt == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ptr, rank, dims, strides_bytes,
                           box, nullptr, swizzle, "pointwise operand");
}

}  // namespace

bool pointwise_tc_supported(Pass pass, int dtype, int variant, const Geom& g) {
    if (pass != PASS_FWD && pass != PASS_BWD_DATA) return false;
    if (dtype != PCB_F16 && dtype != PCB_BF16) return false;
    if (g.nc != 4 || variant != PCB_VARIANT_16_PRODUCT || g.real_in || g.w_io || g.dw_io) return false;   // quaternion-only kernels
    if (!(g.KH == 1 && g.KW == 1 && g.SH == 1 && g.SW == 1 && g.PT == 0 && g.PL == 0 && g.HO == g.H && g.WO == g.W)) return false;
    const int cout = pass == PASS_FWD ? g.Co : g.Ci;
    // TMA: every global stride a multiple of 16 bytes. The channel tile is 128 wide, so a layer with fewer output channels
    // wastes MMA rows -- but such layers are bound by HBM, and this kernel reads and writes the tensors exactly once,
    // straight from and to the reference layout (measured: 5-9x the staged kernels on 16- and 64-channel layers).
    // Below 32 channels the fixed cost per tile (32 MMAs whatever the channel count) outweighs that.
    return (g.Ci % 8 == 0) && (g.Co % 8 == 0) && ((g.H * g.W) % 8 == 0) && (cout >= 96 || (g.Ci >= 32 && g.Co >= 32));
}

int pointwise_tc_launch(Pass pass, int dtype, const Geom& g, const void* w, const void* act, const void* bias, void* out,
                        int* status, cudaStream_t stream) {
    const int fmt = dtype == PCB_F16 ? 0 : 1;
    const int HW = g.H * g.W;
    const bool bwd = pass == PASS_BWD_DATA;
    UParams p;
    p.Nb = g.Nb; p.HW = HW; p.fmt = fmt; p.has_bias = (!bwd && g.has_bias) ? 1 : 0; p.bwd = bwd ? 1 : 0;
    p.Cout = bwd ? g.Ci : g.Co;
    p.Cred = bwd ? g.Co : g.Ci;
    p.blocks_per_image = (HW + 63) / 64;
    const int blocks = p.blocks_per_image * g.Nb;
    p.n_px_tiles = (blocks + 1) / 2;
    p.n_c_tiles = (p.Cout + CT - 1) / CT;

    alignas(64) CUtensorMap map_w, map_act, map_out;
    {   // filters [4][Co][Ci]: (ci, co, r)
        const cuuint64_t dims[3] = {(cuuint64_t)g.Ci, (cuuint64_t)g.Co, 4};
        const cuuint64_t strides[2] = {(cuuint64_t)g.Ci * 2, (cuuint64_t)g.Co * g.Ci * 2};
        int rc;
        if (!bwd) { const cuuint32_t box[3] = {KS, CT, 4}; rc = make_map(&map_w, fmt, w, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B); }
        else      { const cuuint32_t box[3] = {64, KS, 4}; rc = make_map(&map_w, fmt, w, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B); }
        if (rc != PCB_OK) return rc;
    }
    {   // activations [4][Nb][C][HW]: (px, channel, image, component)
        const int C = p.Cred;
        const cuuint64_t dims[4] = {(cuuint64_t)HW, (cuuint64_t)C, (cuuint64_t)g.Nb, 4};
        const cuuint64_t strides[3] = {(cuuint64_t)HW * 2, (cuuint64_t)C * HW * 2, (cuuint64_t)g.Nb * C * HW * 2};
        const cuuint32_t box[4] = {64, KS, 1, 4};
        const int rc = make_map(&map_act, fmt, act, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != PCB_OK) return rc;
    }
    {   // output [4][Nb][Cout][HW]: (px, channel, image, component); every epilogue warp stores [32 channels][64 pixels] boxes
        const cuuint64_t dims[4] = {(cuuint64_t)HW, (cuuint64_t)p.Cout, (cuuint64_t)g.Nb, 4};
        const cuuint64_t strides[3] = {(cuuint64_t)HW * 2, (cuuint64_t)p.Cout * HW * 2, (cuuint64_t)g.Nb * p.Cout * HW * 2};
        const cuuint32_t box[4] = {64, 32, 1, 1};
        const int rc = make_map(&map_out, fmt, out, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != PCB_OK) return rc;
    }
    const int n_tiles = p.n_px_tiles * p.n_c_tiles;
    int grid = n_tiles < sm_count() ? n_tiles : sm_count();
    // forward with at most 128 reduced channels: keep the CTA's weight slices in shared memory for all its tiles
    // (halves the L2 -> shared-memory traffic); needs every CTA to stay on one channel tile
    p.a_resident = 0;
    if (!bwd && (p.Cred + KS - 1) / KS <= MAX_RESIDENT_K && grid >= p.n_c_tiles) {
        grid -= grid % p.n_c_tiles;
        p.a_resident = 1;
    }
    if (!bwd) {
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_pointwise_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)U_SMEM_BYTES));
        qconv_pointwise_tc_kernel<false><<<grid, U_THREADS, U_SMEM_BYTES, stream>>>(map_w, map_act, map_out, p, (const uint16_t*)bias, status);
    } else {
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_pointwise_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)U_SMEM_BYTES));
        qconv_pointwise_tc_kernel<true><<<grid, U_THREADS, U_SMEM_BYTES, stream>>>(map_w, map_act, map_out, p, (const uint16_t*)bias, status);
    }
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

bool pointwise_filter_tc_supported(int dtype, int variant, const Geom& g) {
    if (dtype != PCB_F16 && dtype != PCB_BF16) return false;
    if (g.nc != 4 || variant != PCB_VARIANT_16_PRODUCT || g.real_in || g.w_io || g.dw_io) return false;   // quaternion-only kernels
    if (!(g.KH == 1 && g.KW == 1 && g.SH == 1 && g.SW == 1 && g.PT == 0 && g.PL == 0 && g.HO == g.H && g.WO == g.W)) return false;
    return (g.Ci % 8 == 0) && (g.Co % 8 == 0) && ((g.H * g.W) % 8 == 0) && g.Ci >= 32 && g.Co >= 32;
}

int pointwise_filter_tc_launch(int dtype, const Geom& g, const void* dy, const void* x, void* dw, float* scratch, int* status,
                               cudaStream_t stream) {
    const int fmt = dtype == PCB_F16 ? 0 : 1;
    const int HW = g.H * g.W;
    FParams p;
    p.Nb = g.Nb; p.Co = g.Co; p.Ci = g.Ci; p.HW = HW; p.fmt = fmt;
    p.blocks_per_image = (HW + FKP - 1) / FKP;
    p.n_co_tiles = (g.Co + 127) / 128;
    p.n_ci_tiles = (g.Ci + 127) / 128;
    p.steps_total = g.Nb * p.blocks_per_image;
    const int n_out_tiles = p.n_co_tiles * p.n_ci_tiles;
    int splits = sm_count() / n_out_tiles;
    if (splits < 1) splits = 1;
    if (splits > p.steps_total) splits = p.steps_total;
    p.steps_per_split = (p.steps_total + splits - 1) / splits;
    splits = (p.steps_total + p.steps_per_split - 1) / p.steps_per_split;

    alignas(64) CUtensorMap map_dy, map_x;
    const cuuint32_t box[4] = {FKP, 128, 1, 4};
    {
        const cuuint64_t dims[4] = {(cuuint64_t)HW, (cuuint64_t)g.Co, (cuuint64_t)g.Nb, 4};
        const cuuint64_t strides[3] = {(cuuint64_t)HW * 2, (cuuint64_t)g.Co * HW * 2, (cuuint64_t)g.Nb * g.Co * HW * 2};
        const int rc = make_map(&map_dy, fmt, dy, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc != PCB_OK) return rc;
    }
    {
        const cuuint64_t dims[4] = {(cuuint64_t)HW, (cuuint64_t)g.Ci, (cuuint64_t)g.Nb, 4};
        const cuuint64_t strides[3] = {(cuuint64_t)HW * 2, (cuuint64_t)g.Ci * HW * 2, (cuuint64_t)g.Nb * g.Ci * HW * 2};
        const int rc = make_map(&map_x, fmt, x, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc != PCB_OK) return rc;
    }
    const size_t numel = (size_t)4 * g.Co * g.Ci;
    PCB_CUDA_TRY(cudaMemsetAsync(scratch, 0, numel * sizeof(float), stream));
    if (pointwise_filter_pair_tc_supported(g)) {        // multiples of 256 output channels: 256 x 128 blocks on pairs of SMs
        const int rc = pointwise_filter_pair_tc_launch(fmt, g, dy, x, scratch, status, stream);
        if (rc != PCB_OK) return rc;
    } else {
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_pointwise_filter_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F_SMEM_BYTES));
        qconv_pointwise_filter_tc_kernel<<<n_out_tiles * splits, U_THREADS, F_SMEM_BYTES, stream>>>(map_dy, map_x, p, scratch, status);
        PCB_CUDA_TRY(cudaGetLastError());
    }
    const int blocks = (int)((numel + 255) / 256 < 1184 ? (numel + 255) / 256 : 1184);
    if (dtype == PCB_F16) cast_f32_kernel<__half><<<blocks, 256, 0, stream>>>(scratch, (__half*)dw, numel);
    else cast_f32_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(scratch, (__nv_bfloat16*)dw, numel);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

}  // namespace pcb
