// Forward pointwise (1x1, stride 1) quaternion convolution on PAIRS of SMs: the kernel of pointwise_tc.cu with every
// tcgen05.mma issued for a two-CTA cluster (cta_group::2), for layers with a multiple of 256 output channels and at most
// 128 input channels (the benchmark layer: 128 -> 256 channels).
//
// A CTA pair computes a 256 x 128 tile per accumulator: each SM holds 128 of the 256 output channels (its own filter rows,
// resident in its shared memory) and HALF of the 128 pixels of the streamed activation tile; the tensor cores of both SMs read
// the two halves across the pair. Per MMA and SM that is 4 KB + 2 KB of shared-memory operand reads instead of 8 KB, and each
// activation tile is fetched from L2 once per 256 channels instead of once per 128.
// What it buys, measured on the 128 -> 256 channel layer at 56 x 56: with one pass over the K slices per tile, 3-4 % (the steady
// 75-80 clocks per MMA are the tensor pipe's own rate for 128-column MMAs, not a shared-memory limit). The larger gain is the
// schedule the four-stage activation ring allows: all K slices of a tile are resident at once, so a tile is issued in TWO
// PHASES (accumulators 0,1 over every slice, then 2,3 over every slice) and the epilogue's drain of one accumulator pair always
// overlaps the MMAs of the other: forward 0.185 -> 0.165 ms.
//
//   D_d[co, px] += s(l,d) * w[l^d][co, ci-slice] * x_l[ci-slice, px]      d, l = 0..3       (src/algebras.cc:28-49)
//
// Roles per CTA: warp 0 = TMA producer (its filter rows once; its 64-pixel half of every activation stage), warp 1 = tensor
// memory (allocated for the pair by both CTAs) and, in the even CTA only, the thread that issues all MMAs and commits;
// warps 2-9 = epilogue of this CTA's 128 channels. Barriers: `full` lives in the even CTA and counts the bytes of both
// CTAs' copies (each copy names that barrier through its cluster address; these are ordinary TMA loads of this GPU's
// memory, one destination each); `empty` and `tmem_full` exist in both CTAs and the issuing thread commits to each of them;
// `tmem_empty` lives in the even CTA and takes the arrivals of both CTAs' epilogue warps. Every wait is bounded; on expiry
// the status word is set and everybody leaves through the common teardown (a cluster barrier, then the pair's tensor
// memory is released).
#include <cuda_runtime.h>

#include "tc_common.cuh"
#include "tensor_path.cuh"

namespace pcb {
namespace {

using namespace umma;
using namespace tc;

constexpr int P_CT = 128;                              // channels per CTA (MMA M = 256 for the pair)
constexpr int P_PT = 128;                              // pixels per tile (MMA N), 64 held by each CTA
constexpr int P_KS = 32;                               // channels per component per stage
constexpr int P_STAGES = 4;
constexpr int P_MAX_K = 4;                             // resident filter slices (4 x 32 KB)
constexpr uint32_t P_A_BYTES = 4 * P_CT * P_KS * 2;    // 32 KB: four filter components of one K slice
constexpr uint32_t P_B_BYTES = 4 * P_KS * 64 * 2;      // 16 KB: this CTA's 64 pixels of four activation components
constexpr uint32_t P_OUT_HALF = 64 * P_CT * 2;         // 16 KB: one component of a 64-pixel block, [128 channels][64 pixels]
constexpr uint32_t P_OUT_BYTES = 2 * P_OUT_HALF;
constexpr int P_THREADS = 320;
constexpr size_t P_SMEM_BYTES = 1024 + P_MAX_K * P_A_BYTES + P_STAGES * P_B_BYTES + P_OUT_BYTES + 256;
constexpr int ST_P_PRODUCER = 0x10000, ST_P_MMA = 0x20000, ST_P_EPILOGUE = 0x40000;

struct PParams {
    int Nb, Cout, Cred, HW;
    int blocks_per_image;        // ceil(HW / 64)
    int n_px_tiles, n_cp;        // pixel tiles (128 pixels), channel pairs (256 channels)
    int fmt, has_bias;
};

constexpr uint64_t DESC_SWIZZLE_64B_P = 4ull << 61;
__device__ __forceinline__ uint64_t desc_kmajor_sw64_p(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(512 >> 4) << 32) | DESC_VERSION_SM100 | DESC_SWIZZLE_64B_P;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Cluster address of the location `local_addr` (a shared::cta address of this CTA) in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Relaxed: the arrival orders nothing but the tensor-memory reads before it, which tcgen05.wait::ld and the tcgen05 fences on
// both sides already order; a cluster-scope release here made every arrival wait for the thread's outstanding stores.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA loads of one box into this CTA's shared memory whose bytes are counted by a barrier given by its cluster address
// (the even CTA's `full` barrier). One destination, no multicast.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem_addr, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem_addr), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t tmem_addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_addr), "r"(cols) : "memory");
}
// D[tmem of both CTAs] (+)= A * B for the pair; issued by one thread of the even CTA. Descriptors as two 32-bit words.
__device__ __forceinline__ void mma_f16_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// Arrives on the barrier at the given cluster address once every MMA issued so far for the pair has completed.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar_cluster) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}

__global__ void __launch_bounds__(P_THREADS, 1)
qconv_pointwise_pair_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_act,
                               const __grid_constant__ CUtensorMap map_out, PParams p, const uint16_t* __restrict__ bias, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const uint32_t rank = cluster_ctarank();           // 0 = even CTA (issues the MMAs), 1 = its peer
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr uint32_t OPERANDS = P_MAX_K * P_A_BYTES + P_STAGES * P_B_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + OPERANDS + P_OUT_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * P_STAGES + 9);
    const uint32_t tiles_addr = smem_u32(base);
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + P_STAGES);
    const uint32_t tmem_full0 = smem_u32(bars + 2 * P_STAGES), tmem_full1 = smem_u32(bars + 2 * P_STAGES + 1);
    const uint32_t tmem_empty = smem_u32(bars + 2 * P_STAGES + 2);        // four barriers, one per component (even CTA)
    const uint32_t a_full = smem_u32(bars + 2 * P_STAGES + 6);
    const uint32_t out_addr = tiles_addr + OPERANDS;

    const int n_tiles = p.n_px_tiles * p.n_cp;
    const int n_k = (p.Cred + P_KS - 1) / P_KS;
    const int cp = pair % p.n_cp;                       // the grid holds a multiple of n_cp pairs: a pair keeps its channels
    const int c0 = cp * 2 * P_CT + (int)rank * P_CT;    // first output channel of this CTA
    auto a_slot = [&](int k) { return tiles_addr + k * P_A_BYTES; };
    auto b_slot = [&](int s) { return tiles_addr + P_MAX_K * P_A_BYTES + s * P_B_BYTES; };

    if (t == 0) {
        for (int s = 0; s < P_STAGES; ++s) { mbar_init(full_bar + 8 * s, 1); mbar_init(empty_bar + 8 * s, 1); }
        mbar_init(tmem_full0, 1); mbar_init(tmem_full1, 1);
        for (int o = 0; o < 4; ++o) mbar_init(tmem_empty + 8 * o, 16);   // eight epilogue warps of each CTA
        mbar_init(a_full, 1);
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                                 // both CTAs' barriers exist before anything signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (both CTAs)
        if (lane == 0) {
            int s = 0;
            uint32_t par = 1;                            // parity the `empty` barrier of stage s is waited with
            bool ok = true;
            const uint32_t lead_a_full = map_to_cta(a_full, 0);
            if (pair < n_tiles) {
                if (rank == 0) mbar_arrive_expect_tx(a_full, 2u * (uint32_t)n_k * P_A_BYTES);
                for (int k = 0; k < n_k; ++k) tma_load_3d_pair(a_slot(k), &map_w, k * P_KS, c0, 0, lead_a_full);   // [r][128 co][32 ci]
            }
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
                const int px_tile = tile / p.n_cp;
                const int blk = 2 * px_tile + (int)rank;                   // this CTA's 64-pixel block of the tile
                const int img = blk / p.blocks_per_image;                  // == Nb past the end: fully out of range -> zeros
                const int pix = (blk - img * p.blocks_per_image) * 64;
                for (int k = 0; k < n_k && ok; ++k) {
                    ok = mbar_wait_bounded(empty_bar + 8 * s, par, status, ST_P_PRODUCER);
                    if (!ok) break;
                    if (rank == 0) mbar_arrive_expect_tx(full_bar + 8 * s, 2u * P_B_BYTES);
                    tma_load_4d_pair(b_slot(s), &map_act, pix, k * P_KS, img, 0, map_to_cta(full_bar + 8 * s, 0));   // [comp][32 ch][64 px]
                    if (++s == P_STAGES) { s = 0; par ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (even CTA, one thread)
        if (lane == 0 && rank == 0) {
            int s = 0, local_tile = 0;
            uint32_t par = 0;
            bool ok = true;
            const uint32_t idesc_pos = make_idesc_f16(p.fmt, 2 * P_CT, P_PT, false, true, false, false);
            const uint32_t idesc_neg = make_idesc_f16(p.fmt, 2 * P_CT, P_PT, false, true, true, false);
            const uint32_t peer_empty = map_to_cta(empty_bar, 1), peer_full0 = map_to_cta(tmem_full0, 1), peer_full1 = map_to_cta(tmem_full1, 1);
            uint32_t a_lo = 0, a_hi = 0, b_lo = 0, b_hi = 0;
            auto issue = [&](int j, int i, int o, uint32_t accumulate) {
                const int r = i ^ o;
                const uint32_t a_off = (uint32_t)(r * (P_CT * P_KS * 2) + j * 32) >> 4;
                const uint32_t b_off = (uint32_t)(i * (P_KS * 128) + j * 2048) >> 4;
                mma_f16_pair(tmem_base + o * P_PT, a_lo + a_off, a_hi, b_lo + b_off, b_hi, quat_negative(i, o) ? idesc_neg : idesc_pos, accumulate);
            };
            // A tile is issued in two phases. All its K slices fit the activation ring (n_k <= P_STAGES), so phase A runs every
            // slice into accumulators 0,1 and signals them complete, and phase B runs the same slices again into accumulators
            // 2,3, releasing each stage as it goes. The epilogue drains 0,1 while phase B computes and 2,3 while the next tile's
            // phase A computes: the turnover of the single-buffered accumulators costs no tensor time (with one pass over
            // the slices, both pairs completed at the very end of the tile and the next tile waited for their drain).
            // Inside a phase the MMAs alternate between the two accumulators of the pair.
            if (pair < n_tiles) ok = mbar_wait_bounded(a_full, 0, status, ST_P_MMA);
            uint32_t a_lo_k[P_MAX_K], a_hi_k[P_MAX_K], b_lo_k[P_MAX_K], b_hi_k[P_MAX_K];
            int s_k[P_MAX_K];
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++local_tile) {
#pragma unroll
                for (int ph = 0; ph < 2; ++ph) {
                    if (local_tile > 0) {           // both CTAs' epilogues have drained this pair of the previous tile
                        ok = ok && mbar_wait_bounded(tmem_empty + 8 * (2 * ph), (local_tile - 1) & 1, status, ST_P_MMA) &&
                             mbar_wait_bounded(tmem_empty + 8 * (2 * ph + 1), (local_tile - 1) & 1, status, ST_P_MMA);
                        if (!ok) break;
                        tc_fence_after_sync();
                    }
#pragma unroll
                    for (int k = 0; k < P_MAX_K; ++k) {
                        if (k >= n_k) break;
                        if (ph == 0) {              // first touch of the slice: wait for its data, keep its descriptors
                            ok = mbar_wait_bounded(full_bar + 8 * s, par, status, ST_P_MMA);
                            if (!ok) break;
                            tc_fence_after_sync();
                            const uint64_t ad = desc_kmajor_sw64_p(a_slot(k));
                            const uint64_t bd = make_desc_mnmajor(b_slot(s), P_B_BYTES);
                            a_lo_k[k] = (uint32_t)ad; a_hi_k[k] = (uint32_t)(ad >> 32); b_lo_k[k] = (uint32_t)bd; b_hi_k[k] = (uint32_t)(bd >> 32);
                            s_k[k] = s;
                            if (++s == P_STAGES) { s = 0; par ^= 1u; }
                        }
                        a_lo = a_lo_k[k]; a_hi = a_hi_k[k]; b_lo = b_lo_k[k]; b_hi = b_hi_k[k];
#pragma unroll
                        for (int j = 0; j < P_KS / 16; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i)
#pragma unroll
                                for (int oo = 0; oo < 2; ++oo) issue(j, i, 2 * ph + oo, (k > 0 || j > 0 || i > 0) ? 1u : 0u);
                        if (ph == 1) {              // the stage is free in both CTAs
                            mma_commit_pair(empty_bar + 8 * s_k[k]);
                            mma_commit_pair(peer_empty + 8 * s_k[k]);
                        }
                    }
                    if (!ok) break;
                    mma_commit_pair(ph == 0 ? tmem_full0 : tmem_full1);
                    mma_commit_pair(ph == 0 ? peer_full0 : peer_full1);
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9, both CTAs: own 128 channels)
        const int q = warp & 3;                   // TMEM lane quadrant this warp may read
        const int chalf = (warp - 2) >> 2;        // which 64-pixel block of the tile (64 accumulator columns)
        const int row = q * 32 + lane;
        const int c = c0 + row;
        // every warp owns the 4 KB of the staging box that hold its 32 rows and stores them itself: no warp waits for another
        const uint32_t warp_out = out_addr + chalf * P_OUT_HALF + q * (32 * 128);
        const uint32_t my_out = warp_out + lane * 128;
        const uint32_t lead_tmem_empty = map_to_cta(tmem_empty, 0);
        int local_tile = 0;
        bool ok = true;
        for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++local_tile) {
            const int px_tile = tile / p.n_cp;
            uint32_t packed[4][32];
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + chalf * 64;
#pragma unroll
            for (int o = 0; o < 4; ++o) {
                if ((o & 1) == 0) {
                    ok = mbar_wait_bounded(o == 0 ? tmem_full0 : tmem_full1, local_tile & 1, status, ST_P_EPILOGUE);
                    ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
                    if (!ok) break;
                    tc_fence_after_sync();
                }
                float badd = 0.f;
                if (p.has_bias && c < p.Cout) {
                    const uint16_t raw = bias[o * p.Cout + c];
                    badd = p.fmt == 0 ? __half2float(__ushort_as_half(raw)) : __bfloat162float(__ushort_as_bfloat16(raw));
                }
                uint32_t v[64];
                tmem_ld_32x32b_x64(lane_addr + o * P_PT, v);
                tmem_ld_wait();
                tmem_regs_ready(v);
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(lead_tmem_empty + 8 * o);   // this warp has drained component o
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
                    if (img < p.Nb) tma_store_4d(&map_out, warp_out, pix, c0 + q * 32, img, o);
                    bulk_commit_group();
                }
            }
        }
        if (lane == 0) bulk_wait_read_all();                // shared memory must outlive the last bulk store's reads
    }

    // teardown: nobody leaves while its peer may still signal its barriers or read its shared memory
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

// ===================================================================================================
// Backward-filter of the pointwise convolution on pairs of SMs (layers with a multiple of 256 output channels):
//   D_r[co, ci] += s(l, l^r) * dy_{l^r}[co, px-slice] * x_l[ci, px-slice]^T          l, r = 0..3
// A pair accumulates a 256 (co) x 128 (ci) block per filter component r: each SM holds its own 128 rows of dy and HALF (64
// rows) of the x tile, so a stage is 48 KB per SM instead of 64 KB, four stages fit where the single-SM kernel
// (pointwise_tc.cu) has three, and every x tile is fetched once per 256 output channels. K = all pixels of all images, split
// over the pairs; both SMs add their 4 x 128 x 128 partial sums into the fp32 scratch with vector reductions.
// Roles and barriers as in the forward kernel above (no accumulator hand-back: one accumulation per CTA pair).
// ===================================================================================================
constexpr int PF_KP = 32;                                // pixels per stage and component: 64-byte rows, 64-byte swizzle
constexpr int PF_STAGES = 4;
constexpr uint32_t PF_A_BYTES = 4 * 128 * PF_KP * 2;     // 32 KB: this CTA's 128 rows of the four dy components
constexpr uint32_t PF_B_BYTES = 4 * 64 * PF_KP * 2;      // 16 KB: this CTA's 64 rows of the four x components
constexpr uint32_t PF_STAGE_BYTES = PF_A_BYTES + PF_B_BYTES;
constexpr size_t PF_SMEM_BYTES = 1024 + PF_STAGES * PF_STAGE_BYTES + 256;

struct PFParams {
    int Nb, Co, Ci, HW;
    int blocks_per_image;     // ceil(HW / 32)
    int n_co_pairs, n_ci_tiles;
    int steps_total;          // Nb * blocks_per_image
    int steps_per_split;
    int fmt;
};

__global__ void __launch_bounds__(P_THREADS, 1)
qconv_pointwise_filter_pair_tc_kernel(const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_x, PFParams p,
                                      float* __restrict__ dw32, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const uint32_t rank = cluster_ctarank();
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + PF_STAGES * PF_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PF_STAGES + 1);
    const uint32_t tiles_addr = smem_u32(base);
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + PF_STAGES), tmem_full = smem_u32(bars + 2 * PF_STAGES);

    const int n_out_tiles = p.n_co_pairs * p.n_ci_tiles;
    const int pair = blockIdx.x >> 1;
    const int out_tile = pair % n_out_tiles, split = pair / n_out_tiles;
    const int co0 = (out_tile / p.n_ci_tiles) * 256 + (int)rank * 128;      // this CTA's rows of dy and of the result
    const int ci0 = (out_tile % p.n_ci_tiles) * 128;
    const int step_beg = split * p.steps_per_split;
    const int step_end = min(p.steps_total, step_beg + p.steps_per_split);
    const int n_steps = max(0, step_end - step_beg);

    if (t == 0) {
        for (int s = 0; s < PF_STAGES; ++s) { mbar_init(full_bar + 8 * s, 1); mbar_init(empty_bar + 8 * s, 1); }
        mbar_init(tmem_full, 1);
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                 // both CTAs' barriers exist before anybody signals across the pair
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (both CTAs: own dy rows, own half of x)
        if (lane == 0) {
            bool ok = true;
            int s = 0;
            uint32_t par = 1;           // parity of a stage that has never been used: the wait passes at once
            for (int it = 0; it < n_steps && ok; ++it) {
                ok = mbar_wait_bounded(empty_bar + 8 * s, par, status, ST_P_PRODUCER);
                if (!ok) break;
                const int step = step_beg + it;
                const int img = step / p.blocks_per_image, px0 = (step - img * p.blocks_per_image) * PF_KP;
                const uint32_t dst = tiles_addr + s * PF_STAGE_BYTES, lead_full = map_to_cta(full_bar + 8 * s, 0);
                if (rank == 0) mbar_arrive_expect_tx(full_bar + 8 * s, 2u * PF_STAGE_BYTES);
                tma_load_4d_pair(dst, &map_dy, px0, co0, img, 0, lead_full);                          // [d][128 co][32 px]
                tma_load_4d_pair(dst + PF_A_BYTES, &map_x, px0, ci0 + (int)rank * 64, img, 0, lead_full);   // [l][64 ci][32 px]
                if (++s == PF_STAGES) { s = 0; par ^= 1u; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (even CTA, one thread)
        if (lane == 0 && rank == 0) {
            bool ok = true;
            int s = 0;
            uint32_t par = 0;
            const uint32_t idesc_pos = make_idesc_f16(p.fmt, 256, 128, false, false, false, false);
            const uint32_t idesc_neg = make_idesc_f16(p.fmt, 256, 128, false, false, true, false);
            const uint32_t peer_empty = map_to_cta(empty_bar, 1), peer_tmem_full = map_to_cta(tmem_full, 1);
            for (int it = 0; it < n_steps && ok; ++it) {
                ok = mbar_wait_bounded(full_bar + 8 * s, par, status, ST_P_MMA);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t ad = desc_kmajor_sw64_p(tiles_addr + s * PF_STAGE_BYTES);
                const uint64_t bd = desc_kmajor_sw64_p(tiles_addr + s * PF_STAGE_BYTES + PF_A_BYTES);
                const uint32_t a_lo = (uint32_t)ad, a_hi = (uint32_t)(ad >> 32), b_lo = (uint32_t)bd, b_hi = (uint32_t)(bd >> 32);
#pragma unroll
                for (int j = 0; j < PF_KP / 16; ++j) {
#pragma unroll
                    for (int l = 0; l < 4; ++l) {
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            const int d = l ^ r;
                            const uint32_t a_off = (uint32_t)(d * (128 * PF_KP * 2) + j * 32) >> 4, b_off = (uint32_t)(l * (64 * PF_KP * 2) + j * 32) >> 4;
                            mma_f16_pair(tmem_base + r * 128, a_lo + a_off, a_hi, b_lo + b_off, b_hi, quat_negative(l, d) ? idesc_neg : idesc_pos,
                                         (it > 0 || j > 0 || l > 0) ? 1u : 0u);
                        }
                    }
                }
                mma_commit_pair(empty_bar + 8 * s);
                mma_commit_pair(peer_empty + 8 * s);
                if (it == n_steps - 1) { mma_commit_pair(tmem_full); mma_commit_pair(peer_tmem_full); }
                if (++s == PF_STAGES) { s = 0; par ^= 1u; }
            }
            if (n_steps == 0) { mbar_arrive(tmem_full); mbar_arrive_cluster(peer_tmem_full); }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9 of both CTAs: own 128 rows)
        const int q = warp & 3, half = (warp - 2) >> 2;
        bool ok = mbar_wait_bounded(tmem_full, 0, status, ST_P_EPILOGUE);
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
    // teardown: nobody leaves while its peer may still signal its barriers or read its shared memory
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

int make_map_p(CUtensorMap* map, int fmt, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
               const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
    return make_tensor_map(map, fmt == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ptr, rank, dims, strides_bytes,
                           box, nullptr, swizzle, "pointwise pair operand");
}

}  // namespace

bool pointwise_pair_tc_supported(Pass pass, int dtype, int variant, const Geom& g) {
    if (pass != PASS_FWD) return false;
    if (dtype != PCB_F16 && dtype != PCB_BF16) return false;
    if (g.nc != 4 || variant != PCB_VARIANT_16_PRODUCT || g.real_in || g.w_io || g.dw_io || !g.plain) return false;
    if (!(g.KH == 1 && g.KW == 1 && g.SH == 1 && g.SW == 1 && g.PT == 0 && g.PL == 0 && g.HO == g.H && g.WO == g.W)) return false;
    if ((g.Ci % 8) || (g.Co % 256) || ((g.H * g.W) % 8)) return false;
    if ((g.Ci + P_KS - 1) / P_KS > P_MAX_K) return false;                 // the filter rows of a CTA stay in its shared memory
    // Measured against the single-SM kernel (batch 64..128, forward, two-phase schedule): 0.165 vs 0.189 ms at 128 -> 256 channels
    // and 56 x 56; 0.112 vs 0.115 ms at 64 -> 256; 0.113 vs 0.115 ms at 64 -> 512 and 28 x 28; 3 % slower at 32 input channels, where
    // the layer is bound by HBM and the pair's common tile schedule costs more than the halved activation traffic saves.
    if (g.Ci < 64) return false;
    // enough pixel blocks to give every SM at least one
    return (long long)g.Nb * ((g.H * g.W + 63) / 64) >= (long long)sm_count();
}

int pointwise_pair_tc_launch(int dtype, const Geom& g, const void* w, const void* x, const void* bias, void* y, int* status, cudaStream_t stream) {
    const int fmt = dtype == PCB_F16 ? 0 : 1;
    const int HW = g.H * g.W;
    PParams p;
    p.Nb = g.Nb; p.HW = HW; p.fmt = fmt; p.has_bias = g.has_bias ? 1 : 0;
    p.Cout = g.Co; p.Cred = g.Ci;
    p.blocks_per_image = (HW + 63) / 64;
    p.n_px_tiles = (p.blocks_per_image * g.Nb + 1) / 2;
    p.n_cp = g.Co / (2 * P_CT);
    alignas(64) CUtensorMap map_w, map_act, map_out;
    {   // filters [4][Co][Ci]: (ci, co, r)
        const cuuint64_t dims[3] = {(cuuint64_t)g.Ci, (cuuint64_t)g.Co, 4};
        const cuuint64_t strides[2] = {(cuuint64_t)g.Ci * 2, (cuuint64_t)g.Co * g.Ci * 2};
        const cuuint32_t box[3] = {P_KS, P_CT, 4};
        const int rc = make_map_p(&map_w, fmt, w, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc != PCB_OK) return rc;
    }
    {   // x [4][Nb][Ci][HW]: (px, channel, image, component)
        const cuuint64_t dims[4] = {(cuuint64_t)HW, (cuuint64_t)g.Ci, (cuuint64_t)g.Nb, 4};
        const cuuint64_t strides[3] = {(cuuint64_t)HW * 2, (cuuint64_t)g.Ci * HW * 2, (cuuint64_t)g.Nb * g.Ci * HW * 2};
        const cuuint32_t box[4] = {64, P_KS, 1, 4};
        const int rc = make_map_p(&map_act, fmt, x, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != PCB_OK) return rc;
    }
    {   // y [4][Nb][Co][HW]; every epilogue warp stores [32 channels][64 pixels] boxes
        const cuuint64_t dims[4] = {(cuuint64_t)HW, (cuuint64_t)g.Co, (cuuint64_t)g.Nb, 4};
        const cuuint64_t strides[3] = {(cuuint64_t)HW * 2, (cuuint64_t)g.Co * HW * 2, (cuuint64_t)g.Nb * g.Co * HW * 2};
        const cuuint32_t box[4] = {64, 32, 1, 1};
        const int rc = make_map_p(&map_out, fmt, y, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != PCB_OK) return rc;
    }
    const int n_tiles = p.n_px_tiles * p.n_cp;
    int pairs = sm_count() / 2;
    if (pairs > n_tiles) pairs = n_tiles;
    pairs -= pairs % p.n_cp;                            // every pair keeps one channel pair for all its tiles
    if (pairs < p.n_cp) pairs = p.n_cp;
    PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_pointwise_pair_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P_SMEM_BYTES));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(P_THREADS, 1, 1);
    cfg.dynamicSmemBytes = P_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PCB_CUDA_TRY(cudaLaunchKernelEx(&cfg, qconv_pointwise_pair_tc_kernel, map_w, map_act, map_out, p, (const uint16_t*)bias, status));
    return PCB_OK;
}

// The pair form of the pointwise filter gradient: the caller (pointwise_tc.cu) has zeroed the fp32 scratch and casts it afterwards.
bool pointwise_filter_pair_tc_supported(const Geom& g) {
    if ((g.Co % 256) || (g.Ci % 4) || ((g.H * g.W) % 8)) return false;
    const long long steps = (long long)g.Nb * ((g.H * g.W + PF_KP - 1) / PF_KP);
    const int n_out_tiles = (g.Co / 256) * ((g.Ci + 127) / 128);
    // every pair of SMs gets a share of the pixels that is worth a pipeline
    return n_out_tiles <= sm_count() / 2 && steps >= 8ll * (sm_count() / 2 / n_out_tiles);
}

int pointwise_filter_pair_tc_launch(int fmt, const Geom& g, const void* dy, const void* x, float* scratch, int* status, cudaStream_t stream) {
    const int HW = g.H * g.W;
    PFParams p;
    p.Nb = g.Nb; p.Co = g.Co; p.Ci = g.Ci; p.HW = HW; p.fmt = fmt;
    p.blocks_per_image = (HW + PF_KP - 1) / PF_KP;
    p.n_co_pairs = g.Co / 256;
    p.n_ci_tiles = (g.Ci + 127) / 128;
    p.steps_total = g.Nb * p.blocks_per_image;
    const int n_out_tiles = p.n_co_pairs * p.n_ci_tiles;
    int splits = (sm_count() / 2) / n_out_tiles;
    if (splits < 1) splits = 1;
    if (splits > p.steps_total) splits = p.steps_total;
    p.steps_per_split = (p.steps_total + splits - 1) / splits;
    splits = (p.steps_total + p.steps_per_split - 1) / p.steps_per_split;

    alignas(64) CUtensorMap map_dy, map_x;
    {
        const cuuint64_t dims[4] = {(cuuint64_t)HW, (cuuint64_t)g.Co, (cuuint64_t)g.Nb, 4};
        const cuuint64_t strides[3] = {(cuuint64_t)HW * 2, (cuuint64_t)g.Co * HW * 2, (cuuint64_t)g.Nb * g.Co * HW * 2};
        const cuuint32_t box[4] = {PF_KP, 128, 1, 4};
        const int rc = make_map_p(&map_dy, fmt, dy, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc != PCB_OK) return rc;
    }
    {
        const cuuint64_t dims[4] = {(cuuint64_t)HW, (cuuint64_t)g.Ci, (cuuint64_t)g.Nb, 4};
        const cuuint64_t strides[3] = {(cuuint64_t)HW * 2, (cuuint64_t)g.Ci * HW * 2, (cuuint64_t)g.Nb * g.Ci * HW * 2};
        const cuuint32_t box[4] = {PF_KP, 64, 1, 4};
        const int rc = make_map_p(&map_x, fmt, x, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc != PCB_OK) return rc;
    }
    PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_pointwise_filter_pair_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM_BYTES));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * n_out_tiles * splits, 1, 1);
    cfg.blockDim = dim3(P_THREADS, 1, 1);
    cfg.dynamicSmemBytes = PF_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PCB_CUDA_TRY(cudaLaunchKernelEx(&cfg, qconv_pointwise_filter_pair_tc_kernel, map_dy, map_x, p, scratch, status));
    return PCB_OK;
}

}  // namespace pcb
