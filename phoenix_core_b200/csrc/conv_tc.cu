// General quaternion convolution on the tensor cores (tcgen05 / TMEM / TMA): any filter size, stride 1 or 2,
// any TF-style padding, any channel count; forward, backward-data and backward-filter.
//
// The reference layout (NCHW, components stacked on the batch axis) cannot feed tap-shifted TMA boxes: the
// innermost TMA coordinate must be a multiple of 16 bytes, and a filter tap shifts the pixel axis by single
// elements. So a convolution with taps first stages two small-or-cheap things in the caller's workspace:
//   * the activations, channels-last and zero-padded:  xp[comp][img][hp][wp][c16]   (pack_activations_kernel)
//   * the filters as the signed, permuted real matrix of the Hamilton product, one slab per tap:
//       Wexp[tap][(d,co)][(l,ci)] = s(l,d) * w[l^d][co][ci][tap]                    (pack_filters_kernel)
//     (reference sign table src/algebras.cc:28-49; for backward-data the transposed block with flipped taps)
// and then runs ONE implicit-GEMM kernel: D[(d,co), pixel] = sum over (tap, l, ci). With channels innermost a
// tap is a shift of the *outer* TMA coordinates (free), stride 2 is the tensor map's element stride, and
// padding is materialised zeros or TMA out-of-bounds fill. This replaces the 8/16 cuDNN calls and their
// crop / insert / accumulate kernels (src/conv2d.hpp:167-275, :433-562; src/backend/cudnn/conv2d.hpp:280-309,
// :447-488; src/backend/cudnn/kernels.cu:39-156).
//
// Kernel: persistent, one CTA per SM. Tile = 128 rows (d,co) x 256 pixels (a PW x PH x PN box of the output);
// K slice per stage = one tap, one input component, KS channels; A and B both K-major, both by TMA;
// tcgen05.mma M=128 N=256 K=16; the accumulator is double-buffered in TMEM (2 x 256 columns) so the epilogue
// (8 warps: TMEM -> bias -> cast -> NCHW stores) of tile i overlaps the main loop of tile i+1.
// All mbarrier waits are bounded.
#include "tc_common.cuh"
#include "tensor_path.cuh"

namespace pcb {
namespace {

using namespace umma;
using namespace tc;

constexpr int GM = 128, GN = 256;
constexpr int G_THREADS = 320;                       // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue
constexpr int ST_G_PRODUCER = 0x100, ST_G_MMA = 0x200, ST_G_EPILOGUE = 0x400;

struct GParams {
    int Nb, Mvalid, Cout;        // quaternion batch; valid GEMM rows (4*Cout); channels per output component
    int HO, WO;                  // output plane
    int Cp;                      // padded channels per input component (multiple of 16)
    int KH, KW, SH, SW, DH, DW;
    int PW, PH, PN;              // output tile box, PW*PH*PN == 256
    int tiles_w, tiles_h, tiles_n, tiles_m;
    int fmt, has_bias;
    int LK;                      // input components along K: 4, or 1 for a real-valued (type-0) input
    int store_vec;               // output pixels per store: largest power of two <= 16 dividing WO (and the pointer alignment)
    int n_cols;                  // columns of the tile in use (256, or 8 * PH in halo mode)
    int lw, lh;                  // log2(PW), log2(PH) (lh = -1: PH is not a power of two, and then PN == 1)
    int n_stages;                // operand stages in shared memory
    int plane_mode;              // the tile box covers whole output planes and 128 rows are 128 channels of one component:
                                 // the tile leaves through shared memory as one contiguous bulk copy per image
    // halo mode
    int Wt, Ht;
    uint32_t stage_bytes;
    int off_w, off_h;            // added to the pixel coordinates of every activation box: 0 for a staged (padded) copy, minus the
                                 // padding when the caller's channels-last tensor is read in place (the padding is TMA zero fill)
    int o_generic;               // the output is addressed through the element strides below (channels-last tensors, channel
    int o_p, o_c, o_h, o_w;      // slices of grouped layers, boxes narrower than 8 pixels): one 16-bit store per element
    int o_cl32;                  // channels-last output whose channel count is a multiple of 32: a warp transposes its 32 rows x 32
                                 // columns through shared memory and stores 16-byte runs of channels
    int bias_ld;                 // bias is [components][bias_ld]
    int exact;                   // plane mode with a tile box of exactly PN whole planes (WO x HO x PN pixels, any plane size up to
                                 // 256 pixels): the MMAs are n_cols = PN * WO * HO rounded up to 16 columns wide
    uint32_t b_tx;               // bytes one activation box brings (plain form)
};
constexpr uint32_t G_PLANE_BYTES = GM * GN * 2;      // staging buffer of the plane-mode epilogue

// K-major operand tile whose rows hold KS 16-bit elements (KS*2 bytes, swizzle span == row size):
// 8-row groups are 8*KS*2 bytes apart. KS = 64 -> 128-byte swizzle, KS = 32 -> 64-byte, KS = 16 -> 32-byte.
template <int KS>
__device__ __forceinline__ uint64_t make_desc_kmajor_rows(uint32_t smem_addr) {
    constexpr uint64_t layout = (KS == 64 ? 2ull : (KS == 32 ? 4ull : 6ull)) << 61;
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)((8 * KS * 2) >> 4) << 32) | DESC_VERSION_SM100 | layout;
}

// The same rows with the 8-row groups `group_bytes` apart: the halo tile, where a group is 8 consecutive pixels of one
// tile row and the next group is one halo-row pitch further. The swizzle is a function of the absolute shared-memory
// address (TMA writes it that way and the MMA reads it that way), so the start address may sit anywhere on a pixel.
__device__ __forceinline__ uint64_t make_desc_kmajor_sw64_groups(uint32_t smem_addr, uint32_t group_bytes) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)((group_bytes >> 4) & 0x3FFFu) << 32) | DESC_VERSION_SM100 |
           (4ull << 61);
}

// Plane-mode epilogue, one thread's 32 accumulator columns (32 >> LW rows of the tile box, PW = 1 << LW pixels each): the
// valid pixels go to the thread's channel plane in the staging buffer. The box row is decoded once per row, the pixel
// index is a compile-time constant: the epilogue warps are few (two per scheduler), so every instruction saved per
// element shortens the tile by its issue latency.
template <int LW>
__device__ __forceinline__ void plane_pack(const uint32_t (&v)[32], int col0, const GParams& p, uint16_t* mine, int HWo, float badd) {
    constexpr int PWc = 1 << LW, ROWS = 32 >> LW;
    const bool pairs = ((HWo | p.WO) & 1) == 0;          // even planes and rows: 4-byte stores of two pixels
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int jr = (col0 >> LW) + r;
        const int hl = jr & (p.PH - 1), nl = jr >> p.lh;
        if (hl >= p.HO) continue;                         // warp-uniform
        uint16_t* dst = mine + (size_t)nl * GM * HWo + hl * p.WO;
#pragma unroll
        for (int wl = 0; wl < PWc; wl += 2) {
            const float f0 = __uint_as_float(v[r * PWc + wl]) + badd, f1 = __uint_as_float(v[r * PWc + wl + 1]) + badd;
            uint32_t both;
            if (p.fmt == 0) { const __half2 h = __floats2half2_rn(f0, f1); both = *reinterpret_cast<const uint32_t*>(&h); }
            else { const __nv_bfloat162 h = __floats2bfloat162_rn(f0, f1); both = *reinterpret_cast<const uint32_t*>(&h); }
            if (pairs) {
                if (wl < p.WO) *reinterpret_cast<uint32_t*>(dst + wl) = both;
            } else {
                if (wl < p.WO) dst[wl] = (uint16_t)(both & 0xffffu);
                if (wl + 1 < p.WO) dst[wl + 1] = (uint16_t)(both >> 16);
            }
        }
    }
}

// The same for a box of exactly PN whole planes: column j is pixel j % (HO * WO) of image j / (HO * WO) of the tile, in the
// order the plane is stored, so a thread's columns are runs of consecutive elements of its channel plane.
__device__ __forceinline__ void plane_pack_exact(const uint32_t (&v)[32], int col0, const GParams& p, uint16_t* mine, int HWo, float badd) {
    int nl = col0 / HWo, pix = col0 - nl * HWo;
    const int valid = p.PN * HWo;
#pragma unroll
    for (int e = 0; e < 32; ++e) {
        if (col0 + e < valid) {
            const float f = __uint_as_float(v[e]) + badd;
            uint16_t bits;
            if (p.fmt == 0) bits = __half_as_ushort(__float2half_rn(f)); else bits = __bfloat16_as_ushort(__float2bfloat16_rn(f));
            mine[(size_t)nl * GM * HWo + pix] = bits;
        }
        if (++pix == HWo) { pix = 0; ++nl; }
    }
}

// HALO (KS == 32, stride-1 correlation, tile = 8 x PH pixels of one image): a stage is one 32-channel slice of one
// component -- the halo tile [Ht][Wt][32 channels] of the output tile and the filter slices of ALL taps -- and every
// tap's MMAs read the same halo tile at a shifted start address. Per MMA the kernel then moves 5 KB from L2 instead
// of 12 KB, which is what bounds the plain form.
template <int KS, bool HALO>
__global__ void __launch_bounds__(G_THREADS, 1)
qconv_general_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GParams p,
                        const uint16_t* __restrict__ bias, uint16_t* __restrict__ out, int* __restrict__ status) {
    constexpr uint32_t A_BYTES = GM * KS * 2, B_BYTES = GN * KS * 2;
    constexpr int MAX_STAGES = KS == 64 ? 4 : (KS == 32 ? 8 : 12);     // 192 KB of operand stages
    const uint32_t STAGE = HALO ? p.stage_bytes : A_BYTES + B_BYTES;
    const int STAGES = p.n_stages;
    const int taps = p.KH * p.KW;
    extern __shared__ uint8_t smem_raw[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + STAGES * STAGE);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 5);
    const uint32_t tiles_addr = smem_u32(base);
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + MAX_STAGES);
    const uint32_t tmem_full = smem_u32(bars + 2 * MAX_STAGES), tmem_empty = smem_u32(bars + 2 * MAX_STAGES + 2);
    const uint32_t epi_bar = smem_u32(bars + 2 * MAX_STAGES + 4);
    uint8_t* plane_buf = base + STAGES * STAGE + 512;              // plane mode only: [image][128 rows][HO * WO]

    const int tiles_px = p.tiles_w * p.tiles_h * p.tiles_n;
    const int n_tiles = tiles_px * p.tiles_m;
    const int c_steps = p.Cp / KS;
    const int n_k = (HALO ? 1 : taps) * p.LK * c_steps;           // stages per tile

    if (t == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) { mbar_init(full_bar + 8 * s, 1); mbar_init(empty_bar + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tmem_full + 8 * b, 1); mbar_init(tmem_empty + 8 * b, 8); }
        mbar_init(epi_bar, 8);
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
            int s = 0, phase = 1;                  // ring position and the parity its `empty` barrier is waited with
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int tm = tile % p.tiles_m;
                int rest = tile / p.tiles_m;
                const int tw = rest % p.tiles_w; rest /= p.tiles_w;
                const int th = rest % p.tiles_h;
                const int tn = rest / p.tiles_h;
                const int m0 = tm * GM, ow0 = tw * p.PW, oh0 = th * p.PH, n0 = tn * p.PN;
                if (HALO) {
                    for (int l = 0; l < p.LK && ok; ++l) {
                        for (int cs = 0; cs < c_steps; ++cs) {
                            ok = mbar_wait_bounded(empty_bar + 8 * s, phase, status, ST_G_PRODUCER);
                            if (!ok) break;
                            const uint32_t a_dst = tiles_addr + s * STAGE, bar = full_bar + 8 * s;
                            mbar_arrive_expect_tx(bar, taps * A_BYTES + (uint32_t)p.Wt * p.Ht * KS * 2);
                            tma_load_3d(a_dst, &map_w, l * p.Cp + cs * KS, m0, 0, bar);                       // [tap][128 rows][32 channels]
                            tma_load_5d(a_dst + taps * A_BYTES, &map_x, cs * KS, ow0 + p.off_w, oh0 + p.off_h, n0, l, bar);   // [Ht][Wt][32 channels]
                            if (++s == STAGES) { s = 0; phase ^= 1; }
                        }
                    }
                    continue;
                }
                for (int tap = 0; tap < p.KH * p.KW && ok; ++tap) {
                    const int kh = tap / p.KW, kw = tap - kh * p.KW;
                    const int wp0 = ow0 * p.SW + kw * p.DW + p.off_w, hp0 = oh0 * p.SH + kh * p.DH + p.off_h;
                    for (int l = 0; l < p.LK && ok; ++l) {
                        for (int cs = 0; cs < c_steps; ++cs) {
                            ok = mbar_wait_bounded(empty_bar + 8 * s, phase, status, ST_G_PRODUCER);
                            if (!ok) break;
                            const uint32_t a_dst = tiles_addr + s * STAGE, bar = full_bar + 8 * s;
                            mbar_arrive_expect_tx(bar, A_BYTES + p.b_tx);
                            tma_load_3d(a_dst, &map_w, l * p.Cp + cs * KS, m0, tap, bar);
                            tma_load_5d(a_dst + A_BYTES, &map_x, cs * KS, wp0, hp0, n0, l, bar);
                            if (++s == STAGES) { s = 0; phase ^= 1; }
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        // One thread runs the whole loop (waits, descriptor stepping, MMAs, commits): whatever it executes between two MMAs is
        // time the tensor pipe idles, so there is no warp synchronisation inside and a stage's two descriptors are built once
        // and stepped by adding to the address field of their low words (16-byte units, never carrying out of the field).
        if (lane == 0) {
            const uint32_t idesc = make_idesc_f16(p.fmt, GM, (HALO || p.exact) ? p.n_cols : GN, false, false);
            int s = 0, phase = 0, local_tile = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++local_tile) {
                const int buf = local_tile & 1, use = local_tile >> 1;       // use-th time this accumulator buffer is filled
                if (use > 0) {
                    ok = mbar_wait_bounded(tmem_empty + 8 * buf, (use - 1) & 1, status, ST_G_MMA);
                    if (!ok) break;
                    tc_fence_after_sync();
                }
                const uint32_t d_tmem = tmem_base + buf * GN;
                for (int k = 0; k < n_k && ok; ++k) {
                    ok = mbar_wait_bounded(full_bar + 8 * s, phase, status, ST_G_MMA);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = tiles_addr + s * STAGE, b_addr = a_addr + (HALO ? taps * A_BYTES : A_BYTES);
                    const uint64_t ad = make_desc_kmajor_rows<KS>(a_addr);
                    const uint32_t a_lo = (uint32_t)ad, a_hi = (uint32_t)(ad >> 32);
                    if (HALO) {
                        const uint64_t bd = make_desc_kmajor_sw64_groups(b_addr, p.Wt * KS * 2);
                        const uint32_t b_lo = (uint32_t)bd, b_hi = (uint32_t)(bd >> 32);
                        const uint32_t row_step = (uint32_t)(p.DH * p.Wt * KS * 2) >> 4, col_step = (uint32_t)(p.DW * KS * 2) >> 4;
                        uint32_t a_tap = a_lo, b_row = b_lo, b_tap = b_lo;
                        int kw = 0;
                        for (int tap = 0; tap < taps; ++tap) {
#pragma unroll
                            for (int j = 0; j < KS / 16; ++j)
                                mma_f16_ss_words(d_tmem, a_tap + 2 * j, a_hi, b_tap + 2 * j, b_hi, idesc, (k > 0 || tap > 0 || j > 0) ? 1u : 0u);
                            a_tap += A_BYTES >> 4;
                            if (++kw == p.KW) { kw = 0; b_row += row_step; b_tap = b_row; } else b_tap += col_step;
                        }
                    } else {
                        const uint64_t bd = make_desc_kmajor_rows<KS>(b_addr);
                        const uint32_t b_lo = (uint32_t)bd, b_hi = (uint32_t)(bd >> 32);
#pragma unroll
                        for (int j = 0; j < KS / 16; ++j)
                            mma_f16_ss_words(d_tmem, a_lo + 2 * j, a_hi, b_lo + 2 * j, b_hi, idesc, (k > 0 || j > 0) ? 1u : 0u);
                    }
                    mma_commit(empty_bar + 8 * s);
                    if (k == n_k - 1) mma_commit(tmem_full + 8 * buf);
                    if (++s == STAGES) { s = 0; phase ^= 1; }
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9)
        const int q = warp & 3;                    // TMEM lane quadrant
        const int chalf = (warp - 2) >> 2;         // which 128 of the 256 columns
        const int sv = p.store_vec;                // pixels per store instruction: 16, 8, 4, 2 or 1
        const bool vec_ok = sv >= 8;
        const bool issuer = warp == 2 && lane == 0;
        const int HWo = p.HO * p.WO;
        int local_tile = 0, epi_phase = 0;
        bool ok = true;
        // all eight warps meet; bounded like every other wait of the kernel
        auto epi_sync = [&]() {
            __syncwarp();
            if (lane == 0) mbar_arrive(epi_bar);
            const bool done = mbar_wait_bounded(epi_bar, epi_phase & 1, status, ST_G_EPILOGUE);
            ++epi_phase;
            return __all_sync(0xffffffffu, done);
        };
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++local_tile) {
            const int buf = local_tile & 1, use = local_tile >> 1;
            const int tm = tile % p.tiles_m;
            int rest = tile / p.tiles_m;
            const int tw = rest % p.tiles_w; rest /= p.tiles_w;
            const int th = rest % p.tiles_h;
            const int tn = rest / p.tiles_h;
            const int ow0 = tw * p.PW, oh0 = th * p.PH, n0 = tn * p.PN;
            const int m = tm * GM + q * 32 + lane;
            const bool row_ok = m < p.Mvalid;
            const int d = row_ok ? m / p.Cout : 0, co = m - d * p.Cout;
            float badd = 0.f;
            if (row_ok && p.has_bias) {
                const uint16_t raw = bias[d * p.bias_ld + co];
                badd = p.fmt == 0 ? __half2float(__ushort_as_half(raw)) : __bfloat162float(__ushort_as_bfloat16(raw));
            }
            ok = mbar_wait_bounded(tmem_full + 8 * buf, use & 1, status, ST_G_EPILOGUE);
            ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
            if (!ok) break;
            tc_fence_after_sync();
            if (p.plane_mode) {
                // Small planes (14 x 14, 7 x 7): a thread's 32 columns are a few short runs of its channel's plane, and
                // 32 lanes scatter them over 32 planes -- stores of 2 to 8 bytes that cost more than the tile's MMAs.
                // The valid pixels are packed [image][row][plane] in shared memory instead; the 128 rows of a tile are 128
                // consecutive channels of one component, so each image of the tile is ONE contiguous range of the output.
                if (issuer) bulk_wait_read_all();                  // the previous tile has left the staging buffer
                ok = epi_sync();
                if (!ok) break;
                uint16_t* mine = reinterpret_cast<uint16_t*>(plane_buf) + (size_t)(q * 32 + lane) * HWo;
#pragma unroll 1
                for (int cb = 0; cb < 4; ++cb) {
                    uint32_t v[32];
                    const int col0 = chalf * 128 + cb * 32;
                    tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * GN + col0, v);
                    tmem_ld_wait();
                    if (p.exact) { if (col0 < p.n_cols) plane_pack_exact(v, col0, p, mine, HWo, badd); }
                    else if (p.lw == 3) plane_pack<3>(v, col0, p, mine, HWo, badd);
                    else plane_pack<4>(v, col0, p, mine, HWo, badd);
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_empty + 8 * buf);
                fence_proxy_async_smem();
                ok = epi_sync();
                if (!ok) break;
                if (issuer) {
                    const int m0 = tm * GM, d0 = m0 / p.Cout, co0 = m0 - d0 * p.Cout;
                    for (int nl = 0; nl < p.PN; ++nl)
                        if (n0 + nl < p.Nb)
                            bulk_store_1d(out + ((size_t)(d0 * p.Nb + n0 + nl) * p.Cout + co0) * HWo,
                                          smem_u32(plane_buf) + (uint32_t)nl * GM * HWo * 2, (uint32_t)GM * HWo * 2);
                    bulk_commit_group();
                }
                continue;
            }
#pragma unroll 1
            for (int cb = 0; cb < 4; ++cb) {
                uint32_t v[32];
                const int col0 = chalf * 128 + cb * 32;
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * GN + col0, v);
                tmem_ld_wait();
                if (!row_ok) continue;
                // convert the 32 columns once, then store runs of 16 pixels (32 bytes) where a run stays inside one
                // output row and rows are 32-byte aligned, runs of 8 pixels (16 bytes) where rows are 16-byte aligned,
                // single elements otherwise
                uint32_t packed[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const float f0 = __uint_as_float(v[2 * e]) + badd, f1 = __uint_as_float(v[2 * e + 1]) + badd;
                    if (p.fmt == 0) { const __half2 h = __floats2half2_rn(f0, f1); packed[e] = *reinterpret_cast<const uint32_t*>(&h); }
                    else { const __nv_bfloat162 h = __floats2bfloat162_rn(f0, f1); packed[e] = *reinterpret_cast<const uint32_t*>(&h); }
                }
                if (p.o_cl32) {
                    // channels-last output, 32 consecutive channels per warp: the 32 x 32 block goes through 2 KB of shared memory
                    // ([pixel][32 channels]) and leaves as 16-byte stores, 64 contiguous bytes per pixel (the strided path below
                    // writes one 2-byte element per store instruction)
                    const uint32_t tbuf = smem_u32(plane_buf) + (uint32_t)(warp - 2) * 2048u;
                    __syncwarp();
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        st_shared_u16(tbuf + (2 * e) * 64 + lane * 2, (uint16_t)(packed[e] & 0xffffu));
                        st_shared_u16(tbuf + (2 * e + 1) * 64 + lane * 2, (uint16_t)(packed[e] >> 16));
                    }
                    __syncwarp();
                    const int row0 = tm * GM + q * 32, d0 = row0 / p.Cout, cch = row0 - d0 * p.Cout + (lane & 3) * 8;
#pragma unroll
                    for (int it = 0; it < 4; ++it) {
                        const int px = it * 8 + (lane >> 2), je = col0 + px;
                        if (je >= p.n_cols) continue;
                        const int wl = je & (p.PW - 1), hl = p.lh >= 0 ? ((je >> p.lw) & (p.PH - 1)) : (je >> p.lw), nl = p.lh >= 0 ? (je >> (p.lw + p.lh)) : 0;
                        const int ow = ow0 + wl, oh = oh0 + hl, img = n0 + nl;
                        if (ow >= p.WO || oh >= p.HO || img >= p.Nb) continue;
                        const uint4 val = ld_shared_v4(tbuf + px * 64 + (lane & 3) * 16);
                        *reinterpret_cast<uint4*>(out + (size_t)(d0 * p.Nb + img) * p.o_p + (size_t)oh * p.o_h + (size_t)ow * p.o_w + cch) = val;
                    }
                    continue;
                }
                const bool wide = !p.o_generic && sv >= 16 && (p.PW % 16) == 0;
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {
                    if (wide && (g8 & 1)) continue;                      // the odd groups were written with their even neighbours
                    const int j = col0 + g8 * 8;                         // column -> (image, row, pixel) of the tile box
                    if (j >= p.n_cols) continue;
                    if (p.o_generic) {
                        // Output addressed through element strides: channels-last tensors (consecutive lanes hold consecutive
                        // channels, so a warp's stores of one pixel are contiguous), channel slices of grouped layers, and boxes
                        // narrower than 8 pixels (dense layers are 1 x 1 images: the columns are batch rows). Every column is
                        // decoded on its own.
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const int je = j + e;
                            if (je >= p.n_cols) continue;
                            const int wl = je & (p.PW - 1), hl = p.lh >= 0 ? ((je >> p.lw) & (p.PH - 1)) : (je >> p.lw), nl = p.lh >= 0 ? (je >> (p.lw + p.lh)) : 0;
                            const int ow = ow0 + wl, oh = oh0 + hl, img = n0 + nl;
                            if (ow >= p.WO || oh >= p.HO || img >= p.Nb) continue;
                            out[(size_t)(d * p.Nb + img) * p.o_p + (size_t)co * p.o_c + (size_t)oh * p.o_h + (size_t)ow * p.o_w] =
                                (uint16_t)((packed[4 * g8 + (e >> 1)] >> ((e & 1) * 16)) & 0xffffu);
                        }
                        continue;
                    }
                    // PW is a power of two; PH too unless the tile is one image tall (PN == 1, halo mode)
                    const int wl = j & (p.PW - 1), hl = p.lh >= 0 ? ((j >> p.lw) & (p.PH - 1)) : (j >> p.lw), nl = p.lh >= 0 ? (j >> (p.lw + p.lh)) : 0;
                    const int ow = ow0 + wl, oh = oh0 + hl, img = n0 + nl;
                    if (ow >= p.WO || oh >= p.HO || img >= p.Nb) continue;
                    uint16_t* dst = out + (((size_t)(d * p.Nb + img) * p.Cout + co) * p.HO + oh) * p.WO + ow;
                    if (wide) {
                        st_global_v8(dst, &packed[4 * g8]);
                    } else if (vec_ok) {
                        *reinterpret_cast<uint4*>(dst) = make_uint4(packed[4 * g8], packed[4 * g8 + 1], packed[4 * g8 + 2], packed[4 * g8 + 3]);
                    } else if (sv == 4) {          // rows are 8-byte aligned: two 4-pixel stores
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                            if (ow + 4 * h < p.WO) *reinterpret_cast<uint2*>(dst + 4 * h) = make_uint2(packed[4 * g8 + 2 * h], packed[4 * g8 + 2 * h + 1]);
                    } else if (sv == 2) {          // rows are 4-byte aligned: pixel pairs
#pragma unroll
                        for (int h = 0; h < 4; ++h)
                            if (ow + 2 * h < p.WO) *reinterpret_cast<uint32_t*>(dst + 2 * h) = packed[4 * g8 + h];
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (ow + e < p.WO) dst[e] = (uint16_t)((packed[4 * g8 + (e >> 1)] >> ((e & 1) * 16)) & 0xffffu);
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty + 8 * buf);
        }
        if (issuer) bulk_wait_read_all();                           // shared memory must outlive the last bulk store's reads
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---- staging kernels ------------------------------------------------------------------------------
// xp[comp][img][hp][wp][c] = x[comp][img][c][hp - pad_top][wp - pad_left] (zero outside, zero for c >= C).
// One thread per (pixel, 8-channel group): reads are coalesced along w, writes are 16-byte vectors.
// The source is addressed through element strides (plane, channel, row, pixel), so it may be NCHW, channels-last, or a
// channel slice of a wider tensor (one group of a grouped layer).
struct SrcStrides { long long p, c, h, w; };
template <typename T>
__global__ void pack_activations_kernel(const T* __restrict__ x, T* __restrict__ xp, int planes /*4*Nb*/, int C, int H, int W,
                                        int Hp, int Wp, int Cp, int pad_top, int pad_left, int ins_h, int ins_w, int cb, int Nb, SrcStrides ss) {
    const int groups = Cp / 8;
    const unsigned total = (unsigned)planes * Hp * Wp * groups;       // 32-bit indices: the staged copy is capped at 8 GB
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        // wp fastest so that a warp reads consecutive pixels of one channel
        const int wp = (int)(idx % Wp);
        unsigned rest = idx / Wp;
        const int grp = (int)(rest % groups); rest /= groups;
        const int hp = (int)(rest % Hp);
        const int plane = (int)(rest / Hp);
        // ins_h / ins_w > 1 spread the source pixels ins apart with zeros between them (the zero-insertion that
        // turns the backward-data pass of a strided convolution into a stride-1 correlation)
        int ih = hp - pad_top, iw = wp - pad_left;
        bool inside = ih >= 0 && iw >= 0;
        if (inside && (ins_h > 1 || ins_w > 1)) {
            inside = (ih % ins_h == 0) && (iw % ins_w == 0);
            ih /= ins_h; iw /= ins_w;
        }
        inside = inside && ih < H && iw < W;
        alignas(16) T vals[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int c = grp * 8 + e;
            T v = T(0.f);
            if (c < C && inside) v = x[(long long)plane * ss.p + (long long)c * ss.c + (long long)ih * ss.h + (long long)iw * ss.w];
            vals[e] = v;
        }
        T* dst = xp + (((size_t)plane * Hp + hp) * Wp + wp) * Cp + grp * 8;
        if (cb > 0) {   // blocks of cb channels, block index outermost: xp[comp * (Cp / cb) + c / cb][img][hp][wp][cb]
            const int comp = plane / Nb, img = plane - comp * Nb, b = (grp * 8) / cb;
            dst = xp + (((((size_t)comp * (Cp / cb) + b) * Nb + img) * Hp + hp) * Wp + wp) * cb + (grp * 8 - b * cb);
        }
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(vals);
    }
}

// The general staging through shared memory for dense NCHW sources whose plane (all channels of one image and component,
// one contiguous block of C * H * W elements) fits there: the block is read once with coalesced 16-byte loads, and the
// padded / zero-inserted / channel-blocked copy is written from it with the channel groups of a pixel on neighbouring
// threads, so that a warp writes whole pixels (Cp * 2 contiguous bytes each). One CTA per plane. The general kernel above
// reads 2-byte elements H * W apart, which on 7 x 7 planes and on zero-inserted copies runs at a quarter of this.
constexpr int PACK_SMEM_THREADS = 256;
constexpr size_t PACK_SMEM_MAX_BYTES = 96 * 1024;               // two CTAs per SM
template <typename T>
__global__ void __launch_bounds__(PACK_SMEM_THREADS)
pack_activations_smem_kernel(const T* __restrict__ x, T* __restrict__ xp, int C, int H, int W, int Hp, int Wp, int Cp, int pad_top, int pad_left,
                             int ins_h, int ins_w, int cb, int Nb, int scatter) {
    extern __shared__ __align__(16) uint8_t pack_smem[];
    T* tile = reinterpret_cast<T*>(pack_smem);                   // [C][H * W]
    const int plane = blockIdx.x, HW = H * W, n = C * HW;
    const T* src = x + (size_t)plane * n;
    if ((n & 7) == 0) {                                          // every plane starts on a 16-byte boundary (the tensor does)
        for (int i = threadIdx.x; i < n / 8; i += PACK_SMEM_THREADS)
            reinterpret_cast<uint4*>(tile)[i] = __ldg(reinterpret_cast<const uint4*>(src) + i);
    } else {
        for (int i = threadIdx.x; i < n; i += PACK_SMEM_THREADS) tile[i] = src[i];
    }
    __syncthreads();
    // scatter: the copy was zeroed beforehand (zero-inserted copies are three quarters zeros) and only the source pixels are
    // visited and written to their places; otherwise every element of the copy is visited and written
    const int groups = Cp / 8, items = (scatter ? H * W : Hp * Wp) * groups;
    const int comp = plane / Nb, img = plane - comp * Nb;
    for (int idx = threadIdx.x; idx < items; idx += PACK_SMEM_THREADS) {
        const int grp = idx % groups, pix = idx / groups;
        int hp, wp, ih, iw;
        bool inside;
        if (scatter) {
            ih = pix / W; iw = pix - ih * W;
            hp = pad_top + ih * ins_h; wp = pad_left + iw * ins_w;
            if (hp < 0 || hp >= Hp || wp < 0 || wp >= Wp) continue;
            inside = true;
        } else {
            hp = pix / Wp; wp = pix - hp * Wp;
            ih = hp - pad_top; iw = wp - pad_left;
            inside = ih >= 0 && iw >= 0;
            if (inside && (ins_h > 1 || ins_w > 1)) {
                inside = (ih % ins_h == 0) && (iw % ins_w == 0);
                ih /= ins_h; iw /= ins_w;
            }
            inside = inside && ih < H && iw < W;
        }
        alignas(16) T vals[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int c = grp * 8 + e;
            vals[e] = (inside && c < C) ? tile[c * HW + ih * W + iw] : T(0.f);
        }
        T* dst = xp + (((size_t)plane * Hp + hp) * Wp + wp) * Cp + grp * 8;
        if (cb > 0) {
            const int b = (grp * 8) / cb;
            dst = xp + (((((size_t)comp * (Cp / cb) + b) * Nb + img) * Hp + hp) * Wp + wp) * cb + (grp * 8 - b * cb);
        }
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(vals);
    }
}

// Host dispatch of the activation staging: the 4- or 2-pixel form where it applies, the general form otherwise.
// cb > 0 selects the channel-block layout of the filter-gradient kernels (Nb images per component).
// `ss` = nullptr: a dense NCHW source (the fast forms apply); otherwise its element strides.
void stage_activations(int fmt, const void* src, void* dst, int planes, int C, int H, int W, int Hp, int Wp, int Cp, int pad_top, int pad_left,
                       int ins_h, int ins_w, cudaStream_t stream, int cb = 0, int Nb = 1, const SrcStrides* ss = nullptr) {
    const size_t total = (size_t)planes * Hp * Wp * (Cp / 8);
    const int px = ss ? 0 : pack_rows_px(src, W, Wp, pad_left, ins_h, ins_w);
    const SrcStrides dense = {(long long)C * H * W, (long long)H * W, (long long)W, 1};
    const SrcStrides st = ss ? *ss : dense;
    if (px == 4) {
        const int blocks = grid_cap(total / 4 + 1, 256, 16);
        if (fmt == 0) pack_rows_kernel<__half, 4><<<blocks, 256, 0, stream>>>((const __half*)src, (__half*)dst, planes, C, H, W, Hp, Wp, Cp / 8, pad_top, pad_left, 0, cb, Nb);
        else pack_rows_kernel<__nv_bfloat16, 4><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, planes, C, H, W, Hp, Wp, Cp / 8, pad_top, pad_left, 0, cb, Nb);
    } else if (px == 2) {
        const int blocks = grid_cap(total / 2 + 1, 256, 16);
        if (fmt == 0) pack_rows_kernel<__half, 2><<<blocks, 256, 0, stream>>>((const __half*)src, (__half*)dst, planes, C, H, W, Hp, Wp, Cp / 8, pad_top, pad_left, 0, cb, Nb);
        else pack_rows_kernel<__nv_bfloat16, 2><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, planes, C, H, W, Hp, Wp, Cp / 8, pad_top, pad_left, 0, cb, Nb);
    } else if (!ss && (size_t)C * H * W * 2 <= PACK_SMEM_MAX_BYTES && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
        const size_t smem = ((size_t)C * H * W * 2 + 15) / 16 * 16;
        const int scatter = (ins_h > 1 || ins_w > 1) ? 1 : 0;
        if (scatter) cudaMemsetAsync(dst, 0, (size_t)planes * Hp * Wp * Cp * 2, stream);
        if (fmt == 0) {
            cudaFuncSetAttribute(pack_activations_smem_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PACK_SMEM_MAX_BYTES);
            pack_activations_smem_kernel<__half><<<planes, PACK_SMEM_THREADS, smem, stream>>>((const __half*)src, (__half*)dst, C, H, W, Hp, Wp, Cp, pad_top, pad_left,
                                                                                           ins_h, ins_w, cb, Nb, scatter);
        } else {
            cudaFuncSetAttribute(pack_activations_smem_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PACK_SMEM_MAX_BYTES);
            pack_activations_smem_kernel<__nv_bfloat16><<<planes, PACK_SMEM_THREADS, smem, stream>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, C, H, W, Hp, Wp, Cp,
                                                                                                  pad_top, pad_left, ins_h, ins_w, cb, Nb, scatter);
        }
    } else {
        const int blocks = grid_cap(total, 256, 16);
        if (fmt == 0) pack_activations_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)src, (__half*)dst, planes, C, H, W, Hp, Wp, Cp, pad_top, pad_left, ins_h, ins_w, cb, Nb, st);
        else pack_activations_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, planes, C, H, W, Hp, Wp, Cp, pad_top, pad_left, ins_h, ins_w, cb, Nb, st);
    }
}

// Forward:       Wexp[tap][m = d*Co + co][k = l*Cp + ci]  = s(l,d) * w[l^d][co][ci][tap]
// Backward-data: Wexp[tap][m = l*Ci + ci][k = d*Cop + co] = s(l,d) * w[l^d][co][ci][taps-1-tap]   (flipped taps)
// The filters are addressed through element strides (component, output channel, input channel, tap row, tap column): OIHW, OHWI,
// HWIO, the input-major dense layout, or the slice of one group.
struct FilterStrides { long long r, o, i, h, w; int KW; };
template <typename T>
__global__ void pack_filters_kernel(const T* __restrict__ w, T* __restrict__ wexp, int Co, int Ci, int taps, int Mp, int Kp,
                                    int Cp /*padded channels of the reduced side*/, int transposed, int nc, int ga, unsigned long long neg,
                                    FilterStrides fs) {
    // one row (tap, m) of the expanded matrix per threadIdx.y; the row is decoded once, the threads of a row walk k
    const int Cm = transposed ? Ci : Co;     // channels on the M side
    const int Ck = transposed ? Co : Ci;     // channels on the K side
    const int rows = taps * Mp;
    for (int row = blockIdx.x * blockDim.y + threadIdx.y; row < rows; row += gridDim.x * blockDim.y) {
        const int tap = row / Mp, m = row - tap * Mp;
        const int cm_comp = m / Cm, cm = m - cm_comp * Cm;
        const int src_tap = transposed ? taps - 1 - tap : tap;
        T* dst = wexp + (size_t)row * Kp;
        for (int ck_comp = 0, k0 = 0; k0 < Kp; ++ck_comp, k0 += Cp) {
            const int d = transposed ? ck_comp : cm_comp, l = transposed ? cm_comp : ck_comp;
            const bool comp_ok = cm_comp < nc && ck_comp < nc;
            const bool negative = comp_ok && alg_negative(neg, l, d);
            // forward: w[r][co = cm][ci = ck][tap]; backward-data: w[r][co = ck][ci = cm][tap]
            const T* src = nullptr;
            const long long ck_stride = transposed ? fs.o : fs.i;
            if (comp_ok) {
                const int kh = src_tap / fs.KW, kw = src_tap - kh * fs.KW;
                src = w + (long long)alg_pair(ga, l, d) * fs.r + (long long)kh * fs.h + (long long)kw * fs.w + (long long)cm * (transposed ? fs.i : fs.o);
            }
            for (int ck = threadIdx.x; ck < Cp; ck += blockDim.x) {
                float v = 0.f;
                if (comp_ok && ck < Ck) { v = DType<T>::load(src + ck * ck_stride); if (negative) v = -v; }
                DType<T>::store(dst + k0 + ck, v);
            }
        }
    }
}

// The same matrix for filters whose (input channel, tap) run is contiguous (OIHW), tile by tile through shared memory: a block
// takes one filter component r and a 32 x 64 block of (M-side, K-side) channels with all its taps, reads it as whole runs
// (coalesced, where the row-per-thread kernel above strides by a whole output channel in the transposed case), and writes, for
// every (l, d) pair whose product component is r, 64 consecutive K columns per row. Requires taps <= PACK_TILE_MAX_TAPS and no
// padded rows beyond the last component (Mp == nc * Cm).
constexpr int PACK_TM = 32, PACK_TK = 64;   // rows (M-side channels) and K columns of a tile
constexpr int PACK_TILE_MAX_TAPS = 9;     // 37 KB of shared memory at 9 taps
// (16-bit elements are moved as raw bits; a negative coefficient flips the sign bit; every thread writes 8 consecutive K columns
// with one 16-byte store)
__global__ void __launch_bounds__(256)
pack_filters_tiled_kernel(const uint16_t* __restrict__ w, uint16_t* __restrict__ wexp, int Co, int Ci, int taps, int Mp, int Kp, int Cp, int transposed,
                          int nc, int ga, unsigned long long neg, FilterStrides fs, int tap_split) {
    extern __shared__ uint8_t pack_smem[];
    uint16_t* tile = reinterpret_cast<uint16_t*>(pack_smem);
    const int Cm = transposed ? Ci : Co, Ck = transposed ? Co : Ci;
    // small layers have few tiles: then blockIdx.z also splits the taps a block WRITES (every block still reads whole runs)
    const int ck0 = blockIdx.x * PACK_TK, cm0 = blockIdx.y * PACK_TM, r = blockIdx.z / tap_split, tpart = blockIdx.z - r * tap_split;
    const int taps_per = (taps + tap_split - 1) / tap_split, tap_beg = tpart * taps_per, tap_end = min(taps, tap_beg + taps_per);
    const int co0 = transposed ? ck0 : cm0, ci0 = transposed ? cm0 : ck0;
    const int n_co = transposed ? PACK_TK : PACK_TM, n_ci = transposed ? PACK_TM : PACK_TK;
    const int run = n_ci * taps;               // elements of the tile's input channels x all taps of one output channel
    const int pitch = run + 2;                 // an odd number of 32-bit words
    {   // load: a warp takes whole runs (one output channel each); a run is a multiple of 32 elements, so the loop unrolls into
        // independent loads
        const int e_limit = min(run, max(0, (Ci - ci0) * taps));      // elements of a run that belong to existing input channels
        const uint16_t* src = w + (long long)r * fs.r + (long long)co0 * fs.o + (long long)ci0 * fs.i;
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int co = warp; co < n_co; co += 8) {
            const uint16_t* row = src + (long long)co * fs.o;
            const int limit = co0 + co < Co ? e_limit : 0;
            uint16_t* trow = tile + co * pitch;
#pragma unroll 9
            for (int e = lane; e < run; e += 32) trow[e] = e < limit ? __ldg(row + e) : (uint16_t)0;
        }
    }
    __syncthreads();
    // write: a thread keeps its row cm and its 8 K columns for every tap and every (l, d) pair
    const int j = threadIdx.x & (PACK_TK / 8 - 1), cm = threadIdx.x >> 3;
    const int ck = ck0 + 8 * j;
    if (cm0 + cm >= Cm || ck >= Cp) return;
    const uint16_t* src0 = transposed ? tile + (8 * j) * pitch + cm * taps : tile + cm * pitch + (8 * j) * taps;
    const int step = transposed ? pitch : taps;
    uint32_t keep[4];                     // columns beyond the K-side channel count are zero
#pragma unroll
    for (int t = 0; t < 4; ++t) keep[t] = (ck + 2 * t < Ck ? 0xFFFFu : 0u) | (ck + 2 * t + 1 < Ck ? 0xFFFF0000u : 0u);
    for (int l = 0; l < nc; ++l) {
        int d = -1;
        for (int dd = 0; dd < nc; ++dd)
            if (alg_pair(ga, l, dd) == r) d = dd;
        if (d < 0) continue;
        const uint32_t flip = alg_negative(neg, l, d) ? 0x80008000u : 0u;
        const int m_comp = transposed ? l : d, k_comp = transposed ? d : l;
        uint16_t* dst = wexp + ((size_t)m_comp * Cm + cm0 + cm) * Kp + (size_t)k_comp * Cp + ck;
        for (int tap = tap_beg; tap < tap_end; ++tap) {
            const uint16_t* src = src0 + (transposed ? taps - 1 - tap : tap);
            uint32_t q[4];
#pragma unroll
            for (int t = 0; t < 4; ++t)
                q[t] = (((uint32_t)src[(2 * t) * step] | ((uint32_t)src[(2 * t + 1) * step] << 16)) ^ flip) & keep[t];
            *reinterpret_cast<uint4*>(dst + (size_t)tap * Mp * Kp) = make_uint4(q[0], q[1], q[2], q[3]);
        }
    }
}

template <typename T>
void pack_filters(const T* w, T* wexp, int Co, int Ci, int taps, int Mp, int Kp, int Cp, int transposed, int nc, int ga, unsigned long long neg,
                  const FilterStrides& fs, cudaStream_t stream) {
    const int Cm = transposed ? Ci : Co;
    const bool runs = fs.w == 1 && fs.h == fs.KW && fs.i == taps;
    if (runs && taps <= PACK_TILE_MAX_TAPS && Mp == nc * Cm && Cm >= PACK_TM && (reinterpret_cast<uintptr_t>(wexp) & 15u) == 0) {
        const int tiles = ((Cp + PACK_TK - 1) / PACK_TK) * ((Cm + PACK_TM - 1) / PACK_TM) * nc;
        const int tap_split = tiles < sm_count() / 2 ? taps : 1;
        const dim3 grid((Cp + PACK_TK - 1) / PACK_TK, (Cm + PACK_TM - 1) / PACK_TM, nc * tap_split);
        static_assert(sizeof(T) == 2, "the tiled kernel moves 16-bit elements");
        const size_t smem = (size_t)(transposed ? PACK_TK * (PACK_TM * taps + 2) : PACK_TM * (PACK_TK * taps + 2)) * 2;
        pack_filters_tiled_kernel<<<grid, 256, smem, stream>>>(reinterpret_cast<const uint16_t*>(w), reinterpret_cast<uint16_t*>(wexp), Co, Ci, taps, Mp,
                                                              Kp, Cp, transposed, nc, ga, neg, fs, tap_split);
    } else {
        const dim3 wthreads(Cp >= 64 ? 64 : 32, Cp >= 64 ? 4 : 8);
        const int wblocks = grid_cap((size_t)taps * Mp, (int)wthreads.y, 32);
        pack_filters_kernel<T><<<wblocks, wthreads, 0, stream>>>(w, wexp, Co, Ci, taps, Mp, Kp, Cp, transposed, nc, ga, neg, fs);
    }
}

// ===================================================================================================
// General backward-filter. Both operands come from channels-last staged copies (dy unpadded, x padded as for
// the forward pass) and are MN-major: K = output pixels, M = (d, co), N = (l, ci). One work item = one
// filter tap, one 128-row M tile, one <=256-column N tile and one slice of the pixels; its accumulator is
// the real-valued gradient block G[(d,co),(l,ci)] which the epilogue folds through the quaternion table,
//   dw[l^d][co][ci][tap] += s(l,d) * G[(d,co),(l,ci)],
// into an fp32 scratch laid out [tap][r][co][ci] with vector reductions; a last kernel transposes and casts.
// (replaces the 8/16 cudnnConvolutionBackwardFilter calls and accumulate passes of src/conv2d.hpp:433-562.)
// ===================================================================================================
constexpr int FK = 64;                               // pixels per stage
constexpr int F_STAGES = 4;
constexpr uint32_t F_STAGE = (GM + GN) * FK * 2;     // 48 KB
constexpr size_t FG_SMEM = 1024 + F_STAGES * F_STAGE + 512;

struct FGParams {
    int Nb, Co, Ci, HO, WO;
    int Cop, Cip;                 // padded channels per component of dy / x
    int cbA, cbB;                 // channel-block width (elements) of the two operands: 64, 32 or 16
    int KH, KW, SH, SW, DH, DW;
    int PW, PH, PN;               // pixel box per stage, PW*PH*PN == FK
    int tiles_w, tiles_h, tiles_n;
    int m_tiles, n_tiles, n_tile_cols;   // N columns per tile (multiple of 16, <= 256)
    int splits, steps_per_split;
    int fmt;
    int LK;                       // components of x (1 for a real-valued input)
    int TPG;                      // x-major variant: taps stacked along M per work item
    int nc, ga;                   // algebra: components, GA(3,0,0) component order
    unsigned long long neg;       // negative entries of the block, bit (8*l + d)
    int off_w, off_h;             // added to the pixel coordinates of every x box: 0 for the staged (padded) copy, minus the padding
                                  // when the caller's channels-last x is read in place
};

__device__ __forceinline__ uint64_t make_desc_mn_blocks(uint32_t smem_addr, int cb, uint32_t block_bytes) {
    // MN-major tile made of blocks of `cb` elements: K-rows of cb*2 bytes, 8-row groups contiguous.
    const uint64_t layout = cb == 64 ? 2ull : (cb == 32 ? 4ull : 6ull);
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)((block_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)(((8u * cb * 2u) >> 4) & 0x3FFFu) << 32) | DESC_VERSION_SM100 | (layout << 61);
}

__global__ void __launch_bounds__(G_THREADS, 1)
qconv_filter_general_tc_kernel(const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_x, FGParams p,
                               float* __restrict__ dw32, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + F_STAGES * F_STAGE);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * F_STAGES + 1);
    const uint32_t tiles_addr = smem_u32(base);
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + F_STAGES), tmem_full = smem_u32(bars + 2 * F_STAGES);

    // work item of this CTA
    // items (tap, tiles) vary fastest so that the CTAs running at the same time read the same pixel slice (L2 reuse)
    const int n_items = p.m_tiles * p.n_tiles * p.KH * p.KW;
    int item = blockIdx.x % n_items;
    const int split = blockIdx.x / n_items;
    const int mt = item % p.m_tiles; item /= p.m_tiles;
    const int nt = item % p.n_tiles;
    const int tap = item / p.n_tiles;
    const int kh = tap / p.KW, kw = tap - kh * p.KW;
    const int steps_total = p.tiles_w * p.tiles_h * p.tiles_n;
    const int step_beg = split * p.steps_per_split;
    const int n_steps = max(0, min(steps_total, step_beg + p.steps_per_split) - step_beg);

    const int nblkA = GM / p.cbA, nblkB = p.n_tile_cols / p.cbB;
    const int bpcA = p.Cop / p.cbA, bpcB = p.Cip / p.cbB;               // channel blocks per component
    const uint32_t blkA_bytes = FK * p.cbA * 2, blkB_bytes = FK * p.cbB * 2;
    const uint32_t a_bytes = nblkA * blkA_bytes, b_bytes = nblkB * blkB_bytes;
    const int blockA0 = mt * nblkA, blockB0 = nt * (GN / p.cbB);

    if (t == 0) {
        for (int s = 0; s < F_STAGES; ++s) { mbar_init(full_bar + 8 * s, 1); mbar_init(empty_bar + 8 * s, 1); }
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
            // one copy per operand and stage (the staged tensors keep the channel-block index outermost, so the blocks of
            // a tile are one box even across components), and a running (tw, th, tn) of the pixel box: the thread that
            // issues the copies runs no division in this loop -- at a few hundred cycles per copy it used to bound the kernel
            int tw = step_beg % p.tiles_w, th = (step_beg / p.tiles_w) % p.tiles_h, tn = step_beg / (p.tiles_w * p.tiles_h);
            int s = 0, phase = 1;
            bool ok = true;
            for (int it = 0; it < n_steps && ok; ++it) {
                ok = mbar_wait_bounded(empty_bar + 8 * s, phase, status, ST_G_PRODUCER);
                if (!ok) break;
                const int ow0 = tw * p.PW, oh0 = th * p.PH, n0 = tn * p.PN;
                const uint32_t a_dst = tiles_addr + s * F_STAGE, b_dst = a_dst + GM * FK * 2, bar = full_bar + 8 * s;
                if (++tw == p.tiles_w) { tw = 0; if (++th == p.tiles_h) { th = 0; ++tn; } }
                if (++s == F_STAGES) { s = 0; phase ^= 1; }
                mbar_arrive_expect_tx(bar, a_bytes + b_bytes);
                tma_load_5d(a_dst, &map_dy, 0, ow0, oh0, n0, blockA0, bar);
                tma_load_5d(b_dst, &map_x, 0, ow0 * p.SW + kw * p.DW + p.off_w, oh0 * p.SH + kh * p.DH + p.off_h, n0, blockB0, bar);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        const uint32_t idesc = make_idesc_f16(p.fmt, GM, p.n_tile_cols, true, true);
        bool ok = true;
        for (int it = 0; it < n_steps && ok; ++it) {
            const int s = it % F_STAGES;
            ok = mbar_wait_bounded(full_bar + 8 * s, (it / F_STAGES) & 1, status, ST_G_MMA);
            if (!ok) break;
            tc_fence_after_sync();
            if (lane == 0) {
                const uint32_t a_addr = tiles_addr + s * F_STAGE, b_addr = a_addr + GM * FK * 2;
                // consecutive MMAs alternate between two accumulators (summed by the epilogue): back-to-back MMAs into one
                // accumulator run at about two thirds of the rate of independent ones
#pragma unroll
                for (int j = 0; j < FK / 16; ++j)
                    mma_f16_ss(tmem_base + (j & 1) * GN, make_desc_mn_blocks(a_addr + j * 16 * p.cbA * 2, p.cbA, blkA_bytes),
                               make_desc_mn_blocks(b_addr + j * 16 * p.cbB * 2, p.cbB, blkB_bytes), idesc, (it > 0 || j > 1) ? 1u : 0u);
                mma_commit(empty_bar + 8 * s);
                if (it == n_steps - 1) mma_commit(tmem_full);
            }
            __syncwarp();
        }
        if (n_steps == 0 && lane == 0) mbar_arrive(tmem_full);
        __syncwarp();
    } else {
        const int q = warp & 3, chalf = (warp - 2) >> 2;
        bool ok = mbar_wait_bounded(tmem_full, 0, status, ST_G_EPILOGUE);
        ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
        tc_fence_after_sync();
        if (ok && n_steps > 0) {
            // row of the tile -> (output component d, channel co)
            const int row = q * 32 + lane;
            const int blk = blockA0 + row / p.cbA;
            const int d = blk / bpcA, co = (blk % bpcA) * p.cbA + row % p.cbA;
            const bool row_ok = d < p.nc && co < p.Co;
            const size_t comp_stride = (size_t)p.Co * p.Ci;
            float* tap_base = dw32 + (size_t)tap * p.nc * comp_stride;
#pragma unroll 1
            for (int cb = 0; cb < 4; ++cb) {
                const int col0 = chalf * 128 + cb * 32;
                if (col0 >= p.n_tile_cols) break;                         // warp-uniform
                uint32_t v[32], u[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + col0, v);
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + GN + col0, u);
                tmem_ld_wait();
                if (!row_ok) continue;
#pragma unroll
                for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) + __uint_as_float(u[e]));
#pragma unroll
                for (int g4 = 0; g4 < 8; ++g4) {
                    const int col = col0 + g4 * 4;                        // 4 consecutive columns share (l, channel block)
                    if (col >= p.n_tile_cols) continue;
                    const int nblk = blockB0 + col / p.cbB;
                    const int l = nblk / bpcB, ci = (nblk % bpcB) * p.cbB + col % p.cbB;
                    if (l >= p.LK || ci >= p.Ci) continue;
                    const float sgn = alg_negative(p.neg, l, d) ? -1.f : 1.f;
                    float* dst = tap_base + (size_t)alg_pair(p.ga, l, d) * comp_stride + (size_t)co * p.Ci + ci;
                    if ((p.Ci & 3) == 0) {
                        red_add_f32x4(dst, sgn * __uint_as_float(v[4 * g4]), sgn * __uint_as_float(v[4 * g4 + 1]),
                                      sgn * __uint_as_float(v[4 * g4 + 2]), sgn * __uint_as_float(v[4 * g4 + 3]));
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (ci + e < p.Ci) atomicAdd(dst + e, sgn * __uint_as_float(v[4 * g4 + e]));
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------------------------------
// Backward-filter for narrow layers, "x-major": the M side is the *input* with several filter taps stacked
// (rows = (tap, l, ci), one tap-shifted TMA box per tap), the N side is dy (columns = (d, co)). One dy tile
// then serves up to 8 taps instead of being re-read for every tap, which is what bounds the layers with 16
// or 32 quaternion channels and the 49-tap stem. Used when 4*Cop <= 256 and one x box per tap fits in M.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(G_THREADS, 1)
qconv_filter_xmajor_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_dy, FGParams p,
                              float* __restrict__ dw32, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + F_STAGES * F_STAGE);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * F_STAGES + 1);
    const uint32_t tiles_addr = smem_u32(base);
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + F_STAGES), tmem_full = smem_u32(bars + 2 * F_STAGES);

    const int taps = p.KH * p.KW;
    const int n_groups = (taps + p.TPG - 1) / p.TPG;
    const int tg = blockIdx.x % n_groups, split = blockIdx.x / n_groups;
    const int steps_total = p.tiles_w * p.tiles_h * p.tiles_n;
    const int step_beg = split * p.steps_per_split;
    const int n_steps = max(0, min(steps_total, step_beg + p.steps_per_split) - step_beg);
    const uint32_t tap_bytes = p.LK * FK * p.cbB * 2;          // one tap's x box: LK components of cbB channels
    const uint32_t blkX_bytes = FK * p.cbB * 2, blkY_bytes = FK * p.cbA * 2;
    const int n_cols = p.nc * p.cbA;                            // (d, co) with co padded to the channel block
    const uint32_t a_bytes = p.TPG * tap_bytes, b_bytes = p.nc * blkY_bytes;

    if (t == 0) {
        for (int s = 0; s < F_STAGES; ++s) { mbar_init(full_bar + 8 * s, 1); mbar_init(empty_bar + 8 * s, 1); }
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
            // per-tap offsets of the x boxes and the running (tw, th, tn) of the pixel box: no division in the loop
            int w_ofs[8], h_ofs[8], comp[8];
            for (int tl = 0; tl < p.TPG && tl < 8; ++tl) {
                const int tap = tg * p.TPG + tl;
                const int kh = tap / p.KW, kw = tap - kh * p.KW;
                w_ofs[tl] = kw * p.DW; h_ofs[tl] = kh * p.DH;
                comp[tl] = tap < taps ? 0 : p.LK;     // a tap past the end is loaded from component LK: entirely out of range, i.e. zeros
            }
            int tw = step_beg % p.tiles_w, th = (step_beg / p.tiles_w) % p.tiles_h, tn = step_beg / (p.tiles_w * p.tiles_h);
            int s = 0, phase = 1;
            bool ok = true;
            for (int it = 0; it < n_steps && ok; ++it) {
                ok = mbar_wait_bounded(empty_bar + 8 * s, phase, status, ST_G_PRODUCER);
                if (!ok) break;
                const int ow0 = tw * p.PW, oh0 = th * p.PH, n0 = tn * p.PN;
                const uint32_t a_dst = tiles_addr + s * F_STAGE, b_dst = a_dst + GM * FK * 2, bar = full_bar + 8 * s;
                if (++tw == p.tiles_w) { tw = 0; if (++th == p.tiles_h) { th = 0; ++tn; } }
                if (++s == F_STAGES) { s = 0; phase ^= 1; }
                mbar_arrive_expect_tx(bar, a_bytes + b_bytes);
                for (int tl = 0; tl < p.TPG; ++tl)
                    tma_load_5d(a_dst + tl * tap_bytes, &map_x, 0, ow0 * p.SW + w_ofs[tl] + p.off_w, oh0 * p.SH + h_ofs[tl] + p.off_h, n0, comp[tl], bar);
                tma_load_5d(b_dst, &map_dy, 0, ow0, oh0, n0, 0, bar);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        const uint32_t idesc = make_idesc_f16(p.fmt, GM, n_cols, true, true);
        bool ok = true;
        for (int it = 0; it < n_steps && ok; ++it) {
            const int s = it % F_STAGES;
            ok = mbar_wait_bounded(full_bar + 8 * s, (it / F_STAGES) & 1, status, ST_G_MMA);
            if (!ok) break;
            tc_fence_after_sync();
            if (lane == 0) {
                const uint32_t a_addr = tiles_addr + s * F_STAGE, b_addr = a_addr + GM * FK * 2;
#pragma unroll
                for (int j = 0; j < FK / 16; ++j)           // two accumulators in turn, as in the general kernel
                    mma_f16_ss(tmem_base + (j & 1) * GN, make_desc_mn_blocks(a_addr + j * 16 * p.cbB * 2, p.cbB, blkX_bytes),
                               make_desc_mn_blocks(b_addr + j * 16 * p.cbA * 2, p.cbA, blkY_bytes), idesc, (it > 0 || j > 1) ? 1u : 0u);
                mma_commit(empty_bar + 8 * s);
                if (it == n_steps - 1) mma_commit(tmem_full);
            }
            __syncwarp();
        }
        if (n_steps == 0 && lane == 0) mbar_arrive(tmem_full);
        __syncwarp();
    } else {
        const int q = warp & 3, chalf = (warp - 2) >> 2;
        bool ok = mbar_wait_bounded(tmem_full, 0, status, ST_G_EPILOGUE);
        ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
        tc_fence_after_sync();
        if (ok && n_steps > 0) {
            const int row = q * 32 + lane;                       // row -> (tap, input component l, channel ci)
            const int blk = row / p.cbB;
            const int tap = tg * p.TPG + blk / p.LK, l = blk % p.LK, ci = row % p.cbB;
            const bool row_ok = tap < taps && ci < p.Ci;
            const size_t comp_stride = (size_t)p.Co * p.Ci;
            float* tap_base = dw32 + (size_t)tap * p.nc * comp_stride + ci;
#pragma unroll 1
            for (int cb = 0; cb < 4; ++cb) {
                const int col0 = chalf * 128 + cb * 32;
                if (col0 >= n_cols) break;
                uint32_t v[32], u[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + col0, v);
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + GN + col0, u);
                tmem_ld_wait();
                if (!row_ok) continue;
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int col = col0 + e;
                    const int d = col / p.cbA, co = col - d * p.cbA;
                    if (col < n_cols && co < p.Co) {
                        const float val = __uint_as_float(v[e]) + __uint_as_float(u[e]);
                        atomicAdd(tap_base + (size_t)alg_pair(p.ga, l, d) * comp_stride + (size_t)co * p.Ci, alg_negative(p.neg, l, d) ? -val : val);
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// scratch [tap][r][co][ci] fp32 -> dw in the tensor type. `dense_oihw`: dw is [r][co][ci][tap] and the threads walk the
// destination (coalesced stores); otherwise the destination is addressed through the filter-gradient strides (OHWI, HWIO,
// the input-major dense gradient, the slice of one group) and the threads walk the source.
template <typename T>
__global__ void unpack_filter_grad_kernel(const float* __restrict__ src, T* __restrict__ dw, int taps, size_t per_tap, int dense_oihw,
                                          int Co, int Ci, FilterStrides ds) {
    const size_t total = per_tap * taps;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        if (dense_oihw) {
            const int tap = (int)(idx % taps);
            const size_t e = idx / taps;
            DType<T>::store(dw + idx, src[(size_t)tap * per_tap + e]);
            continue;
        }
        const int ci = (int)(idx % Ci);
        size_t rest = idx / Ci;
        const int co = (int)(rest % Co); rest /= Co;
        const size_t comps = per_tap / ((size_t)Co * Ci);
        const int r = (int)(rest % comps), tap = (int)(rest / comps);
        const int kh = tap / ds.KW, kw = tap - kh * ds.KW;
        DType<T>::store(dw + (long long)r * ds.r + (long long)co * ds.o + (long long)ci * ds.i + (long long)kh * ds.h + (long long)kw * ds.w, src[idx]);
    }
}

// Geometry of one launch of the implicit-GEMM kernel: "input" is the tensor being convolved (x forward,
// dy backward-data), "output" the tensor produced.
struct Plan {
    int Cin, Cout;                 // channels per component of the convolved / produced tensor
    int Hin, Win, Hout, Wout;
    int pad_top, pad_left;         // zero padding materialised in the staged copy
    int SH, SW;
    int ins_h, ins_w;              // zero-insertion factors of the staged copy (strided backward-data)
    int Cp, Hp, Wp, Mp, Kp;
    int LK;                        // components of the convolved tensor (1 for a real-valued input)
    int KS;
    size_t xp_bytes, w_bytes;
};

Plan make_plan(Pass pass, const Geom& g) {
    Plan pl;
    if (pass == PASS_FWD) {
        pl.Cin = g.Ci; pl.Cout = g.Co; pl.Hin = g.H; pl.Win = g.W; pl.Hout = g.HO; pl.Wout = g.WO;
        pl.pad_top = g.PT; pl.pad_left = g.PL; pl.SH = g.SH; pl.SW = g.SW; pl.ins_h = pl.ins_w = 1;
    } else {   // backward-data: stride-1 correlation of dy (zero-inserted by the stride, padded by k-1-pad) with the
               // flipped, transposed filters
        pl.Cin = g.Co; pl.Cout = g.Ci; pl.Hin = g.HO; pl.Win = g.WO; pl.Hout = g.H; pl.Wout = g.W;
        pl.pad_top = (g.KH - 1) * g.DH - g.PT; pl.pad_left = (g.KW - 1) * g.DW - g.PL; pl.SH = 1; pl.SW = 1;
        pl.ins_h = g.SH; pl.ins_w = g.SW;
    }
    pl.LK = (pass == PASS_FWD && g.real_in) ? 1 : g.nc;
    pl.Cp = round_up(pl.Cin, 16);
    pl.KS = (pl.Cp % 64 == 0) ? 64 : ((pl.Cp % 32 == 0) ? 32 : 16);   // the widest slice: a TMA copy costs about the same whatever its size
    pl.Hp = (pl.Hout - 1) * pl.SH + (g.KH - 1) * g.DH + 1;
    pl.Wp = (pl.Wout - 1) * pl.SW + (g.KW - 1) * g.DW + 1;
    pl.Mp = round_up(g.nc * pl.Cout, GM);
    pl.Kp = pl.LK * pl.Cp;
    pl.xp_bytes = ((size_t)pl.LK * g.Nb * pl.Hp * pl.Wp * pl.Cp * 2 + 1023) / 1024 * 1024;
    pl.w_bytes = ((size_t)g.KH * g.KW * pl.Mp * pl.Kp * 2 + 1023) / 1024 * 1024;
    return pl;
}

}  // namespace

bool conv_tc_supported(Pass pass, int dtype, int variant, const Geom& g) {
    if (pass != PASS_FWD && pass != PASS_BWD_DATA) return false;
    if (dtype != PCB_F16 && dtype != PCB_BF16) return false;
    if (variant != PCB_VARIANT_16_PRODUCT) return false;
    if (g.w_io && g.KH * g.KW != 1) return false;                       // input-major filters: dense layers (1x1 images, one tap)
    if (g.real_in && pass != PASS_FWD) return false;
    if (g.SH > 2 || g.SW > 2) return false;
    if (pass == PASS_BWD_DATA) {
        if ((g.KH - 1) * g.DH < g.PT || (g.KW - 1) * g.DW < g.PL) return false;
    }
    const Plan pl = make_plan(pass, g);
    if (pl.Hp > 65535 || pl.Wp > 65535) return false;
    if ((long long)pl.Wp * pl.Cp * 2 > (1ll << 31) || pl.xp_bytes > (size_t)8 << 30) return false;
    return true;
}

size_t conv_tc_scratch_bytes(Pass pass, const Geom& g) {
    const Plan pl = make_plan(pass, g);
    return pl.xp_bytes + pl.w_bytes;
}

int conv_tc_launch(Pass pass, int dtype, const Geom& g, const void* w, const void* act, const void* bias, void* out,
                   void* scratch, int* status, cudaStream_t stream) {
    EncodeTiledFn encode = encode_fn();
    if (!encode) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return PCB_ERR_CUDA; }
    const int fmt = dtype == PCB_F16 ? 0 : 1;
    const Plan pl = make_plan(pass, g);
    const int taps = g.KH * g.KW;
    uint8_t* xp = static_cast<uint8_t*>(scratch);
    uint8_t* wexp = xp + pl.xp_bytes;
    // element strides of the convolved tensor (x forward, dy backward-data) and of the produced one
    const SrcStrides sa = pass == PASS_FWD ? SrcStrides{g.xp, g.xc, g.xh, g.xw} : SrcStrides{g.yp, g.yc, g.yh, g.yw};
    const SrcStrides so = pass == PASS_FWD ? SrcStrides{g.yp, g.yc, g.yh, g.yw} : SrcStrides{g.xp, g.xc, g.xh, g.xw};
    // A channels-last tensor whose channel count is a multiple of 16 already IS the staged layout: it is read in place, the
    // padding comes from the zero fill of out-of-range TMA coordinates, and no copy of the activations is made at all.
    // (Not for zero-inserted gradients, channel slices of grouped layers, or images smaller than a tile box.)
    bool direct = !g.plain && sa.c == 1 && sa.w == pl.Cin && sa.h == (long long)pl.Win * pl.Cin && sa.p == (long long)pl.Hin * pl.Win * pl.Cin &&
                  pl.Cin % 16 == 0 && pl.ins_h == 1 && pl.ins_w == 1 && (reinterpret_cast<uintptr_t>(act) & 15u) == 0;

    // stage the operands
    {
        const size_t total = (size_t)pl.LK * g.Nb * pl.Hp * pl.Wp * (pl.Cp / 8);
        const int blocks = (int)((total + 255) / 256 < (size_t)sm_count() * 16 ? (total + 255) / 256 : (size_t)sm_count() * 16);
        (void)blocks;
        // the filter matrix is packed beside the staging pass, on the side stream (neither reads what the other writes): the
        // side stream is forked off before the staging kernel is enqueued and joined before the convolution kernel
        SideStream& ss = side_stream();
        const cudaStream_t wstream = direct ? stream : ss.fork(stream);
        if (!direct)
            stage_activations(fmt, act, xp, pl.LK * g.Nb, pl.Cin, pl.Hin, pl.Win, pl.Hp, pl.Wp, pl.Cp, pl.pad_top, pl.pad_left, pl.ins_h, pl.ins_w, stream,
                              0, 1, g.plain ? nullptr : &sa);
        const FilterStrides fs = {g.wr, g.wo, g.wi, g.wh, g.ww, g.KW};
        if (fmt == 0) {
            pack_filters<__half>((const __half*)w, (__half*)wexp, g.Co, g.Ci, taps, pl.Mp, pl.Kp, pl.Cp, pass == PASS_BWD_DATA ? 1 : 0, g.nc, g.ga, g.neg, fs,
                                 wstream);
        } else {
            pack_filters<__nv_bfloat16>((const __nv_bfloat16*)w, (__nv_bfloat16*)wexp, g.Co, g.Ci, taps, pl.Mp, pl.Kp, pl.Cp,
                                        pass == PASS_BWD_DATA ? 1 : 0, g.nc, g.ga, g.neg, fs, wstream);
        }
        ss.join(stream, wstream);
        PCB_CUDA_TRY(cudaGetLastError());
    }

    // pick the output tile box (PW x PH x PN = 256 pixels) that wastes the fewest MMA columns
    GParams p;
    {
        long long best = -1;
        // (dense layers are 1 x 1 images: their box is 1 x 1 x 256, so that the columns of a tile are batch rows and none is wasted)
        const bool dense_like = pl.Wout == 1 && pl.Hout == 1;
        for (int pw = dense_like ? 1 : 8; pw <= 128; pw *= 2)
            for (int ph = 1; ph * pw <= 256; ph *= 2) {
                const int pn = 256 / (pw * ph);
                if (pw * pl.SW > 256 || ph * pl.SH > 256) continue;
                const long long vol = (long long)round_up(pl.Wout, pw) * round_up(pl.Hout, ph) * round_up(g.Nb, pn);
                if (best < 0 || vol < best || (vol == best && pw > p.PW)) { best = vol; p.PW = pw; p.PH = ph; p.PN = pn; }
            }
    }
    // Planes that fit one tile box and 128-channel row tiles: take whole planes per tile even if that wastes a few more
    // columns, because the tile then leaves as bulk copies (plane mode, see the epilogue) instead of 2..8-byte stores
    // scattered over 128 planes, which saturate the store path long before the tensor pipe.
    {
        int pw = 8, ph = 1;
        while (pw < pl.Wout) pw *= 2;
        while (ph < pl.Hout) ph *= 2;
        if (pw * ph <= 256 && pl.Cout % GM == 0 && pl.Wout % 8 != 0 && !(pl.Wout == 1 && pl.Hout == 1)) { p.PW = pw; p.PH = ph; p.PN = 256 / (pw * ph); }
    }
    // Halo mode (see the kernel): stride-1 correlation, 32-channel slices, several taps, and an image tall enough for
    // tiles of 8 x PH >= 192 pixels (smaller tiles re-read the filter slices too often to gain anything).
    // channels-last output with a multiple of 32 channels and 16-byte aligned pixels: the transposing epilogue (16 KB of shared memory)
    const bool cl32 = !g.plain && so.c == 1 && pl.Cout % 32 == 0 && so.w % 8 == 0 && so.h % 8 == 0 && so.p % 8 == 0 &&
                      (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
    constexpr int CL32_BYTES = 8 * 2048;
    bool halo = false;
    p.n_cols = 256; p.Wt = p.Ht = 0; p.n_stages = 0; p.stage_bytes = 0;
    if (pl.Cp % 32 == 0 && pl.SH == 1 && pl.SW == 1 && taps >= 4 && pl.Wout >= 8) {
        const int rows = (pl.Hout + 31) / 32;
        const int ph = (((pl.Hout + rows - 1) / rows) + 1) & ~1;
        const int wt = 8 + (g.KW - 1) * g.DW, ht = ph + (g.KH - 1) * g.DH;
        const uint32_t stage = ((uint32_t)taps * GM * 32 * 2 + (uint32_t)wt * ht * 64 + 1023) / 1024 * 1024;
        const int n_stages = (int)((227 * 1024 - 1024 - 512 - (cl32 ? CL32_BYTES : 0)) / stage);
        if (ph >= 24 && wt <= 256 && ht <= 256 && taps <= 256 && n_stages >= 2) {
            halo = true;
            p.PW = 8; p.PH = ph; p.PN = 1; p.n_cols = 8 * ph; p.Wt = wt; p.Ht = ht;
            p.n_stages = n_stages > 8 ? 8 : n_stages; p.stage_bytes = stage;
        }
    }
    {
        auto log2i = [](int v) { int l = 0; while ((1 << l) < v) ++l; return (1 << l) == v ? l : -1; };
        p.lw = log2i(p.PW); p.lh = log2i(p.PH);
    }
    // plane mode (see the epilogue): whole output planes per tile, 128 rows = 128 consecutive channels of one component
    // strided output: anything but a dense NCHW tensor, and the narrow boxes of dense layers
    p.o_generic = (!g.plain || p.lw < 3) ? 1 : 0;
    p.o_cl32 = (cl32 && p.o_generic && p.lw >= 0) ? 1 : 0;
    p.o_p = (int)so.p; p.o_c = (int)so.c; p.o_h = (int)so.h; p.o_w = (int)so.w;
    p.bias_ld = g.bias_ld;
    p.off_w = direct ? -pl.pad_left : 0; p.off_h = direct ? -pl.pad_top : 0;
    p.plane_mode = (!p.o_generic && !halo && p.PW >= pl.Wout && p.PH >= pl.Hout && pl.Cout % GM == 0 && p.lh >= 0 && (p.lw == 3 || p.lw == 4) &&
                    (reinterpret_cast<uintptr_t>(out) & 15u) == 0) ? 1 : 0;
    // Planes of at most 256 pixels: the box is exactly PN whole planes (7 x 7 x 5 = 245 of 256 columns instead of 8 x 8 x 4 with
    // 49 of every 64 in use; 14 x 14 x 1 = 196 columns in MMAs 208 wide instead of 256), and the tile still leaves as one bulk
    // copy per image.
    p.exact = 0;
    if (!p.o_generic && !halo && pl.Cout % GM == 0 && pl.Hout * pl.Wout <= 256 && pl.Wout <= 256 && pl.Hout <= 256 &&
        (pl.Wout - 1) * pl.SW + 1 <= 256 && (pl.Hout - 1) * pl.SH + 1 <= 256 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
        const int HWo = pl.Hout * pl.Wout;
        int pn = 256 / HWo;
        if (pn > g.Nb) pn = g.Nb;
        // only where it puts more pixels into a tile than the power-of-two box does (measured: a 14 x 14 plane gains nothing
        // from MMAs 208 instead of 256 columns wide)
        const int pow2_valid = p.plane_mode ? HWo * p.PN : 0;
        if (pn * HWo > pow2_valid) {
            p.exact = 1; p.plane_mode = 1;
            p.PW = pl.Wout; p.PH = pl.Hout; p.PN = pn;
            p.n_cols = round_up(p.PW * p.PH * p.PN, 16);
            p.lw = p.lh = 0;
        }
    }
    p.b_tx = (uint32_t)(p.exact ? p.PW * p.PH * p.PN : GN) * (uint32_t)pl.KS * 2u;
    if (!halo) {
        const int max_stages = pl.KS == 64 ? 4 : (pl.KS == 32 ? 8 : 12);
        const int fit = (int)((227 * 1024 - 1024 - 512 - (p.plane_mode ? G_PLANE_BYTES : (p.o_cl32 ? CL32_BYTES : 0))) / ((GM + GN) * pl.KS * 2));
        p.n_stages = fit < max_stages ? fit : max_stages;
    }
    p.Nb = g.Nb; p.Cout = pl.Cout; p.Mvalid = g.nc * pl.Cout; p.HO = pl.Hout; p.WO = pl.Wout; p.Cp = pl.Cp;
    p.KH = g.KH; p.KW = g.KW; p.SH = pl.SH; p.SW = pl.SW; p.DH = g.DH; p.DW = g.DW;
    p.tiles_w = (pl.Wout + p.PW - 1) / p.PW; p.tiles_h = (pl.Hout + p.PH - 1) / p.PH; p.tiles_n = (g.Nb + p.PN - 1) / p.PN;
    p.tiles_m = pl.Mp / GM;
    p.fmt = fmt; p.has_bias = (pass == PASS_FWD && g.has_bias) ? 1 : 0;
    p.LK = pl.LK;
    p.store_vec = 1;
    while (p.store_vec < 16 && pl.Wout % (p.store_vec * 2) == 0 && (reinterpret_cast<uintptr_t>(out) % (size_t)(p.store_vec * 4)) == 0) p.store_vec *= 2;

    const CUtensorMapDataType dt = fmt == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const int ks = halo ? 32 : pl.KS;
    const CUtensorMapSwizzle sw = ks == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : (ks == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    alignas(64) CUtensorMap map_w, map_x;
    {
        const cuuint64_t dims[3] = {(cuuint64_t)pl.Kp, (cuuint64_t)pl.Mp, (cuuint64_t)taps};
        const cuuint64_t strides[2] = {(cuuint64_t)pl.Kp * 2, (cuuint64_t)pl.Mp * pl.Kp * 2};
        const cuuint32_t box[3] = {(cuuint32_t)ks, GM, (cuuint32_t)(halo ? taps : 1)};
        const cuuint32_t es[3] = {1, 1, 1};
        const CUresult r = encode(&map_w, dt, 3, wexp, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (filters) failed with code %d", (int)r); return PCB_ERR_CUDA; }
    }
    {
        // staged copy [comp][img][Hp][Wp][Cp], or the caller's channels-last tensor [comp][img][Hin][Win][Cin] read in place
        const int Wd = direct ? pl.Win : pl.Wp, Hd = direct ? pl.Hin : pl.Hp;
        const cuuint64_t dims[5] = {(cuuint64_t)pl.Cp, (cuuint64_t)Wd, (cuuint64_t)Hd, (cuuint64_t)g.Nb, (cuuint64_t)pl.LK};
        const cuuint64_t strides[4] = {(cuuint64_t)pl.Cp * 2, (cuuint64_t)Wd * pl.Cp * 2, (cuuint64_t)Hd * Wd * pl.Cp * 2,
                                       (cuuint64_t)g.Nb * Hd * Wd * pl.Cp * 2};
        // with an element stride s the box extent is given in input elements: s * (pixels - 1) + 1 of them hold the pixels loaded
        const cuuint32_t box[5] = {(cuuint32_t)ks, (cuuint32_t)(halo ? p.Wt : (p.PW - 1) * pl.SW + 1), (cuuint32_t)(halo ? p.Ht : (p.PH - 1) * pl.SH + 1),
                                   (cuuint32_t)p.PN, 1};
        const cuuint32_t es[5] = {1, (cuuint32_t)pl.SW, (cuuint32_t)pl.SH, 1, 1};
        const CUresult r = encode(&map_x, dt, 5, direct ? const_cast<void*>(act) : static_cast<void*>(xp), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (activations) failed with code %d", (int)r); return PCB_ERR_CUDA; }
    }

    const int n_tiles = p.tiles_w * p.tiles_h * p.tiles_n * p.tiles_m;
    const int grid = n_tiles < sm_count() ? n_tiles : sm_count();
    if (halo) {
        const size_t smem = 1024 + (size_t)p.n_stages * p.stage_bytes + 512 + (p.o_cl32 ? CL32_BYTES : 0);
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_general_tc_kernel<32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        qconv_general_tc_kernel<32, true><<<grid, G_THREADS, smem, stream>>>(map_w, map_x, p, (const uint16_t*)bias, (uint16_t*)out, status);
    } else if (pl.KS == 64) {
        const size_t smem = 1024 + (size_t)p.n_stages * (GM + GN) * 64 * 2 + 512 + (p.plane_mode ? G_PLANE_BYTES : (p.o_cl32 ? CL32_BYTES : 0));
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_general_tc_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        qconv_general_tc_kernel<64, false><<<grid, G_THREADS, smem, stream>>>(map_w, map_x, p, (const uint16_t*)bias, (uint16_t*)out, status);
    } else if (pl.KS == 32) {
        const size_t smem = 1024 + (size_t)p.n_stages * (GM + GN) * 32 * 2 + 512 + (p.plane_mode ? G_PLANE_BYTES : (p.o_cl32 ? CL32_BYTES : 0));
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_general_tc_kernel<32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        qconv_general_tc_kernel<32, false><<<grid, G_THREADS, smem, stream>>>(map_w, map_x, p, (const uint16_t*)bias, (uint16_t*)out, status);
    } else {
        const size_t smem = 1024 + (size_t)p.n_stages * (GM + GN) * 16 * 2 + 512 + (p.plane_mode ? G_PLANE_BYTES : (p.o_cl32 ? CL32_BYTES : 0));
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_general_tc_kernel<16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        qconv_general_tc_kernel<16, false><<<grid, G_THREADS, smem, stream>>>(map_w, map_x, p, (const uint16_t*)bias, (uint16_t*)out, status);
    }
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

namespace {
int channel_block(int cp) { return cp % 64 == 0 ? 64 : (cp % 32 == 0 ? 32 : 16); }

struct FilterPlan {
    int Cop, Cip, Hp, Wp;
    size_t xp_bytes, dyp_bytes, acc_bytes;
};

FilterPlan make_filter_plan(const Geom& g) {
    FilterPlan f;
    f.Cop = round_up(g.Co, 16);
    f.Cip = round_up(g.Ci, 16);
    f.Hp = (g.HO - 1) * g.SH + (g.KH - 1) * g.DH + 1;
    f.Wp = (g.WO - 1) * g.SW + (g.KW - 1) * g.DW + 1;
    f.xp_bytes = ((size_t)(g.real_in ? 1 : g.nc) * g.Nb * f.Hp * f.Wp * f.Cip * 2 + 1023) / 1024 * 1024;
    f.dyp_bytes = ((size_t)g.nc * g.Nb * g.HO * g.WO * f.Cop * 2 + 1023) / 1024 * 1024;
    f.acc_bytes = ((size_t)g.nc * g.Co * g.Ci * g.KH * g.KW * sizeof(float) + 1023) / 1024 * 1024;
    return f;
}
}  // namespace

namespace {
// x-major variant: one x box per tap must tile M = 128 exactly and dy's (d, co) columns must fit one MMA.
bool filter_xmajor(const Geom& g, const FilterPlan& f) {
    const int lk = g.real_in ? 1 : g.nc;
    const int cbx = channel_block(f.Cip), cby = channel_block(f.Cop);
    return f.Cip == cbx && f.Cop == cby && lk * cbx <= 64 && g.nc * cby <= 256;
}
}  // namespace

bool conv_filter_tc_supported(int dtype, int variant, const Geom& g) {
    if (dtype != PCB_F16 && dtype != PCB_BF16) return false;
    if (variant != PCB_VARIANT_16_PRODUCT) return false;
    if (g.dw_io && g.KH * g.KW != 1) return false;                      // input-major gradient: dense layers
    if (g.real_in && !filter_xmajor(g, make_filter_plan(g))) return false;
    if (g.SH > 2 || g.SW > 2) return false;
    const FilterPlan f = make_filter_plan(g);
    if (f.Hp > 65535 || f.Wp > 65535 || f.xp_bytes + f.dyp_bytes > (size_t)12 << 30) return false;
    return true;
}

size_t conv_filter_tc_scratch_bytes(const Geom& g) {
    const FilterPlan f = make_filter_plan(g);
    return f.xp_bytes + f.dyp_bytes + f.acc_bytes;
}

bool conv_filter_tc_stages_like_forward(const Geom& g) {
    const FilterPlan f = make_filter_plan(g);
    return g.plain && channel_block(f.Cip) == f.Cip && f.xp_bytes == make_plan(PASS_FWD, g).xp_bytes;
}

bool conv_tc_staged_dy_view(const Geom& g, StagedView* view, size_t* bytes) {
    if (!g.plain || g.SH != 1 || g.SW != 1) return false;       // strided layers: backward-data reads a zero-inserted copy
    const FilterPlan f = make_filter_plan(g);
    if (channel_block(f.Cop) != f.Cop) return false;            // the filter gradient would block the channels
    const Plan pl = make_plan(PASS_BWD_DATA, g);
    if (pl.Cp != f.Cop || pl.pad_top < 0 || pl.pad_left < 0) return false;
    view->Hp = pl.Hp; view->Wp = pl.Wp; view->pad_top = pl.pad_top; view->pad_left = pl.pad_left;
    *bytes = pl.xp_bytes;
    return true;
}

int conv_filter_tc_launch(int dtype, const Geom& g, const void* dy, const void* x, void* dw, void* scratch, int* status,
                          cudaStream_t stream, const void* kept_x, const StagedView* kept_dy) {
    EncodeTiledFn encode = encode_fn();
    if (!encode) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return PCB_ERR_CUDA; }
    const int fmt = dtype == PCB_F16 ? 0 : 1;
    const FilterPlan f = make_filter_plan(g);
    const int taps = g.KH * g.KW;
    // with one channel block per component the staged x is the forward pass's: a copy it kept is read in place
    uint8_t* xp = kept_x ? static_cast<uint8_t*>(const_cast<void*>(kept_x)) : static_cast<uint8_t*>(scratch);
    uint8_t* dyp = static_cast<uint8_t*>(scratch) + f.xp_bytes;
    float* acc = reinterpret_cast<float*>(dyp + f.dyp_bytes);

    // A channels-last tensor with one channel block per component (16, 32 or 64 channels) already is the staged layout
    // [component][image][h][w][channels]: it is read in place, x with its padding supplied by out-of-range TMA coordinates.
    const bool direct_x = !g.plain && g.xc == 1 && g.xw == g.Ci && g.xh == g.W * g.Ci && (long long)g.xp == (long long)g.H * g.W * g.Ci &&
                          channel_block(f.Cip) == g.Ci && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    const bool direct_dy = !g.plain && g.yc == 1 && g.yw == g.Co && g.yh == g.WO * g.Co && (long long)g.yp == (long long)g.HO * g.WO * g.Co &&
                           channel_block(f.Cop) == g.Co && (reinterpret_cast<uintptr_t>(dy) & 15u) == 0;
    {   // stage both activations channels-last
        const int lk = g.real_in ? 1 : g.nc;
        const size_t tx = (size_t)lk * g.Nb * f.Hp * f.Wp * (f.Cip / 8), ty = (size_t)g.nc * g.Nb * g.HO * g.WO * (f.Cop / 8);
        const size_t cap = (size_t)sm_count() * 16;
        const int bx = (int)((tx + 255) / 256 < cap ? (tx + 255) / 256 : cap), by = (int)((ty + 255) / 256 < cap ? (ty + 255) / 256 : cap);
        (void)bx; (void)by;
        const SrcStrides sx = {g.xp, g.xc, g.xh, g.xw}, sy = {g.yp, g.yc, g.yh, g.yw};
        if (!direct_x && !kept_x)
            stage_activations(fmt, x, xp, lk * g.Nb, g.Ci, g.H, g.W, f.Hp, f.Wp, f.Cip, g.PT, g.PL, 1, 1, stream, channel_block(f.Cip), g.Nb, g.plain ? nullptr : &sx);
        if (!direct_dy && !kept_dy)
            stage_activations(fmt, dy, dyp, g.nc * g.Nb, g.Co, g.HO, g.WO, g.HO, g.WO, f.Cop, 0, 0, 1, 1, stream, channel_block(f.Cop), g.Nb, g.plain ? nullptr : &sy);
        PCB_CUDA_TRY(cudaGetLastError());
        PCB_CUDA_TRY(cudaMemsetAsync(acc, 0, (size_t)g.nc * g.Co * g.Ci * taps * sizeof(float), stream));
    }

    FGParams p;
    p.nc = g.nc; p.ga = g.ga; p.neg = g.neg;
    p.Nb = g.Nb; p.Co = g.Co; p.Ci = g.Ci; p.HO = g.HO; p.WO = g.WO; p.Cop = f.Cop; p.Cip = f.Cip;
    p.cbA = channel_block(f.Cop); p.cbB = channel_block(f.Cip);
    p.KH = g.KH; p.KW = g.KW; p.SH = g.SH; p.SW = g.SW; p.DH = g.DH; p.DW = g.DW; p.fmt = fmt;
    {   // pixel box of FK pixels wasting the fewest K rows
        long long best = -1;
        for (int pw = 1; pw <= FK; pw *= 2)
            for (int ph = 1; ph * pw <= FK; ph *= 2) {
                const int pn = FK / (pw * ph);
                const long long vol = (long long)round_up(g.WO, pw) * round_up(g.HO, ph) * round_up(g.Nb, pn);
                if (best < 0 || vol < best || (vol == best && pw > p.PW)) { best = vol; p.PW = pw; p.PH = ph; p.PN = pn; }
            }
    }
    p.tiles_w = (g.WO + p.PW - 1) / p.PW; p.tiles_h = (g.HO + p.PH - 1) / p.PH; p.tiles_n = (g.Nb + p.PN - 1) / p.PN;
    const int m_cols = g.nc * f.Cop, n_cols = g.nc * f.Cip;
    p.m_tiles = (m_cols + GM - 1) / GM;
    p.n_tiles = (n_cols + GN - 1) / GN;
    p.n_tile_cols = n_cols < GN ? n_cols : GN;           // 4*Cip is a multiple of 64; tiles of a multi-tile problem are full or padded by zero blocks
    p.LK = g.real_in ? 1 : g.nc;
    p.off_w = direct_x ? -g.PL : 0; p.off_h = direct_x ? -g.PT : 0;
    const bool xmajor = filter_xmajor(g, f);
    p.TPG = xmajor ? GM / (p.LK * p.cbB) : 1;
    const int steps_total = p.tiles_w * p.tiles_h * p.tiles_n;
    const int items = xmajor ? (taps + p.TPG - 1) / p.TPG : taps * p.m_tiles * p.n_tiles;
    int splits = split_count(items, sm_count());
    if (splits > steps_total) splits = steps_total;
    if (splits < 1) splits = 1;
    p.steps_per_split = (steps_total + splits - 1) / splits;
    p.splits = (steps_total + p.steps_per_split - 1) / p.steps_per_split;

    const CUtensorMapDataType dt = fmt == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    auto swz = [](int cb) { return cb == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : (cb == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B); };
    alignas(64) CUtensorMap map_dy, map_x;
    // staged tensors: [component * blocks per component + channel block][image][h][w][cb channels]; the last box extent is
    // the number of channel blocks one tile takes (blocks past the end read as zeros)
    {
        const cuuint64_t dims[5] = {(cuuint64_t)p.cbA, (cuuint64_t)g.WO, (cuuint64_t)g.HO, (cuuint64_t)g.Nb, (cuuint64_t)(g.nc * (f.Cop / p.cbA))};
        cuuint64_t strides[4] = {(cuuint64_t)p.cbA * 2, (cuuint64_t)g.WO * p.cbA * 2, (cuuint64_t)g.HO * g.WO * p.cbA * 2,
                                 (cuuint64_t)g.Nb * g.HO * g.WO * p.cbA * 2};
        void* dy_base = direct_dy ? const_cast<void*>(dy) : static_cast<void*>(dyp);
        if (kept_dy) {
            // the copy backward-data staged: [d][img][Hp][Wp][Cop] with pixel (0, 0) at (pad_top, pad_left); the map covers the
            // HO x WO pixels only, so the padding is never read and pixels past the end read as zeros, as in the compact copy
            const size_t px = (size_t)f.Cop * 2, plane = (size_t)kept_dy->Hp * kept_dy->Wp * px;
            strides[0] = px; strides[1] = (cuuint64_t)kept_dy->Wp * px; strides[2] = plane; strides[3] = (cuuint64_t)g.Nb * plane;
            dy_base = static_cast<uint8_t*>(const_cast<void*>(kept_dy->base)) + ((size_t)kept_dy->pad_top * kept_dy->Wp + kept_dy->pad_left) * px;
        }
        const cuuint32_t box[5] = {(cuuint32_t)p.cbA, (cuuint32_t)p.PW, (cuuint32_t)p.PH, (cuuint32_t)p.PN, (cuuint32_t)(xmajor ? g.nc : GM / p.cbA)};
        const cuuint32_t es[5] = {1, 1, 1, 1, 1};
        const CUresult r = encode(&map_dy, dt, 5, dy_base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz(p.cbA),
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (dy) failed with code %d", (int)r); return PCB_ERR_CUDA; }
    }
    {
        const int Wd = direct_x ? g.W : f.Wp, Hd = direct_x ? g.H : f.Hp;
        const cuuint64_t dims[5] = {(cuuint64_t)p.cbB, (cuuint64_t)Wd, (cuuint64_t)Hd, (cuuint64_t)g.Nb, (cuuint64_t)(p.LK * (f.Cip / p.cbB))};
        const cuuint64_t strides[4] = {(cuuint64_t)p.cbB * 2, (cuuint64_t)Wd * p.cbB * 2, (cuuint64_t)Hd * Wd * p.cbB * 2,
                                       (cuuint64_t)g.Nb * Hd * Wd * p.cbB * 2};
        const cuuint32_t box[5] = {(cuuint32_t)p.cbB, (cuuint32_t)((p.PW - 1) * g.SW + 1), (cuuint32_t)((p.PH - 1) * g.SH + 1), (cuuint32_t)p.PN,
                                   (cuuint32_t)(xmajor ? p.LK : p.n_tile_cols / p.cbB)};
        const cuuint32_t es[5] = {1, (cuuint32_t)g.SW, (cuuint32_t)g.SH, 1, 1};
        const CUresult r = encode(&map_x, dt, 5, direct_x ? const_cast<void*>(x) : static_cast<void*>(xp), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz(p.cbB),
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (x) failed with code %d", (int)r); return PCB_ERR_CUDA; }
    }
    if (xmajor) {
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_filter_xmajor_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FG_SMEM));
        qconv_filter_xmajor_tc_kernel<<<items * p.splits, G_THREADS, FG_SMEM, stream>>>(map_x, map_dy, p, acc, status);
    } else {
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_filter_general_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FG_SMEM));
        qconv_filter_general_tc_kernel<<<items * p.splits, G_THREADS, FG_SMEM, stream>>>(map_dy, map_x, p, acc, status);
    }
    PCB_CUDA_TRY(cudaGetLastError());
    const size_t per_tap = (size_t)g.nc * g.Co * g.Ci, total = per_tap * taps;
    const int blocks = (int)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
    const FilterStrides ds = {g.dr, g.dco, g.dci, g.dkh, g.dkw, g.KW};
    const int dense_oihw = (g.dci == taps && g.dco == g.Ci * taps && (long long)g.dr == (long long)g.Co * g.Ci * taps && g.dkh == g.KW && g.dkw == 1) ? 1 : 0;
    if (fmt == 0) unpack_filter_grad_kernel<__half><<<blocks, 256, 0, stream>>>(acc, (__half*)dw, taps, per_tap, dense_oihw, g.Co, g.Ci, ds);
    else unpack_filter_grad_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(acc, (__nv_bfloat16*)dw, taps, per_tap, dense_oihw, g.Co, g.Ci, ds);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

}  // namespace pcb
