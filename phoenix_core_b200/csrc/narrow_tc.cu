// tcgen05 kernels for NARROW layers: at most 16 channels per component on the reduced side, stride-1 correlation
// (forward of a stride-1 layer, backward-data of any layer this file's geometry covers, filter gradient of a
// stride-1 layer), 16-bit tensors.
//
// Why a separate family. With 16 channels a pixel is 32 bytes, and the general implicit-GEMM kernels (conv_tc.cu)
// fetch, for every filter tap, a fresh box of such 32-byte rows: per MMA of 128 x 256 x 16 they move 12 KB from L2
// to shared memory and run at 1/7 of the tensor rate; the filter-gradient kernel fares worse. Here every pixel is
// fetched ONCE per tile and all taps read it from shared memory:
//
//   * Staged activations are "planar": xp[comp][img][plane = c / 8][hp][wp][8 channels] (zero padded as in
//     conv_tc.cu), so that pixels of one plane are 16 bytes apart. A tile of 8 x PH output pixels needs the halo
//     tile (8 + (KW-1)*DW) x (PH + (KH-1)*DH), which one TMA box brings in as [plane][row][pixel][8].
//   * That halo tile IS a tcgen05 operand in the layout without swizzle for every tap at once: 8 consecutive pixels
//     of a row are one 128-byte core matrix, the next row of the tile is one halo-row pitch further (the stride
//     offset), the second 8-channel half is one plane further (the leading offset), and tap (kh, kw) is nothing but
//     a different start address, (kh*DH*Wt + kw*DW) * 16 bytes. The same holds for the MN-major view that the filter
//     gradient needs (K = pixels).
//   * The signed/permuted filter matrix Wexp[tap][(d,co)][(l,ci)] (reference sign tables src/algebras.cc:5-145) of such
//     a layer is small (3x3 quaternion: 144 KB) and stays resident in shared memory for the life of the CTA.
//
// Replaces, for these layers, the 8/16 scalar library convolutions and accumulate passes of src/conv2d.hpp:167-275
// (forward), :433-562 (backward).
#include "tc_common.cuh"
#include "tensor_path.cuh"

namespace pcb {
namespace {

using namespace umma;
using namespace tc;

constexpr int NM = 128;                  // MMA M: (d, co) rows, padded
constexpr int N_THREADS = 320;           // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue
constexpr int NB_STAGES = 4;             // halo tiles in flight (one per input component)
constexpr uint32_t NA_BYTES = NM * 16 * 2;   // one (tap, component) slice of the filter matrix: [2 planes][128 rows][8]
constexpr int ST_N_PRODUCER = 0x10000, ST_N_MMA = 0x20000, ST_N_EPILOGUE = 0x40000;

struct NParams {
    int Nb, Mvalid, Cout, HO, WO;        // batch; valid rows (components x Cout); output plane
    int KH, KW, DH, DW;
    int PH;                              // output tile = 8 x PH pixels of one image (PH even, <= 32)
    int Wt, Ht;                          // halo tile
    int tiles_w, tiles_h;
    int LK, taps;
    int fmt, has_bias, store_vec;
    uint32_t stage_bytes;                // shared-memory pitch of one halo stage
    uint32_t plane_bytes;                // Ht * Wt * 16
};

// Operand without swizzle: core matrices of 8 rows x 16 bytes; `lead` = distance between the two 8-element halves of
// the 16 K elements (K-major) or between 8-row K groups (MN-major); `stride` = distance between 8-row groups
// (K-major) or between 8-element MN chunks (MN-major).
__device__ __forceinline__ uint64_t desc_plain(uint32_t smem_addr, uint32_t lead, uint32_t stride) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)((lead >> 4) & 0x3FFFu) << 16) | ((uint64_t)((stride >> 4) & 0x3FFFu) << 32) |
           DESC_VERSION_SM100;
}

// ===================================================================================================
// Forward / backward-data: D[(d,co), pixel] = sum over (tap, l, ci) of Wexp * x, tile 128 x (8 x PH pixels).
// ===================================================================================================
__global__ void __launch_bounds__(N_THREADS, 1)
qconv_narrow_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, NParams p,
                       const uint16_t* __restrict__ bias, uint16_t* __restrict__ out, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t a_bytes = (uint32_t)p.taps * p.LK * NA_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + a_bytes + NB_STAGES * p.stage_bytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NB_STAGES + 5);
    const uint32_t a_addr = smem_u32(base), b_addr = a_addr + a_bytes;
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + NB_STAGES);
    const uint32_t tmem_full = smem_u32(bars + 2 * NB_STAGES), tmem_empty = smem_u32(bars + 2 * NB_STAGES + 2);
    const uint32_t a_full = smem_u32(bars + 2 * NB_STAGES + 4);

    const int tiles_img = p.tiles_w * p.tiles_h;
    const int n_tiles = tiles_img * p.Nb;
    const int n_cols = 8 * p.PH;

    if (t == 0) {
        for (int s = 0; s < NB_STAGES; ++s) { mbar_init(full_bar + 8 * s, 1); mbar_init(empty_bar + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tmem_full + 8 * b, 1); mbar_init(tmem_empty + 8 * b, 8); }
        mbar_init(a_full, 1);
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0 && blockIdx.x < n_tiles) {
            mbar_arrive_expect_tx(a_full, a_bytes);
            for (int tap = 0; tap < p.taps; ++tap)
                for (int l = 0; l < p.LK; ++l)
                    tma_load_4d(a_addr + (tap * p.LK + l) * NA_BYTES, &map_w, 0, 0, 2 * l, tap, a_full);   // [2 planes][128 rows][8]
            int it = 0;
            bool ok = true;
            const uint32_t tx = (uint32_t)p.Wt * p.Ht * 32;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int img = tile / tiles_img, r = tile - img * tiles_img;
                const int th = r / p.tiles_w, tw = r - th * p.tiles_w;
                for (int l = 0; l < p.LK; ++l, ++it) {
                    const int s = it % NB_STAGES;
                    ok = mbar_wait_bounded(empty_bar + 8 * s, ((it / NB_STAGES) & 1) ^ 1, status, ST_N_PRODUCER);
                    if (!ok) break;
                    mbar_arrive_expect_tx(full_bar + 8 * s, tx);
                    tma_load_5d(b_addr + s * p.stage_bytes, &map_x, tw * 64, th * p.PH, 0, img, l, full_bar + 8 * s);   // [2 planes][Ht][Wt][8]
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        const uint32_t idesc = make_idesc_f16(p.fmt, NM, n_cols, false, false);
        int it = 0, local_tile = 0;
        bool ok = blockIdx.x >= n_tiles || mbar_wait_bounded(a_full, 0, status, ST_N_MMA);
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++local_tile) {
            const int buf = local_tile & 1, use = local_tile >> 1;
            if (use > 0) {
                ok = mbar_wait_bounded(tmem_empty + 8 * buf, (use - 1) & 1, status, ST_N_MMA);
                if (!ok) break;
                tc_fence_after_sync();
            }
            for (int l = 0; l < p.LK && ok; ++l, ++it) {
                const int s = it % NB_STAGES;
                ok = mbar_wait_bounded(full_bar + 8 * s, (it / NB_STAGES) & 1, status, ST_N_MMA);
                if (!ok) break;
                tc_fence_after_sync();
                if (lane == 0) {
                    const uint32_t b0 = b_addr + s * p.stage_bytes;
                    int kh = 0, kw = 0;
                    for (int tap = 0; tap < p.taps; ++tap) {
                        const uint32_t shift = (uint32_t)(kh * p.DH * p.Wt + kw * p.DW) * 16;
                        if (++kw == p.KW) { kw = 0; ++kh; }
                        mma_f16_ss(tmem_base + buf * 256, desc_plain(a_addr + (tap * p.LK + l) * NA_BYTES, NM * 16, 128),
                                   desc_plain(b0 + shift, p.plane_bytes, p.Wt * 16), idesc, (l > 0 || tap > 0) ? 1u : 0u);
                    }
                    mma_commit(empty_bar + 8 * s);
                    if (l == p.LK - 1) mma_commit(tmem_full + 8 * buf);
                }
                __syncwarp();
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9)
        const int q = warp & 3;                    // TMEM lane quadrant
        const int chalf = (warp - 2) >> 2;         // which 128 of the 256 columns
        const int sv = p.store_vec;                // output pixels per store: 8, 4, 2 or 1
        int local_tile = 0;
        bool ok = true;
        const int m = q * 32 + lane;
        const bool row_ok = m < p.Mvalid;
        const int d = row_ok ? m / p.Cout : 0, co = m - d * p.Cout;
        float badd = 0.f;
        if (row_ok && p.has_bias) {
            const uint16_t raw = bias[d * p.Cout + co];
            badd = p.fmt == 0 ? __half2float(__ushort_as_half(raw)) : __bfloat162float(__ushort_as_bfloat16(raw));
        }
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++local_tile) {
            const int buf = local_tile & 1, use = local_tile >> 1;
            const int img = tile / tiles_img, r = tile - img * tiles_img;
            const int th = r / p.tiles_w, tw = r - th * p.tiles_w;
            const int ow0 = tw * 8, oh0 = th * p.PH;
            ok = mbar_wait_bounded(tmem_full + 8 * buf, use & 1, status, ST_N_EPILOGUE);
            ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll 1
            for (int cb = 0; cb < 4; ++cb) {
                const int col0 = chalf * 128 + cb * 32;
                if (col0 >= n_cols) break;                               // warp-uniform
                uint32_t v[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256 + col0, v);
                tmem_ld_wait();
                if (!row_ok) continue;
                uint32_t packed[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const float f0 = __uint_as_float(v[2 * e]) + badd, f1 = __uint_as_float(v[2 * e + 1]) + badd;
                    if (p.fmt == 0) { const __half2 h = __floats2half2_rn(f0, f1); packed[e] = *reinterpret_cast<const uint32_t*>(&h); }
                    else { const __nv_bfloat162 h = __floats2bfloat162_rn(f0, f1); packed[e] = *reinterpret_cast<const uint32_t*>(&h); }
                }
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {                         // 8 columns = one row of the tile
                    const int oh = oh0 + (col0 >> 3) + g8;
                    if (col0 + g8 * 8 >= n_cols || oh >= p.HO || ow0 >= p.WO) continue;
                    uint16_t* dst = out + (((size_t)(d * p.Nb + img) * p.Cout + co) * p.HO + oh) * p.WO + ow0;
                    if (sv >= 8) {
                        *reinterpret_cast<uint4*>(dst) = make_uint4(packed[4 * g8], packed[4 * g8 + 1], packed[4 * g8 + 2], packed[4 * g8 + 3]);
                    } else if (sv == 4) {
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                            if (ow0 + 4 * h < p.WO) *reinterpret_cast<uint2*>(dst + 4 * h) = make_uint2(packed[4 * g8 + 2 * h], packed[4 * g8 + 2 * h + 1]);
                    } else if (sv == 2) {
#pragma unroll
                        for (int h = 0; h < 4; ++h)
                            if (ow0 + 2 * h < p.WO) *reinterpret_cast<uint32_t*>(dst + 2 * h) = packed[4 * g8 + h];
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (ow0 + e < p.WO) dst[e] = (uint16_t)((packed[4 * g8 + (e >> 1)] >> ((e & 1) * 16)) & 0xffffu);
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty + 8 * buf);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---- staging ----------------------------------------------------------------------------------------
// xp[plane_in = comp*Nb + img][c / 8 (`groups` planes)][hp][wp][8] = x[plane_in][c][hp - pad_top][wp - pad_left], zero outside and for
// c >= C; ins > 1 spreads the source pixels `ins` apart (the zero insertion of a strided backward-data pass).
// s2d ("space to depth", stride-2 layers with at most 4 channels): staged channel c' = (dy, dx, c) of staged pixel
// (hp, wp) is source channel c at padded position (2*hp + dy, 2*wp + dx); the stride-2 convolution of the source
// is then a stride-1 convolution of the staged tensor with ceil(K/2) taps per axis and 4*C channels.
template <typename T>
__global__ void pack_planar_kernel(const T* __restrict__ x, T* __restrict__ xp, int planes_in, int C, int H, int W, int Hp, int Wp,
                                   int groups /*8-channel planes per component*/, int pad_top, int pad_left, int ins_h, int ins_w, int s2d = 0) {
    const size_t total = (size_t)planes_in * groups * Hp * Wp;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int wp = (int)(idx % Wp);
        size_t rest = idx / Wp;
        const int hp = (int)(rest % Hp); rest /= Hp;
        const int grp = (int)(rest % groups);
        const int plane = (int)(rest / groups);
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
            if (s2d) {
                const int sub = c / C, cs = c - sub * C;                 // sub = dy * 2 + dx
                const int sh = 2 * hp + (sub >> 1) - pad_top, sw = 2 * wp + (sub & 1) - pad_left;
                if (sub < 4 && sh >= 0 && sw >= 0 && sh < H && sw < W) v = x[(((size_t)plane * C + cs) * H + sh) * W + sw];
            } else if (c < C && inside) {
                v = x[(((size_t)plane * C + c) * H + ih) * W + iw];
            }
            vals[e] = v;
        }
        *reinterpret_cast<uint4*>(xp + idx * 8) = *reinterpret_cast<const uint4*>(vals);
    }
}

// The space-to-depth copy for an even left padding and an even line length: a staged pixel's two source columns (dx = 0, 1)
// are one aligned 32-bit word, so a thread makes BOTH 8-channel planes of one staged pixel from 2 * C coalesced 4-byte loads
// (2 source lines x C channels) instead of 16 scattered 2-byte loads.
template <typename T, int C>
__global__ void pack_planar_s2d_pairs_kernel(const T* __restrict__ x, T* __restrict__ xp, int planes_in, int H, int W, int Hp, int Wp,
                                             int pad_top, int pad_left) {
    const size_t total = (size_t)planes_in * Hp * Wp;
    const size_t plane_pitch = (size_t)Hp * Wp * 8;               // elements between the two 8-channel planes
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int wp = (int)(idx % Wp);
        size_t rest = idx / Wp;
        const int hp = (int)(rest % Hp);
        const int plane = (int)(rest / Hp);
        alignas(16) T vals[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) vals[e] = T(0.f);
        const int sw = 2 * wp - pad_left;                        // even: the pair (sw, sw + 1) is one aligned word
#pragma unroll
        for (int dy = 0; dy < 2; ++dy) {
            const int sh = 2 * hp + dy - pad_top;
            if (sh < 0 || sh >= H || sw < 0 || sw >= W) continue; // W is even, so sw + 1 < W as well
#pragma unroll
            for (int cs = 0; cs < C; ++cs) {
                const uint32_t pair = __ldg(reinterpret_cast<const uint32_t*>(x + (((size_t)plane * C + cs) * H + sh) * W + sw));
                const uint16_t lo = (uint16_t)(pair & 0xffffu), hi = (uint16_t)(pair >> 16);
                vals[(dy * 2 + 0) * C + cs] = *reinterpret_cast<const T*>(&lo);       // staged channel (dy, dx, c)
                vals[(dy * 2 + 1) * C + cs] = *reinterpret_cast<const T*>(&hi);
            }
        }
        T* dst = xp + (((size_t)plane * 2) * Hp + hp) * (size_t)Wp * 8 + (size_t)wp * 8;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(vals);
        *reinterpret_cast<uint4*>(dst + plane_pitch) = *reinterpret_cast<const uint4*>(vals + 8);
    }
}

// Launches the paired-load space-to-depth copy where it applies; false if the general kernel has to run.
template <typename T>
bool launch_s2d_pairs(const void* src, void* dst, int planes_in, int C, int H, int W, int Hp, int Wp, int pad_top, int pad_left, cudaStream_t stream) {
    if (C < 1 || C > 4 || (pad_left & 1) || (W & 1) || (reinterpret_cast<uintptr_t>(src) & 3u) || (reinterpret_cast<uintptr_t>(dst) & 15u)) return false;
    const int blocks = grid_cap((size_t)planes_in * Hp * Wp, 256, 16);
    const T* x = static_cast<const T*>(src);
    T* xp = static_cast<T*>(dst);
    if (C == 1) pack_planar_s2d_pairs_kernel<T, 1><<<blocks, 256, 0, stream>>>(x, xp, planes_in, H, W, Hp, Wp, pad_top, pad_left);
    else if (C == 2) pack_planar_s2d_pairs_kernel<T, 2><<<blocks, 256, 0, stream>>>(x, xp, planes_in, H, W, Hp, Wp, pad_top, pad_left);
    else if (C == 3) pack_planar_s2d_pairs_kernel<T, 3><<<blocks, 256, 0, stream>>>(x, xp, planes_in, H, W, Hp, Wp, pad_top, pad_left);
    else pack_planar_s2d_pairs_kernel<T, 4><<<blocks, 256, 0, stream>>>(x, xp, planes_in, H, W, Hp, Wp, pad_top, pad_left);
    return true;
}

// Wexp[tap][k / 8][m][k % 8] with m = (d, co) or (l, ci), k = (l, ci) or (d, co) as in conv_tc.cu; 128 rows, K = LK * 16.
// s2d: staged tap (a, b) of staged channel c' = (dy, dx, ci) is source tap (2a + dy, 2b + dx) of channel ci (zero past the
// filter edge); `taps` counts staged taps, KH x KW is the source filter, KWe the staged filter width.
template <typename T>
__global__ void pack_filters_planar_kernel(const T* __restrict__ w, T* __restrict__ wexp, int Co, int Ci, int taps, int Kp, int transposed,
                                           int nc, int ga, unsigned long long neg, int s2d = 0, int KH = 0, int KW = 0, int KWe = 0) {
    const size_t total = (size_t)taps * NM * Kp;
    const int Cm = transposed ? Ci : Co, Ck = transposed ? Co : Ci;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int k = (int)(idx % Kp);
        const int m = (int)((idx / Kp) % NM);
        const int tap = (int)(idx / ((size_t)Kp * NM));
        const int cm_comp = m / Cm, cm = m - cm_comp * Cm;
        const int ck_comp = k / 16, ck = k - ck_comp * 16;
        float v = 0.f;
        if (s2d) {                                   // forward only: m = (d, co), k = (l, c')
            const int sub = ck / Ci, ci = ck - sub * Ci;
            const int kh = 2 * (tap / KWe) + (sub >> 1), kw = 2 * (tap % KWe) + (sub & 1);
            if (cm_comp < nc && ck_comp < nc && sub < 4 && kh < KH && kw < KW) {
                v = DType<T>::load(w + ((size_t)(alg_pair(ga, ck_comp, cm_comp) * Co + cm) * Ci + ci) * (KH * KW) + kh * KW + kw);
                if (alg_negative(neg, ck_comp, cm_comp)) v = -v;
            }
        } else if (cm_comp < nc && ck_comp < nc && ck < Ck) {
            const int d = transposed ? ck_comp : cm_comp, l = transposed ? cm_comp : ck_comp;
            const int co = transposed ? ck : cm, ci = transposed ? cm : ck;
            const int src_tap = transposed ? taps - 1 - tap : tap;
            v = DType<T>::load(w + ((size_t)(alg_pair(ga, l, d) * Co + co) * Ci + ci) * taps + src_tap);
            if (alg_negative(neg, l, d)) v = -v;
        }
        DType<T>::store(wexp + (((size_t)tap * (Kp / 8) + k / 8) * NM + m) * 8 + (k & 7), v);
    }
}

// ===================================================================================================
// Filter gradient: G_tap[(d,co), (l,ci)] = sum over pixels of dy[(d,co), pixel] * x[(l,ci), pixel + tap], then
// dw[pair(l,d)][co][ci][tap] += sign(l,d) * G_tap. Both operands MN-major (K = pixels) in the layout without swizzle:
// dy tile [d][plane][PH][8 px][8], x halo tile [l][plane][Ht][Wt][8]; 8 consecutive pixels are one core matrix, the
// next tile row is the leading offset, the next 8 channels the stride offset, a tap is a start address. One CTA owns
// a group of taps (as many accumulators of N = LK*16 columns as fit the 512 TMEM columns) and a range of pixel
// tiles; its accumulators stay in TMEM for the whole range and are folded into fp32 scratch at the end.
// M is always 128: with fewer (d, plane) chunks than 16 the upper rows multiply whatever follows the dy tile in
// shared memory and are never read back.
// Folded form (p.fold = KW > 1): an MMA costs about the same whether it is 16 or 128 columns wide, so the kw taps of one
// filter row become columns of ONE MMA. The x tensor map gets the tap as a dimension of its own with a stride of one pixel
// (16 bytes) over the same staged copy -- overlapping views -- so that one box brings the tile shifted by every kw:
// [kw][l][plane][Ht][8 px][8], planes at one uniform pitch, N = KW * LK * 16 columns, one MMA per filter row and 16 pixels.
// A real-valued x (one component) leaves a map dimension free for the filter rows as well (stride: one staged row): the
// box is then [kw][kh][plane][PH][8 px][8] without halo rows and ONE MMA of N = KH * KW * 16 columns serves every tap.
// ===================================================================================================
constexpr int NF_STAGES = 2;
constexpr int NF_MAX_GROUPS = 16;        // tap groups that can be given CTA shares of their own

struct NFParams {
    int Nb, Co, Ci, nc, ga;
    unsigned long long neg;
    int KH, KW, DH, DW;
    int PH, Wt, Ht, tiles_w, tiles_h;
    int LK, taps, taps_per_group, n_groups;
    int fold, fold_h, LKr;               // kw (and, for one-component x, kh) taps folded into the columns of one MMA (1 = none); components of x
    int y_planes;                        // 8-channel planes of dy per component
    int steps_total, steps_per_split;
    // uneven != 0: group g owns the CTAs [cta_begin[g], cta_begin[g + 1]) and walks group_steps[g] pixel tiles per CTA -- a
    // last group with fewer taps gets fewer CTAs, so that every CTA issues about the same number of MMAs
    int uneven, cta_begin[NF_MAX_GROUPS + 1], group_steps[NF_MAX_GROUPS];
    int fmt;
    uint32_t y_bytes, x_bytes, stage_bytes, plane_bytes;
};

__global__ void __launch_bounds__(N_THREADS, 1)
qconv_narrow_filter_tc_kernel(const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_x, NFParams p,
                              float* __restrict__ dw32, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // barriers first: the operand region is followed by slack that the M = 128 operand may read
    uint64_t* bars = reinterpret_cast<uint64_t*>(base);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NF_STAGES + 1);
    const uint32_t tiles_addr = smem_u32(base) + 1024;
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + NF_STAGES), tmem_full = smem_u32(bars + 2 * NF_STAGES);

    int group = blockIdx.x % p.n_groups, split = blockIdx.x / p.n_groups, steps_per_split = p.steps_per_split;
    if (p.uneven) {
        group = 0;
        while (group + 1 < p.n_groups && (int)blockIdx.x >= p.cta_begin[group + 1]) ++group;
        split = blockIdx.x - p.cta_begin[group];
        steps_per_split = p.group_steps[group];
    }
    const int tap0 = group * p.taps_per_group;
    const int n_taps = min(p.taps_per_group, p.taps - tap0);
    const int step_beg = split * steps_per_split;
    const int n_steps = max(0, min(p.steps_total, step_beg + steps_per_split) - step_beg);
    const int tiles_img = p.tiles_w * p.tiles_h;
    const int ncols = p.LK * 16;

    if (t == 0) {
        for (int s = 0; s < NF_STAGES; ++s) { mbar_init(full_bar + 8 * s, 1); mbar_init(empty_bar + 8 * s, 1); }
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
            int img = step_beg / tiles_img, th = (step_beg - img * tiles_img) / p.tiles_w, tw = step_beg - img * tiles_img - th * p.tiles_w;
            for (int it = 0; it < n_steps && ok; ++it) {
                const int s = it % NF_STAGES;
                ok = mbar_wait_bounded(empty_bar + 8 * s, ((it / NF_STAGES) & 1) ^ 1, status, ST_N_PRODUCER);
                if (!ok) break;
                const uint32_t dst = tiles_addr + s * p.stage_bytes, bar = full_bar + 8 * s;
                mbar_arrive_expect_tx(bar, p.y_bytes + p.x_bytes);
                tma_load_5d(dst, &map_dy, tw * 64, th * p.PH, 0, img, 0, bar);                 // [d][plane][PH][8 px][8]
                if (p.fold > 1) tma_load_5d(dst + p.y_bytes, &map_x, tw * 64, th * p.PH, img * 2, 0, 0, bar);   // [kw][l][plane][Ht][8][8]
                else tma_load_5d(dst + p.y_bytes, &map_x, tw * 64, th * p.PH, 0, img, 0, bar);                  // [l][plane][Ht][Wt][8]
                if (++tw == p.tiles_w) { tw = 0; if (++th == p.tiles_h) { th = 0; ++img; } }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        const uint32_t idesc = make_idesc_f16(p.fmt, NM, ncols, true, true);
        bool ok = true;
        for (int it = 0; it < n_steps && ok; ++it) {
            const int s = it % NF_STAGES;
            ok = mbar_wait_bounded(full_bar + 8 * s, (it / NF_STAGES) & 1, status, ST_N_MMA);
            if (!ok) break;
            tc_fence_after_sync();
            if (lane == 0) {
                const uint32_t y0 = tiles_addr + s * p.stage_bytes, x0 = y0 + p.y_bytes;
                int kh = tap0 / p.KW, kw = tap0 - kh * p.KW;
                for (int tl = 0; tl < n_taps; ++tl) {
                    const uint32_t shift = (uint32_t)(kh * p.DH * p.Wt + kw * p.DW) * 16;
                    if (++kw == p.KW) { kw = 0; ++kh; }
                    for (int kk = 0; kk < p.PH / 2; ++kk)               // 16 pixels = two rows of the tile per MMA
                        mma_f16_ss(tmem_base + tl * ncols, desc_plain(y0 + kk * 256, 128, p.PH * 128),
                                   desc_plain(x0 + shift + kk * 2 * p.Wt * 16, p.Wt * 16, p.plane_bytes), idesc, (it > 0 || kk > 0) ? 1u : 0u);
                }
                mma_commit(empty_bar + 8 * s);
                if (it == n_steps - 1) mma_commit(tmem_full);
            }
            __syncwarp();
        }
        if (n_steps == 0 && lane == 0) mbar_arrive(tmem_full);
        __syncwarp();
    } else {
        const int q = warp & 3, tsel = (warp - 2) >> 2;                // two warps per lane quadrant share the taps
        bool ok = mbar_wait_bounded(tmem_full, 0, status, ST_N_EPILOGUE);
        ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
        tc_fence_after_sync();
        if (ok && n_steps > 0) {
            const int m = q * 32 + lane;                                // row -> (d, plane, channel within the plane)
            const int chunk = m >> 3, d = chunk / p.y_planes, co = (chunk - d * p.y_planes) * 8 + (m & 7);
            const bool row_ok = d < p.nc && co < p.Co;
            const size_t comp_stride = (size_t)p.Co * p.Ci;
            for (int tl = tsel; tl < n_taps; tl += 2) {
                for (int c0 = 0; c0 < ncols; c0 += 16) {                // 16 columns = the channels of one input component (of one kw tap)
                    uint32_t v[16];
                    tmem_ld_32x32b_x16(tmem_base + ((uint32_t)(q * 32) << 16) + tl * ncols + c0, v);
                    tmem_ld_wait();
                    if (!row_ok) continue;
                    int kwf, l, tap;
                    if (p.fold_h > 1) { kwf = (c0 >> 4) / p.fold_h; l = 0; tap = ((c0 >> 4) - kwf * p.fold_h) * p.fold + kwf; }
                    else { kwf = (c0 >> 4) / p.LKr; l = (c0 >> 4) - kwf * p.LKr; tap = (tap0 + tl) * p.fold + kwf; }
                    float* tap_base = dw32 + (size_t)tap * p.nc * comp_stride;
                    const float sgn = alg_negative(p.neg, l, d) ? -1.f : 1.f;
                    float* dst = tap_base + (size_t)alg_pair(p.ga, l, d) * comp_stride + (size_t)co * p.Ci;
#pragma unroll
                    for (int g4 = 0; g4 < 4; ++g4) {
                        if ((p.Ci & 3) == 0) {
                            if (4 * g4 < p.Ci)
                                red_add_f32x4(dst + 4 * g4, sgn * __uint_as_float(v[4 * g4]), sgn * __uint_as_float(v[4 * g4 + 1]),
                                              sgn * __uint_as_float(v[4 * g4 + 2]), sgn * __uint_as_float(v[4 * g4 + 3]));
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (4 * g4 + e < p.Ci) atomicAdd(dst + 4 * g4 + e, sgn * __uint_as_float(v[4 * g4 + e]));
                        }
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// scratch [tap][r][co][ci] fp32 -> dw [r][co][ci][tap] in the tensor type
template <typename T>
__global__ void unpack_narrow_filter_grad_kernel(const float* __restrict__ src, T* __restrict__ dw, int taps, size_t per_tap) {
    const size_t total = per_tap * taps;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int tap = (int)(idx % taps);
        DType<T>::store(dw + idx, src[(size_t)tap * per_tap + idx / taps]);
    }
}
// s2d: scratch [staged tap][r][co][c' = (dy, dx, ci)] -> dw [r][co][ci][kh][kw]
template <typename T>
__global__ void unpack_narrow_filter_grad_s2d_kernel(const float* __restrict__ src, T* __restrict__ dw, int rows /*nc*Co*/, int Ci, int KH, int KW,
                                                     int KWe, int taps_e) {
    const size_t total = (size_t)rows * Ci * KH * KW;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int kw = (int)(idx % KW);
        size_t rest = idx / KW;
        const int kh = (int)(rest % KH); rest /= KH;
        const int ci = (int)(rest % Ci);
        const size_t row = rest / Ci;
        const int tap = (kh >> 1) * KWe + (kw >> 1), cp = ((kh & 1) * 2 + (kw & 1)) * Ci + ci;
        DType<T>::store(dw + idx, src[((size_t)tap * rows + row) * (4 * Ci) + cp]);
    }
}

// Stride-2 layers with at most 4 channels and no dilation run as stride-1 layers of a space-to-depth copy.
bool s2d_layer(const Geom& g) { return g.SH == 2 && g.SW == 2 && g.DH == 1 && g.DW == 1 && 4 * g.Ci <= 16; }

struct NPlan {
    int Cin, Cout, Hin, Win, Hout, Wout, pad_top, pad_left, ins_h, ins_w;
    int s2d, KHe, KWe, DHe, DWe;         // effective (staged) filter
    int LK, Hp, Wp, PH, Wt, Ht, tiles_w, tiles_h;
    uint32_t stage_bytes;
    size_t xp_bytes, w_bytes, smem;
};

NPlan make_nplan(Pass pass, const Geom& g) {
    NPlan pl;
    if (pass == PASS_FWD) {
        pl.Cin = g.Ci; pl.Cout = g.Co; pl.Hin = g.H; pl.Win = g.W; pl.Hout = g.HO; pl.Wout = g.WO;
        pl.pad_top = g.PT; pl.pad_left = g.PL; pl.ins_h = pl.ins_w = 1;
    } else {
        pl.Cin = g.Co; pl.Cout = g.Ci; pl.Hin = g.HO; pl.Win = g.WO; pl.Hout = g.H; pl.Wout = g.W;
        pl.pad_top = (g.KH - 1) * g.DH - g.PT; pl.pad_left = (g.KW - 1) * g.DW - g.PL;
        pl.ins_h = g.SH; pl.ins_w = g.SW;
    }
    pl.LK = (pass == PASS_FWD && g.real_in) ? 1 : g.nc;
    pl.s2d = (pass == PASS_FWD && s2d_layer(g)) ? 1 : 0;
    pl.KHe = pl.s2d ? (g.KH + 1) / 2 : g.KH; pl.KWe = pl.s2d ? (g.KW + 1) / 2 : g.KW;
    pl.DHe = pl.s2d ? 1 : g.DH; pl.DWe = pl.s2d ? 1 : g.DW;
    if (pl.s2d) pl.Cin = 4 * g.Ci;
    const int rows = (pl.Hout + 31) / 32;                      // tile rows per image, then the smallest even height that covers them
    pl.PH = (((pl.Hout + rows - 1) / rows) + 1) & ~1;
    pl.tiles_h = (pl.Hout + pl.PH - 1) / pl.PH;
    pl.tiles_w = (pl.Wout + 7) / 8;
    pl.Wt = 8 + (pl.KWe - 1) * pl.DWe;
    pl.Ht = pl.PH + (pl.KHe - 1) * pl.DHe;
    pl.Hp = pl.tiles_h * pl.PH + (pl.KHe - 1) * pl.DHe;         // staged plane covers every halo tile completely
    pl.Wp = pl.tiles_w * 8 + (pl.KWe - 1) * pl.DWe;
    pl.stage_bytes = ((uint32_t)pl.Wt * pl.Ht * 32 + 1023) / 1024 * 1024;
    pl.xp_bytes = ((size_t)pl.LK * g.Nb * 2 * pl.Hp * pl.Wp * 16 + 1023) / 1024 * 1024;
    pl.w_bytes = ((size_t)pl.KHe * pl.KWe * pl.LK * NA_BYTES + 1023) / 1024 * 1024;
    pl.smem = 1024 + (size_t)pl.KHe * pl.KWe * pl.LK * NA_BYTES + (size_t)NB_STAGES * pl.stage_bytes + 256;
    return pl;
}

}  // namespace

bool narrow_tc_supported(Pass pass, int dtype, int variant, const Geom& g) {
    if (pass != PASS_FWD && pass != PASS_BWD_DATA) return false;
    if (dtype != PCB_F16 && dtype != PCB_BF16) return false;
    if (variant != PCB_VARIANT_16_PRODUCT || g.w_io || g.dw_io) return false;
    if (g.real_in && pass != PASS_FWD) return false;
    if (g.H * g.W == 1) return false;
    if (pass == PASS_FWD && (g.SH != 1 || g.SW != 1) && !s2d_layer(g)) return false;   // backward-data is a stride-1 correlation of the zero-inserted dy
    if (pass == PASS_BWD_DATA && (g.SH > 2 || g.SW > 2)) return false;
    if (pass == PASS_BWD_DATA && ((g.KH - 1) * g.DH < g.PT || (g.KW - 1) * g.DW < g.PL)) return false;
    const NPlan pl = make_nplan(pass, g);
    if (pl.Cin > 16 || g.nc * pl.Cout > NM) return false;
    if (pl.Wt > 32 || pl.Ht > 255 || pl.smem > 226 * 1024) return false;
    if (pl.Wout < 8 || pl.Hout < 8) return false;                             // tiny images: the general kernel packs several per tile
    if (pl.xp_bytes > (size_t)8 << 30) return false;
    return true;
}

size_t narrow_tc_scratch_bytes(Pass pass, const Geom& g) {
    const NPlan pl = make_nplan(pass, g);
    return pl.xp_bytes + pl.w_bytes;
}

int narrow_tc_launch(Pass pass, int dtype, const Geom& g, const void* w, const void* act, const void* bias, void* out, void* scratch,
                     int* status, cudaStream_t stream) {
    const int fmt = dtype == PCB_F16 ? 0 : 1;
    const NPlan pl = make_nplan(pass, g);
    const int taps = pl.KHe * pl.KWe, Kp = pl.LK * 16;
    const int src_c = pl.s2d ? g.Ci : pl.Cin;            // channels of the tensor being staged
    uint8_t* xp = static_cast<uint8_t*>(scratch);
    uint8_t* wexp = xp + pl.xp_bytes;
    {
        const size_t total = (size_t)pl.LK * g.Nb * 2 * pl.Hp * pl.Wp;
        const int blocks = grid_cap(total, 256, 16), wblocks = grid_cap((size_t)taps * NM * Kp, 256, 8);
        const bool fast = !pl.s2d && pack_rows_px(act, pl.Win, pl.Wp, pl.pad_left, pl.ins_h, pl.ins_w) == 4;
        const int fblocks = grid_cap(total / 4 + 1, 256, 16);
        // the filter matrix is packed beside the staging pass, on the side stream (neither reads what the other writes): the
        // side stream is forked off before the staging kernel is enqueued and joined before the convolution kernel
        SideStream& ss = side_stream();
        const cudaStream_t wstream = ss.fork(stream);
        if (fast && fmt == 0) {
            pack_rows_kernel<__half, 4><<<fblocks, 256, 0, stream>>>((const __half*)act, (__half*)xp, pl.LK * g.Nb, src_c, pl.Hin, pl.Win, pl.Hp, pl.Wp, 2,
                                                                  pl.pad_top, pl.pad_left, 1);
        } else if (fast) {
            pack_rows_kernel<__nv_bfloat16, 4><<<fblocks, 256, 0, stream>>>((const __nv_bfloat16*)act, (__nv_bfloat16*)xp, pl.LK * g.Nb, src_c, pl.Hin, pl.Win,
                                                                         pl.Hp, pl.Wp, 2, pl.pad_top, pl.pad_left, 1);
        } else if (pl.s2d && (fmt == 0 ? launch_s2d_pairs<__half>(act, xp, pl.LK * g.Nb, src_c, pl.Hin, pl.Win, pl.Hp, pl.Wp, pl.pad_top, pl.pad_left, stream)
                                       : launch_s2d_pairs<__nv_bfloat16>(act, xp, pl.LK * g.Nb, src_c, pl.Hin, pl.Win, pl.Hp, pl.Wp, pl.pad_top, pl.pad_left, stream))) {
            // space-to-depth copy from aligned source pairs
        } else if (fmt == 0) {
            pack_planar_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)act, (__half*)xp, pl.LK * g.Nb, src_c, pl.Hin, pl.Win, pl.Hp, pl.Wp,
                                                                  2, pl.pad_top, pl.pad_left, pl.ins_h, pl.ins_w, pl.s2d);
        } else {
            pack_planar_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)act, (__nv_bfloat16*)xp, pl.LK * g.Nb, src_c, pl.Hin,
                                                                         pl.Win, pl.Hp, pl.Wp, 2, pl.pad_top, pl.pad_left, pl.ins_h, pl.ins_w, pl.s2d);
        }
        if (fmt == 0) pack_filters_planar_kernel<__half><<<wblocks, 256, 0, wstream>>>((const __half*)w, (__half*)wexp, g.Co, g.Ci, taps, Kp,
                                                                                       pass == PASS_BWD_DATA ? 1 : 0, g.nc, g.ga, g.neg, pl.s2d, g.KH, g.KW, pl.KWe);
        else pack_filters_planar_kernel<__nv_bfloat16><<<wblocks, 256, 0, wstream>>>((const __nv_bfloat16*)w, (__nv_bfloat16*)wexp, g.Co, g.Ci, taps, Kp,
                                                                                     pass == PASS_BWD_DATA ? 1 : 0, g.nc, g.ga, g.neg, pl.s2d, g.KH, g.KW, pl.KWe);
        ss.join(stream, wstream);
        PCB_CUDA_TRY(cudaGetLastError());
    }
    NParams p;
    p.Nb = g.Nb; p.Cout = pl.Cout; p.Mvalid = g.nc * pl.Cout; p.HO = pl.Hout; p.WO = pl.Wout;
    p.KH = pl.KHe; p.KW = pl.KWe; p.DH = pl.DHe; p.DW = pl.DWe;
    p.PH = pl.PH; p.Wt = pl.Wt; p.Ht = pl.Ht; p.tiles_w = pl.tiles_w; p.tiles_h = pl.tiles_h;
    p.LK = pl.LK; p.taps = taps; p.fmt = fmt; p.has_bias = (pass == PASS_FWD && g.has_bias) ? 1 : 0;
    p.stage_bytes = pl.stage_bytes; p.plane_bytes = (uint32_t)pl.Ht * pl.Wt * 16;
    p.store_vec = 1;
    while (p.store_vec < 8 && pl.Wout % (p.store_vec * 2) == 0 && (reinterpret_cast<uintptr_t>(out) % (size_t)(p.store_vec * 4)) == 0) p.store_vec *= 2;

    const CUtensorMapDataType dt = fmt == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    alignas(64) CUtensorMap map_w, map_x;
    {   // Wexp[tap][k / 8][128][8] seen as (32 rows x 8, 4, k / 8, tap); box = 2 planes of 128 rows
        const cuuint64_t dims[4] = {256, NM / 32, (cuuint64_t)Kp / 8, (cuuint64_t)taps};
        const cuuint64_t strides[3] = {512, (cuuint64_t)NM * 16, (cuuint64_t)(Kp / 8) * NM * 16};
        const cuuint32_t box[4] = {256, NM / 32, 2, 1};
        const int rc = make_tensor_map(&map_w, dt, wexp, 4, dims, strides, box, nullptr, CU_TENSOR_MAP_SWIZZLE_NONE, "narrow filters");
        if (rc != PCB_OK) return rc;
    }
    {   // xp[comp][img][plane][hp][wp][8] seen as (wp x 8, hp, plane, img, comp); box = the halo tile of one component
        const cuuint64_t dims[5] = {(cuuint64_t)pl.Wp * 8, (cuuint64_t)pl.Hp, 2, (cuuint64_t)g.Nb, (cuuint64_t)pl.LK};
        const cuuint64_t strides[4] = {(cuuint64_t)pl.Wp * 16, (cuuint64_t)pl.Hp * pl.Wp * 16, (cuuint64_t)2 * pl.Hp * pl.Wp * 16,
                                       (cuuint64_t)g.Nb * 2 * pl.Hp * pl.Wp * 16};
        const cuuint32_t box[5] = {(cuuint32_t)pl.Wt * 8, (cuuint32_t)pl.Ht, 2, 1, 1};
        const int rc = make_tensor_map(&map_x, dt, xp, 5, dims, strides, box, nullptr, CU_TENSOR_MAP_SWIZZLE_NONE, "narrow activations");
        if (rc != PCB_OK) return rc;
    }
    const int n_tiles = pl.tiles_w * pl.tiles_h * g.Nb;
    const int grid = n_tiles < sm_count() ? n_tiles : sm_count();
    PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_narrow_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
    qconv_narrow_tc_kernel<<<grid, N_THREADS, pl.smem, stream>>>(map_w, map_x, p, (const uint16_t*)bias, (uint16_t*)out, status);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

namespace {

struct NFPlan {
    int s2d, KHe, KWe, DHe, DWe, Cie;    // effective (staged) filter and channels
    int LK, PH, Wt, Ht, tiles_w, tiles_h, Hp, Wp, HOp, WOp, y_planes, taps_per_group, n_groups;
    int fold, fold_h, LKe, taps;         // kw / kh taps folded into one MMA (1 = none), columns / 16 of one MMA, MMAs per 16 pixels
    uint32_t y_bytes, x_bytes, stage_bytes;
    size_t xp_bytes, dyp_bytes, acc_bytes, smem;
};

NFPlan make_nfplan(const Geom& g) {
    NFPlan f;
    f.LK = g.real_in ? 1 : g.nc;
    f.s2d = s2d_layer(g) ? 1 : 0;
    f.KHe = f.s2d ? (g.KH + 1) / 2 : g.KH; f.KWe = f.s2d ? (g.KW + 1) / 2 : g.KW;
    f.DHe = f.s2d ? 1 : g.DH; f.DWe = f.s2d ? 1 : g.DW;
    f.Cie = f.s2d ? 4 * g.Ci : g.Ci;
    // the staged copies (shared with the forward pass, see forward_keeps_staged_input) follow the standard tile height
    const int rows = (g.HO + 31) / 32;
    const int ph_std = (((g.HO + rows - 1) / rows) + 1) & ~1;
    f.tiles_w = (g.WO + 7) / 8;
    f.HOp = ((g.HO + ph_std - 1) / ph_std) * ph_std; f.WOp = f.tiles_w * 8;
    f.Hp = f.HOp + (f.KHe - 1) * f.DHe; f.Wp = f.WOp + (f.KWe - 1) * f.DWe;
    f.y_planes = (g.Co + 7) / 8;
    // folded form: all kw taps of a filter row in the columns of one MMA, if those fit one MMA (N <= 256)
    f.fold = (f.KWe > 1 && f.KWe * f.LK * 16 <= 256) ? f.KWe : 1;
    // ... and the filter rows too for a one-component x (the tensor map has a dimension to spare)
    f.fold_h = (f.fold > 1 && f.LK == 1 && f.KHe > 1 && f.KHe * f.KWe * 16 <= 256) ? f.KHe : 1;
    f.LKe = f.LK * f.fold * f.fold_h;
    f.taps = f.fold_h > 1 ? 1 : (f.fold > 1 ? f.KHe : f.KHe * f.KWe);
    f.Wt = f.fold > 1 ? 8 : 8 + (f.KWe - 1) * f.DWe;
    const int ncols = f.LKe * 16;
    f.n_groups = (f.taps * ncols + 511) / 512;
    f.taps_per_group = (f.taps + f.n_groups - 1) / f.n_groups;
    f.n_groups = (f.taps + f.taps_per_group - 1) / f.taps_per_group;
    // the kernel's own tile height: the standard one, lowered until two stages fit the shared memory (rows past the staged
    // planes read as zeros through the tensor maps)
    for (int r = rows;; ++r) {
        f.PH = (((g.HO + r - 1) / r) + 1) & ~1;
        f.tiles_h = (g.HO + f.PH - 1) / f.PH;
        f.Ht = f.fold_h > 1 ? f.PH : f.PH + (f.KHe - 1) * f.DHe;
        f.y_bytes = (uint32_t)g.nc * f.y_planes * f.PH * 128;
        f.x_bytes = (uint32_t)f.LKe * 2 * f.Ht * f.Wt * 16;
        f.stage_bytes = (f.y_bytes + f.x_bytes + 1023) / 1024 * 1024;
        // the M = 128 operand spans 16 chunks of PH * 128 bytes from the start of a dy tile
        const size_t slack = (size_t)16 * f.PH * 128;
        f.smem = 1024 + 1024 + (size_t)NF_STAGES * f.stage_bytes + slack;
        if (f.smem <= 226 * 1024 || f.PH <= 2) break;
    }
    f.xp_bytes = ((size_t)f.LK * g.Nb * 2 * f.Hp * f.Wp * 16 + 1023) / 1024 * 1024;
    f.dyp_bytes = ((size_t)g.nc * g.Nb * f.y_planes * f.HOp * f.WOp * 16 + 1023) / 1024 * 1024;
    f.acc_bytes = ((size_t)g.nc * g.Co * f.Cie * f.KHe * f.KWe * sizeof(float) + 1023) / 1024 * 1024;
    return f;
}

}  // namespace

bool narrow_filter_tc_supported(int dtype, int variant, const Geom& g) {
    if (dtype != PCB_F16 && dtype != PCB_BF16) return false;
    if (variant != PCB_VARIANT_16_PRODUCT || g.w_io || g.dw_io) return false;
    if (g.H * g.W == 1 || ((g.SH != 1 || g.SW != 1) && !s2d_layer(g))) return false;
    if ((s2d_layer(g) ? 4 * g.Ci : g.Ci) > 16 || g.nc * ((g.Co + 7) / 8) > 16) return false;   // x: two planes; dy: at most 16 chunks of 8 rows
    if (g.WO < 8 || g.HO < 8) return false;
    const NFPlan f = make_nfplan(g);
    if (f.Wt > 32 || f.Ht > 255 || f.smem > 226 * 1024) return false;
    if (f.xp_bytes + f.dyp_bytes > (size_t)12 << 30) return false;
    return true;
}

size_t narrow_filter_tc_scratch_bytes(const Geom& g) {
    const NFPlan f = make_nfplan(g);
    return f.xp_bytes + f.dyp_bytes + f.acc_bytes;
}

bool narrow_tc_staged_dy_view(const Geom& g, StagedView* view, size_t* bytes) {
    if (g.SH != 1 || g.SW != 1) return false;                   // strided layers: backward-data reads a zero-inserted copy
    const NPlan pl = make_nplan(PASS_BWD_DATA, g);
    view->Hp = pl.Hp; view->Wp = pl.Wp; view->pad_top = pl.pad_top; view->pad_left = pl.pad_left;
    *bytes = pl.xp_bytes;
    return pl.pad_top >= 0 && pl.pad_left >= 0;
}

int narrow_filter_tc_launch(int dtype, const Geom& g, const void* dy, const void* x, void* dw, void* scratch, int* status, cudaStream_t stream,
                            const void* kept_x, const StagedView* kept_dy) {
    const int fmt = dtype == PCB_F16 ? 0 : 1;
    const NFPlan f = make_nfplan(g);
    const int taps = f.KHe * f.KWe;                 // filter taps of the staged problem (the folded form issues KHe MMAs per 16 pixels)
    // the forward pass of a narrow layer stages x exactly as this one does: a copy it kept is read in place
    uint8_t* xp = kept_x ? static_cast<uint8_t*>(const_cast<void*>(kept_x)) : static_cast<uint8_t*>(scratch);
    uint8_t* dyp = static_cast<uint8_t*>(scratch) + f.xp_bytes;
    float* acc = reinterpret_cast<float*>(dyp + f.dyp_bytes);
    {
        // x: padded planar copy (space-to-depth for the stride-2 stem); dy: planar copy rounded up to whole tiles
        auto stage = [&](const void* src, void* dst, int planes_in, int C, int H, int W, int Hp, int Wp, int groups, int pt, int pleft, int s2d) {
            const size_t total = (size_t)planes_in * groups * Hp * Wp;
            if (!s2d && pack_rows_px(src, W, Wp, pleft, 1, 1) == 4) {
                const int blocks = grid_cap(total / 4 + 1, 256, 16);
                if (fmt == 0) pack_rows_kernel<__half, 4><<<blocks, 256, 0, stream>>>((const __half*)src, (__half*)dst, planes_in, C, H, W, Hp, Wp, groups, pt, pleft, 1);
                else pack_rows_kernel<__nv_bfloat16, 4><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, planes_in, C, H, W, Hp, Wp, groups, pt, pleft, 1);
            } else if (s2d && groups == 2 && (fmt == 0 ? launch_s2d_pairs<__half>(src, dst, planes_in, C, H, W, Hp, Wp, pt, pleft, stream)
                                                       : launch_s2d_pairs<__nv_bfloat16>(src, dst, planes_in, C, H, W, Hp, Wp, pt, pleft, stream))) {
                // space-to-depth copy from aligned source pairs
            } else {
                const int blocks = grid_cap(total, 256, 16);
                if (fmt == 0) pack_planar_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)src, (__half*)dst, planes_in, C, H, W, Hp, Wp, groups, pt, pleft, 1, 1, s2d);
                else pack_planar_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, planes_in, C, H, W, Hp, Wp, groups, pt, pleft, 1, 1, s2d);
            }
        };
        if (!kept_x) stage(x, xp, f.LK * g.Nb, g.Ci, g.H, g.W, f.Hp, f.Wp, 2, g.PT, g.PL, f.s2d);
        if (!kept_dy) stage(dy, dyp, g.nc * g.Nb, g.Co, g.HO, g.WO, f.HOp, f.WOp, f.y_planes, 0, 0, 0);
        PCB_CUDA_TRY(cudaGetLastError());
        PCB_CUDA_TRY(cudaMemsetAsync(acc, 0, (size_t)g.nc * g.Co * f.Cie * taps * sizeof(float), stream));
    }
    NFParams p;
    p.Nb = g.Nb; p.Co = g.Co; p.Ci = f.Cie; p.nc = g.nc; p.ga = g.ga; p.neg = g.neg;
    p.KH = f.KHe; p.KW = f.fold > 1 ? 1 : f.KWe; p.DH = f.DHe; p.DW = f.DWe;
    p.PH = f.PH; p.Wt = f.Wt; p.Ht = f.Ht; p.tiles_w = f.tiles_w; p.tiles_h = f.tiles_h;
    p.LK = f.LKe; p.LKr = f.LK; p.fold = f.fold; p.fold_h = f.fold_h;
    p.taps = f.taps; p.taps_per_group = f.taps_per_group; p.n_groups = f.n_groups; p.y_planes = f.y_planes;
    p.fmt = fmt; p.y_bytes = f.y_bytes; p.x_bytes = f.x_bytes; p.stage_bytes = f.stage_bytes; p.plane_bytes = (uint32_t)f.Ht * f.Wt * 16;
    p.steps_total = f.tiles_w * f.tiles_h * g.Nb;
    int splits = split_count(f.n_groups, sm_count());
    if (splits > p.steps_total) splits = p.steps_total;
    if (splits < 1) splits = 1;
    p.steps_per_split = (p.steps_total + splits - 1) / splits;
    splits = (p.steps_total + p.steps_per_split - 1) / p.steps_per_split;
    int grid = f.n_groups * splits;
    p.uneven = 0;
    const int last_taps = f.taps - (f.n_groups - 1) * f.taps_per_group;
    if (f.n_groups > 1 && f.n_groups <= NF_MAX_GROUPS && last_taps < f.taps_per_group) {
        // CTA shares in proportion to the taps of each group (one wave of CTAs)
        const int sms = sm_count();
        int begin = 0;
        for (int gi = 0; gi < f.n_groups; ++gi) {
            const int taps_g = gi + 1 < f.n_groups ? f.taps_per_group : last_taps;
            int share = (int)((long long)sms * taps_g / f.taps);
            if (share < 1) share = 1;
            if (share > p.steps_total) share = p.steps_total;
            p.group_steps[gi] = (p.steps_total + share - 1) / share;
            share = (p.steps_total + p.group_steps[gi] - 1) / p.group_steps[gi];
            p.cta_begin[gi] = begin;
            begin += share;
        }
        p.cta_begin[f.n_groups] = begin;
        p.uneven = 1;
        grid = begin;
    }

    const CUtensorMapDataType dt = fmt == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    alignas(64) CUtensorMap map_dy, map_x;
    {   // dyp[d][img][plane][HOp][WOp][8] seen as (w x 8, h, plane, img, d); box = the tile of all components
        const cuuint64_t dims[5] = {(cuuint64_t)f.WOp * 8, (cuuint64_t)f.HOp, (cuuint64_t)f.y_planes, (cuuint64_t)g.Nb, (cuuint64_t)g.nc};
        const cuuint64_t strides[4] = {(cuuint64_t)f.WOp * 16, (cuuint64_t)f.HOp * f.WOp * 16, (cuuint64_t)f.y_planes * f.HOp * f.WOp * 16,
                                       (cuuint64_t)g.Nb * f.y_planes * f.HOp * f.WOp * 16};
        const cuuint32_t box[5] = {64, (cuuint32_t)f.PH, (cuuint32_t)f.y_planes, 1, (cuuint32_t)g.nc};
        int rc;
        if (kept_dy) {
            // the copy backward-data staged: [d][img][2 planes][Hp][Wp][8] with pixel (0, 0) at (pad_top, pad_left); only the
            // HO x WO pixels are inside the map, so whatever a tile box takes beyond them reads as zeros
            const size_t plane = (size_t)kept_dy->Hp * kept_dy->Wp * 16;
            const cuuint64_t kdims[5] = {(cuuint64_t)g.WO * 8, (cuuint64_t)g.HO, (cuuint64_t)f.y_planes, (cuuint64_t)g.Nb, (cuuint64_t)g.nc};
            const cuuint64_t kstrides[4] = {(cuuint64_t)kept_dy->Wp * 16, plane, 2 * plane, (cuuint64_t)g.Nb * 2 * plane};
            uint8_t* origin = static_cast<uint8_t*>(const_cast<void*>(kept_dy->base)) + ((size_t)kept_dy->pad_top * kept_dy->Wp + kept_dy->pad_left) * 16;
            rc = make_tensor_map(&map_dy, dt, origin, 5, kdims, kstrides, box, nullptr, CU_TENSOR_MAP_SWIZZLE_NONE, "narrow dy (shared)");
        } else {
            rc = make_tensor_map(&map_dy, dt, dyp, 5, dims, strides, box, nullptr, CU_TENSOR_MAP_SWIZZLE_NONE, "narrow dy");
        }
        if (rc != PCB_OK) return rc;
    }
    if (f.fold > 1) {
        // the same copy with the kw tap as a dimension of its own, one pixel (16 bytes) apart: (w x 8, h, image and plane, l, kw);
        // box = the tile, 8 pixels wide, of every component at every kw shift. The first extent stops short of the halo columns so
        // that the shifted views stay inside their rows.
        // With the filter rows folded as well the fourth dimension is kh (one staged row apart) instead of the component, and
        // the second extent stops short of the halo rows for the same reason.
        const size_t plane = (size_t)f.Hp * f.Wp * 16;
        const bool fh = f.fold_h > 1;
        const cuuint64_t dims[5] = {(cuuint64_t)f.WOp * 8, (cuuint64_t)(fh ? f.HOp : f.Hp), (cuuint64_t)2 * g.Nb, (cuuint64_t)(fh ? f.fold_h : f.LK),
                                    (cuuint64_t)f.fold};
        const cuuint64_t strides[4] = {(cuuint64_t)f.Wp * 16, plane, fh ? (cuuint64_t)f.DHe * f.Wp * 16 : (cuuint64_t)g.Nb * 2 * plane,
                                       (cuuint64_t)f.DWe * 16};
        const cuuint32_t box[5] = {64, (cuuint32_t)f.Ht, 2, (cuuint32_t)(fh ? f.fold_h : f.LK), (cuuint32_t)f.fold};
        const int rc = make_tensor_map(&map_x, dt, xp, 5, dims, strides, box, nullptr, CU_TENSOR_MAP_SWIZZLE_NONE, "narrow x (folded)");
        if (rc != PCB_OK) return rc;
    } else {   // xp[l][img][plane][Hp][Wp][8]; box = the halo tile of all components
        const cuuint64_t dims[5] = {(cuuint64_t)f.Wp * 8, (cuuint64_t)f.Hp, 2, (cuuint64_t)g.Nb, (cuuint64_t)f.LK};
        const cuuint64_t strides[4] = {(cuuint64_t)f.Wp * 16, (cuuint64_t)f.Hp * f.Wp * 16, (cuuint64_t)2 * f.Hp * f.Wp * 16,
                                       (cuuint64_t)g.Nb * 2 * f.Hp * f.Wp * 16};
        const cuuint32_t box[5] = {(cuuint32_t)f.Wt * 8, (cuuint32_t)f.Ht, 2, 1, (cuuint32_t)f.LK};
        const int rc = make_tensor_map(&map_x, dt, xp, 5, dims, strides, box, nullptr, CU_TENSOR_MAP_SWIZZLE_NONE, "narrow x");
        if (rc != PCB_OK) return rc;
    }
    PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_narrow_filter_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)f.smem));
    qconv_narrow_filter_tc_kernel<<<grid, N_THREADS, f.smem, stream>>>(map_dy, map_x, p, acc, status);
    PCB_CUDA_TRY(cudaGetLastError());
    const size_t per_tap = (size_t)g.nc * g.Co * g.Ci;
    const int blocks = grid_cap(per_tap * g.KH * g.KW, 256, 16);
    if (f.s2d) {
        if (fmt == 0) unpack_narrow_filter_grad_s2d_kernel<__half><<<blocks, 256, 0, stream>>>(acc, (__half*)dw, g.nc * g.Co, g.Ci, g.KH, g.KW, f.KWe, taps);
        else unpack_narrow_filter_grad_s2d_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(acc, (__nv_bfloat16*)dw, g.nc * g.Co, g.Ci, g.KH, g.KW, f.KWe, taps);
    } else if (fmt == 0) unpack_narrow_filter_grad_kernel<__half><<<blocks, 256, 0, stream>>>(acc, (__half*)dw, taps, per_tap);
    else unpack_narrow_filter_grad_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(acc, (__nv_bfloat16*)dw, taps, per_tap);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

}  // namespace pcb
