// fp32 quaternion convolution and dense on the tensor cores with error-compensated TF32 ("3xTF32").
//
// tcgen05.mma.kind::tf32 keeps 10 mantissa bits of each fp32 operand, far from the 1e-5 parity the fp32 path
// owes. Every operand is therefore split while it is staged into hi = x with the 13 low mantissa bits cleared
// (exactly a TF32 number) and lo = x - hi (exact in fp32), and each K step issues three MMAs into the same fp32
// accumulator: hi*hi + hi*lo + lo*hi. What is dropped is lo*lo and the rounding of lo (both ~2^-22 relative), so
// the result is as good as an fp32 FMA chain. Cost: 3 TF32 MMAs per product and twice the operand bytes.
//
// Structure as in conv_tc.cu: channels-last zero-padded activations and the signed/permuted filter matrix
// Wexp[tap][(d,co)][(l,ci)] (reference sign table src/algebras.cc:28-49) are staged in the workspace, here in fp32
// and twice (hi, lo); the implicit-GEMM kernel is TMA-fed, 128 x 256 tile, double-buffered TMEM accumulator.
// Dense layers are the 1x1 convolution of 1x1 images (pixels = batch); input-major dense filters and the
// input-major dense filter gradient are handled while staging / unstaging. Replaces, for fp32 tensors, the scalar
// fp32 library calls of src/backend/cudnn/conv2d.hpp:280-309, :447-488 and src/backend/cudnn/dense.hpp:102-133, :181-216.
#include "tc_common.cuh"
#include "tensor_path.cuh"

namespace pcb {
namespace {

using namespace umma;
using namespace tc;

constexpr int TM = 128, TN = 256, TKS = 16;                 // tile, channels (fp32) per K slice: 64-byte rows
constexpr int T_THREADS = 320;
constexpr uint32_t TA_BYTES = TM * TKS * 4, TB_BYTES = TN * TKS * 4;
constexpr uint32_t T_STAGE = 2 * (TA_BYTES + TB_BYTES);     // hi and lo of both operands: 48 KB
constexpr int T_STAGES = 4;
constexpr size_t T_SMEM = 1024 + T_STAGES * T_STAGE + 512;
constexpr int ST_T_PRODUCER = 0x1000, ST_T_MMA = 0x2000, ST_T_EPILOGUE = 0x4000;

struct TParams {
    int Nb, Mvalid, Cout, HO, WO, Cp;
    int KH, KW, SH, SW, DH, DW;
    int PW, PH, PN;
    int tiles_w, tiles_h, tiles_n, tiles_m;
    int has_bias, LK, store_vec;
    int n_chunks, chunk_len;          // a work item's K range runs in n_chunks pieces of at most chunk_len stages
    int splits, k_per_split;          // the K loop of a tile is cut into `splits` work items of k_per_split stages; with more than one
                                      // the partial results meet in the (zeroed) output by fp32 reductions
};

// K-major tile with 64-byte rows (16 fp32), 64-byte swizzle.
__device__ __forceinline__ uint64_t desc_k64(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(512 >> 4) << 32) | DESC_VERSION_SM100 | (4ull << 61);
}

// Each MMA truncates when it adds into the TMEM accumulator, so the error of one accumulator grows with the number
// of MMAs it takes (measured: about 3e-8 of the largest output per MMA). K loops are therefore cut into chunks of
// at most T_CHUNK stages; chunks alternate between the two TMEM buffers (as whole tiles do when one chunk is
// enough) and the epilogue warps add them up in registers, rounding to nearest.
constexpr int T_CHUNK = 16;           // 16 stages = 96 MMAs = 256 fp32 of K

template <bool CHUNKED>
__global__ void __launch_bounds__(T_THREADS, 1)
qconv_general_tf32_kernel(const __grid_constant__ CUtensorMap map_w_hi, const __grid_constant__ CUtensorMap map_w_lo,
                          const __grid_constant__ CUtensorMap map_x_hi, const __grid_constant__ CUtensorMap map_x_lo, TParams p,
                          const float* __restrict__ bias, float* __restrict__ out, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + T_STAGES * T_STAGE);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * T_STAGES + 4);
    const uint32_t tiles_addr = smem_u32(base);
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + T_STAGES);
    const uint32_t tmem_full = smem_u32(bars + 2 * T_STAGES), tmem_empty = smem_u32(bars + 2 * T_STAGES + 2);

    const int n_items = p.tiles_w * p.tiles_h * p.tiles_n * p.tiles_m * p.splits;
    const int c_steps = p.Cp / TKS;
    const int n_k = p.KH * p.KW * p.LK * c_steps;

    if (t == 0) {
        for (int s = 0; s < T_STAGES; ++s) { mbar_init(full_bar + 8 * s, 1); mbar_init(empty_bar + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tmem_full + 8 * b, 1); mbar_init(tmem_empty + 8 * b, 8); }
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const int tile = item / p.splits, split = item - tile * p.splits;
                const int tm = tile % p.tiles_m;
                int rest = tile / p.tiles_m;
                const int tw = rest % p.tiles_w; rest /= p.tiles_w;
                const int th = rest % p.tiles_h;
                const int tn = rest / p.tiles_h;
                const int m0 = tm * TM, ow0 = tw * p.PW, oh0 = th * p.PH, n0 = tn * p.PN;
                const int k0 = split * p.k_per_split, k1 = min(n_k, k0 + p.k_per_split);
                // stage k = (tap * LK + l) * c_steps + cs
                int cs = k0 % c_steps, l = (k0 / c_steps) % p.LK, tap = k0 / (c_steps * p.LK);
                for (int k = k0; k < k1; ++k, ++it) {
                    const int kh = tap / p.KW, kw = tap - kh * p.KW;
                    const int wp0 = ow0 * p.SW + kw * p.DW, hp0 = oh0 * p.SH + kh * p.DH;
                    const int s = it % T_STAGES;
                    ok = mbar_wait_bounded(empty_bar + 8 * s, ((it / T_STAGES) & 1) ^ 1, status, ST_T_PRODUCER);
                    if (!ok) break;
                    const uint32_t dst = tiles_addr + s * T_STAGE, bar = full_bar + 8 * s;
                    mbar_arrive_expect_tx(bar, T_STAGE);
                    tma_load_3d(dst, &map_w_hi, l * p.Cp + cs * TKS, m0, tap, bar);
                    tma_load_3d(dst + TA_BYTES, &map_w_lo, l * p.Cp + cs * TKS, m0, tap, bar);
                    tma_load_5d(dst + 2 * TA_BYTES, &map_x_hi, cs * TKS, wp0, hp0, n0, l, bar);
                    tma_load_5d(dst + 2 * TA_BYTES + TB_BYTES, &map_x_lo, cs * TKS, wp0, hp0, n0, l, bar);
                    if (++cs == c_steps) { cs = 0; if (++l == p.LK) { l = 0; ++tap; } }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        const uint32_t idesc = make_idesc_f16(2, TM, TN, false, false);
        int it = 0, unit = 0;                       // unit = one accumulator's worth of work: a chunk of a tile
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int split = item % p.splits;
            const int k0 = split * p.k_per_split, k1 = min(n_k, k0 + p.k_per_split);
            for (int c = 0; c < p.n_chunks && ok; ++c, ++unit) {
                const int buf = unit & 1, use = unit >> 1;
                if (use > 0) {
                    ok = mbar_wait_bounded(tmem_empty + 8 * buf, (use - 1) & 1, status, ST_T_MMA);
                    if (!ok) break;
                    tc_fence_after_sync();
                }
                const int k_beg = k0 + c * p.chunk_len, k_end = min(k1, k_beg + p.chunk_len);
                for (int k = k_beg; k < k_end && ok; ++k, ++it) {
                    const int s = it % T_STAGES;
                    ok = mbar_wait_bounded(full_bar + 8 * s, (it / T_STAGES) & 1, status, ST_T_MMA);
                    if (!ok) break;
                    tc_fence_after_sync();
                    if (lane == 0) {
                        const uint32_t a_hi = tiles_addr + s * T_STAGE, a_lo = a_hi + TA_BYTES, b_hi = a_hi + 2 * TA_BYTES, b_lo = b_hi + TB_BYTES;
                        const uint32_t d = tmem_base + buf * TN;
#pragma unroll
                        for (int j = 0; j < TKS / 8; ++j) {             // 8 fp32 = 32 bytes per MMA along a row
                            mma_tf32_ss(d, desc_k64(a_lo + j * 32), desc_k64(b_hi + j * 32), idesc, (k > k_beg || j > 0) ? 1u : 0u);   // small terms first
                            mma_tf32_ss(d, desc_k64(a_hi + j * 32), desc_k64(b_lo + j * 32), idesc, 1u);
                            mma_tf32_ss(d, desc_k64(a_hi + j * 32), desc_k64(b_hi + j * 32), idesc, 1u);
                        }
                        mma_commit(empty_bar + 8 * s);
                        if (k == k_end - 1) mma_commit(tmem_full + 8 * buf);
                    }
                    __syncwarp();
                }
            }
        }
    } else {
        const int q = warp & 3, chalf = (warp - 2) >> 2;
        const int sv = p.store_vec;                  // pixels per store: 8, 4, 2 or 1
        int unit = 0;
        bool ok = true;
        const bool reduce = p.splits > 1;            // partial sums of a tile meet in the zeroed output
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int tile = item / p.splits, split = item - tile * p.splits;
            const int tm = tile % p.tiles_m;
            int rest = tile / p.tiles_m;
            const int tw = rest % p.tiles_w; rest /= p.tiles_w;
            const int th = rest % p.tiles_h;
            const int tn = rest / p.tiles_h;
            const int ow0 = tw * p.PW, oh0 = th * p.PH, n0 = tn * p.PN;
            const int m = tm * TM + q * 32 + lane;
            const bool row_ok = m < p.Mvalid;
            const int d = row_ok ? m / p.Cout : 0, co = m - d * p.Cout;
            const float badd = (row_ok && p.has_bias && split == 0) ? bias[d * p.Cout + co] : 0.f;
            float part[CHUNKED ? 4 : 1][CHUNKED ? 32 : 1];          // this thread's 128 columns, summed over the chunks so far
            if (CHUNKED) {
#pragma unroll
                for (int cb = 0; cb < 4; ++cb)
#pragma unroll
                    for (int e = 0; e < 32; ++e) part[cb][e] = 0.f;
                for (int c = 0; c + 1 < p.n_chunks && ok; ++c, ++unit) {
                    const int buf = unit & 1, use = unit >> 1;
                    ok = mbar_wait_bounded(tmem_full + 8 * buf, use & 1, status, ST_T_EPILOGUE);
                    ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
                    if (!ok) break;
                    tc_fence_after_sync();
#pragma unroll
                    for (int cb = 0; cb < 4; ++cb) {
                        uint32_t v[32];
                        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * TN + chalf * 128 + cb * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) part[cb][e] += __uint_as_float(v[e]);
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tmem_empty + 8 * buf);
                }
                if (!ok) break;
            }
            const int buf = unit & 1, use = unit >> 1;
            ++unit;
            ok = mbar_wait_bounded(tmem_full + 8 * buf, use & 1, status, ST_T_EPILOGUE);
            ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll(CHUNKED ? 4 : 1)
            for (int cb = 0; cb < 4; ++cb) {
                uint32_t v[32];
                const int col0 = chalf * 128 + cb * 32;
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * TN + col0, v);
                tmem_ld_wait();
                if (!row_ok) continue;
#pragma unroll
                for (int e = 0; e < 32; ++e)
                    v[e] = __float_as_uint(__uint_as_float(v[e]) + (CHUNKED ? part[cb][e] : 0.f) + badd);
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {
                    const int j = col0 + g8 * 8;
                    const int wl = j % p.PW, hl = (j / p.PW) % p.PH, nl = j / (p.PW * p.PH);
                    const int ow = ow0 + wl, oh = oh0 + hl, img = n0 + nl;
                    if (p.PW >= 8) {
                        if (ow >= p.WO || oh >= p.HO || img >= p.Nb) continue;
                        float* dst = out + (((size_t)(d * p.Nb + img) * p.Cout + co) * p.HO + oh) * p.WO + ow;
                        if (reduce) {
                            if (sv >= 4) {
#pragma unroll
                                for (int h = 0; h < 2; ++h)
                                    if (ow + 4 * h < p.WO)
                                        red_add_f32x4(dst + 4 * h, __uint_as_float(v[8 * g8 + 4 * h]), __uint_as_float(v[8 * g8 + 4 * h + 1]),
                                                      __uint_as_float(v[8 * g8 + 4 * h + 2]), __uint_as_float(v[8 * g8 + 4 * h + 3]));
                            } else {
#pragma unroll
                                for (int e = 0; e < 8; ++e)
                                    if (ow + e < p.WO) atomicAdd(dst + e, __uint_as_float(v[8 * g8 + e]));
                            }
                        } else if (sv >= 8) {
                            st_global_v8(dst, &v[8 * g8]);
                        } else if (sv == 4) {
#pragma unroll
                            for (int h = 0; h < 2; ++h)
                                if (ow + 4 * h < p.WO) *reinterpret_cast<uint4*>(dst + 4 * h) = make_uint4(v[8 * g8 + 4 * h], v[8 * g8 + 4 * h + 1], v[8 * g8 + 4 * h + 2], v[8 * g8 + 4 * h + 3]);
                        } else if (sv == 2) {
#pragma unroll
                            for (int h = 0; h < 4; ++h)
                                if (ow + 2 * h < p.WO) *reinterpret_cast<uint2*>(dst + 2 * h) = make_uint2(v[8 * g8 + 2 * h], v[8 * g8 + 2 * h + 1]);
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                if (ow + e < p.WO) dst[e] = __uint_as_float(v[8 * g8 + e]);
                        }
                    } else {
                        // narrow boxes (dense layers: one pixel per image): every column is its own (image, row, pixel)
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const int je = j + e;
                            const int w2 = je % p.PW, h2 = (je / p.PW) % p.PH, n2 = je / (p.PW * p.PH);
                            if (ow0 + w2 < p.WO && oh0 + h2 < p.HO && n0 + n2 < p.Nb) {
                                float* dst = out + (((size_t)(d * p.Nb + n0 + n2) * p.Cout + co) * p.HO + oh0 + h2) * p.WO + ow0 + w2;
                                if (reduce) atomicAdd(dst, __uint_as_float(v[8 * g8 + e]));
                                else *dst = __uint_as_float(v[8 * g8 + e]);
                            }
                        }
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

// ---- staging: fp32 -> (hi, lo) ------------------------------------------------------------------------
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
    hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
    lo = x - hi;
}

// A block takes 32 consecutive padded pixels of one plane and up to 64 channels at a time through shared memory: the NCHW reads
// run along the pixels of one channel (coalesced), the channels-last writes along the channel groups of one pixel (coalesced;
// a thread per (pixel, 4 channels) writes one float4 of hi and one of lo).
__global__ void __launch_bounds__(256)
pack_activations_f32_kernel(const float* __restrict__ x, float* __restrict__ hi, float* __restrict__ lo, int planes, int C,
                            int H, int W, int Hp, int Wp, int Cp, int pad_top, int pad_left, int ins_h, int ins_w,
                            int cb, int Nb) {
    __shared__ float tile[64][33];
    const int PP = Hp * Wp, tiles_pp = (PP + 31) / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long n_tiles = (long long)planes * tiles_pp;
    for (long long t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const int plane = (int)(t / tiles_pp), pp0 = (int)(t - (long long)plane * tiles_pp) * 32;
        const int pp = pp0 + lane;
        const int hp = pp / Wp, wp = pp - hp * Wp;
        int ih = hp - pad_top, iw = wp - pad_left;
        bool inside = pp < PP && ih >= 0 && iw >= 0;
        if (inside && (ins_h > 1 || ins_w > 1)) {
            inside = (ih % ins_h == 0) && (iw % ins_w == 0);
            ih /= ins_h; iw /= ins_w;
        }
        inside = inside && ih < H && iw < W;
        const float* src = x + ((size_t)plane * C * H + ih) * W + iw;      // + c * H * W
        for (int c0 = 0; c0 < Cp; c0 += 64) {
            const int c_pass = min(64, Cp - c0);
            for (int c = warp; c < c_pass; c += 8) tile[c][lane] = (inside && c0 + c < C) ? __ldg(src + (size_t)(c0 + c) * H * W) : 0.f;
            __syncthreads();
            const int groups = c_pass / 4;
            for (int idx = threadIdx.x; idx < 32 * groups; idx += 256) {
                const int g = idx % groups, px = idx / groups;
                if (pp0 + px >= PP) continue;
                float4 vh, vl;
                split_tf32(tile[4 * g][px], vh.x, vl.x);
                split_tf32(tile[4 * g + 1][px], vh.y, vl.y);
                split_tf32(tile[4 * g + 2][px], vh.z, vl.z);
                split_tf32(tile[4 * g + 3][px], vh.w, vl.w);
                const int ch = c0 + 4 * g;
                size_t o = ((size_t)plane * PP + pp0 + px) * Cp + ch;
                if (cb > 0) {   // blocks of cb channels, block index outermost: [comp * (Cp / cb) + c / cb][img][hp][wp][cb]
                    const int comp = plane / Nb, img = plane - comp * Nb, bl = ch / cb;
                    o = ((((size_t)comp * (Cp / cb) + bl) * Nb + img) * PP + pp0 + px) * cb + (ch - bl * cb);
                }
                *reinterpret_cast<float4*>(hi + o) = vh;
                *reinterpret_cast<float4*>(lo + o) = vl;
            }
            __syncthreads();
        }
    }
}

// The same staging, one thread per (pixel, 4 channels), for planes of fewer than 32 padded pixels (dense layers are 1 x 1 images:
// consecutive threads then walk the channel groups of one row, and both sides are contiguous).
__global__ void pack_activations_f32_small_kernel(const float* __restrict__ x, float* __restrict__ hi, float* __restrict__ lo, int planes, int C,
                                                  int H, int W, int Hp, int Wp, int Cp, int pad_top, int pad_left, int ins_h, int ins_w,
                                                  int cb, int Nb) {
    const int groups = Cp / 4;
    const size_t total = (size_t)planes * Hp * Wp * groups;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int wp = (int)(idx % Wp);
        size_t rest = idx / Wp;
        const int grp = (int)(rest % groups); rest /= groups;
        const int hp = (int)(rest % Hp);
        const int plane = (int)(rest / Hp);
        int ih = hp - pad_top, iw = wp - pad_left;
        bool inside = ih >= 0 && iw >= 0;
        if (inside && (ins_h > 1 || ins_w > 1)) {
            inside = (ih % ins_h == 0) && (iw % ins_w == 0);
            ih /= ins_h; iw /= ins_w;
        }
        inside = inside && ih < H && iw < W;
        float4 vh, vl;
        float* ph = &vh.x; float* pl = &vl.x;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int c = grp * 4 + e;
            float v = 0.f;
            if (c < C && inside) v = __ldg(x + (((size_t)plane * C + c) * H + ih) * W + iw);
            split_tf32(v, ph[e], pl[e]);
        }
        size_t o = (((size_t)plane * Hp + hp) * Wp + wp) * Cp + grp * 4;
        if (cb > 0) {
            const int comp = plane / Nb, img = plane - comp * Nb, b = (grp * 4) / cb;
            o = (((((size_t)comp * (Cp / cb) + b) * Nb + img) * Hp + hp) * Wp + wp) * cb + (grp * 4 - b * cb);
        }
        *reinterpret_cast<float4*>(hi + o) = vh;
        *reinterpret_cast<float4*>(lo + o) = vl;
    }
}

void stage_activations_f32(const float* x, float* hi, float* lo, int planes, int C, int H, int W, int Hp, int Wp, int Cp, int pad_top, int pad_left,
                           int ins_h, int ins_w, int cb, int Nb, cudaStream_t stream) {
    if (Hp * Wp < 32) {
        pack_activations_f32_small_kernel<<<grid_cap((size_t)planes * Hp * Wp * (Cp / 4), 256, 16), 256, 0, stream>>>(
            x, hi, lo, planes, C, H, W, Hp, Wp, Cp, pad_top, pad_left, ins_h, ins_w, cb, Nb);
    } else {
        const size_t tiles = (size_t)planes * ((Hp * Wp + 31) / 32);
        pack_activations_f32_kernel<<<grid_cap(tiles, 1, 16), 256, 0, stream>>>(x, hi, lo, planes, C, H, W, Hp, Wp, Cp, pad_top, pad_left, ins_h,
                                                                                 ins_w, cb, Nb);
    }
}

// Forward:       Wexp[tap][m = d*Co + co][k = l*Cp + ci]  = s(l,d) * w[l^d](co, ci, tap)
// Backward-data: Wexp[tap][m = l*Ci + ci][k = d*Cop + co] = s(l,d) * w[l^d](co, ci, taps-1-tap)
// w_io: the filters are stored [r][ci][co] (dense input-major layout, one tap).
__global__ void pack_filters_f32_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo, int Co, int Ci, int taps,
                                        int Mp, int Kp, int Cp, int transposed, int w_io, int nc, int ga, unsigned long long neg) {
    // one row (tap, m) of the expanded matrix per block iteration; the row is decoded once and the threads walk k
    const int Cm = transposed ? Ci : Co, Ck = transposed ? Co : Ci;
    const int rows = taps * Mp;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const int tap = row / Mp, m = row - tap * Mp;
        const int cm_comp = m / Cm, cm = m - cm_comp * Cm;
        const int src_tap = transposed ? taps - 1 - tap : tap;
        float* hrow = hi + (size_t)row * Kp;
        float* lrow = lo + (size_t)row * Kp;
        for (int k = threadIdx.x; k < Kp; k += blockDim.x) {
            const int ck_comp = k / Cp, ck = k - ck_comp * Cp;
            float v = 0.f;
            if (cm_comp < nc && ck_comp < nc && ck < Ck) {
                const int d = transposed ? ck_comp : cm_comp, l = transposed ? cm_comp : ck_comp;
                const int co = transposed ? ck : cm, ci = transposed ? cm : ck;
                const int r = alg_pair(ga, l, d);
                const size_t src = w_io ? ((size_t)r * Ci + ci) * Co + co : ((size_t)(r * Co + co) * Ci + ci) * taps + src_tap;
                v = __ldg(w + src);
                if (alg_negative(neg, l, d)) v = -v;
            }
            float h, lw;
            split_tf32(v, h, lw);
            hrow[k] = h;
            lrow[k] = lw;
        }
    }
}

// ---- backward-filter ------------------------------------------------------------------------------------
// Both staged tensors MN-major (K = pixels, 16 per stage), M = (d, co), N = (l, ci); per K step of 8 pixels three
// TF32 MMAs; the epilogue folds G[(d,co),(l,ci)] through the quaternion table into fp32 scratch [tap][r][co][ci].
// 32-bit MN-major operands exist in one shared-memory layout only: 128-byte rows (32 channels) swizzled in 32-byte
// units over groups of 4 rows (descriptor layout type 1, TMA swizzle 128B_ATOM_32B), so channels are padded to 32.
constexpr int TFK = 16;
constexpr uint32_t TF_STAGE = 2 * (TM + TN) * TFK * 4;      // 48 KB
struct TFParams {
    int Nb, Co, Ci, HO, WO, Cop, Cip, cbA, cbB;             // channel-block width in fp32 elements: 32
    int KH, KW, SH, SW, DH, DW, PW, PH, PN, tiles_w, tiles_h, tiles_n;
    int m_tiles, n_tiles, n_tile_cols, splits, steps_per_split;
    int nc, ga;                                              // algebra: components, GA(3,0,0) component order
    unsigned long long neg;                                  // negative entries of the block, bit (8*l + d)
};

// leading offset = distance between 32-channel blocks, stride offset = distance between groups of 4 pixel rows
__device__ __forceinline__ uint64_t desc_mn_f32(uint32_t addr, int cb, uint32_t block_bytes) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)((block_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)(((4u * cb * 4u) >> 4) & 0x3FFFu) << 32) | DESC_VERSION_SM100 | (1ull << 61);
}

__global__ void __launch_bounds__(T_THREADS, 1)
qconv_filter_tf32_kernel(const __grid_constant__ CUtensorMap map_dy_hi, const __grid_constant__ CUtensorMap map_dy_lo,
                         const __grid_constant__ CUtensorMap map_x_hi, const __grid_constant__ CUtensorMap map_x_lo, TFParams p,
                         float* __restrict__ dw32, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + T_STAGES * TF_STAGE);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * T_STAGES + 4);
    const uint32_t tiles_addr = smem_u32(base);
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + T_STAGES);
    const uint32_t tmem_full = smem_u32(bars + 2 * T_STAGES), tmem_empty = smem_u32(bars + 2 * T_STAGES + 2);

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
    const int n_chunks = (n_steps + T_CHUNK - 1) / T_CHUNK;       // chunks alternate between the two TMEM buffers

    const int nblkA = TM / p.cbA, nblkB = p.n_tile_cols / p.cbB;
    const int bpcA = p.Cop / p.cbA, bpcB = p.Cip / p.cbB;
    const uint32_t blkA_bytes = TFK * p.cbA * 4, blkB_bytes = TFK * p.cbB * 4;
    const uint32_t a_bytes = nblkA * blkA_bytes, b_bytes = nblkB * blkB_bytes;
    const uint32_t A_REGION = TM * TFK * 4, B_REGION = TN * TFK * 4;      // 8 KB, 16 KB
    const int blockA0 = mt * nblkA, blockB0 = nt * (TN / p.cbB);

    if (t == 0) {
        for (int s = 0; s < T_STAGES; ++s) { mbar_init(full_bar + 8 * s, 1); mbar_init(empty_bar + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tmem_full + 8 * b, 1); mbar_init(tmem_empty + 8 * b, 8); }
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // one copy per operand half and stage (the staged tensors keep the channel-block index outermost, so the blocks
            // of a tile are one box even across components) and a running (tw, th, tn) of the pixel box: no division in
            // this loop -- a division per copy used to bound the kernel
            int tw = step_beg % p.tiles_w, th = (step_beg / p.tiles_w) % p.tiles_h, tn = step_beg / (p.tiles_w * p.tiles_h);
            int s = 0, phase = 1;
            bool ok = true;
            for (int it = 0; it < n_steps && ok; ++it) {
                ok = mbar_wait_bounded(empty_bar + 8 * s, phase, status, ST_T_PRODUCER);
                if (!ok) break;
                const int ow0 = tw * p.PW, oh0 = th * p.PH, n0 = tn * p.PN;
                const uint32_t a_hi = tiles_addr + s * TF_STAGE, a_lo = a_hi + A_REGION, b_hi = a_hi + 2 * A_REGION, b_lo = b_hi + B_REGION;
                const uint32_t bar = full_bar + 8 * s;
                if (++tw == p.tiles_w) { tw = 0; if (++th == p.tiles_h) { th = 0; ++tn; } }
                if (++s == T_STAGES) { s = 0; phase ^= 1; }
                mbar_arrive_expect_tx(bar, 2 * (a_bytes + b_bytes));
                tma_load_5d(a_hi, &map_dy_hi, 0, ow0, oh0, n0, blockA0, bar);
                tma_load_5d(a_lo, &map_dy_lo, 0, ow0, oh0, n0, blockA0, bar);
                const int wp0 = ow0 * p.SW + kw * p.DW, hp0 = oh0 * p.SH + kh * p.DH;
                tma_load_5d(b_hi, &map_x_hi, 0, wp0, hp0, n0, blockB0, bar);
                tma_load_5d(b_lo, &map_x_lo, 0, wp0, hp0, n0, blockB0, bar);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        const uint32_t idesc = make_idesc_f16(2, TM, p.n_tile_cols, true, true);
        bool ok = true;
        for (int c = 0; c < n_chunks && ok; ++c) {
            const int buf = c & 1, use = c >> 1;
            if (use > 0) {
                ok = mbar_wait_bounded(tmem_empty + 8 * buf, (use - 1) & 1, status, ST_T_MMA);
                if (!ok) break;
                tc_fence_after_sync();
            }
            const int k_beg = c * T_CHUNK, k_end = min(n_steps, k_beg + T_CHUNK);
            const uint32_t dcol = tmem_base + buf * TN;
            for (int it = k_beg; it < k_end && ok; ++it) {
                const int s = it % T_STAGES;
                ok = mbar_wait_bounded(full_bar + 8 * s, (it / T_STAGES) & 1, status, ST_T_MMA);
                if (!ok) break;
                tc_fence_after_sync();
                if (lane == 0) {
                    const uint32_t a_hi = tiles_addr + s * TF_STAGE, a_lo = a_hi + A_REGION, b_hi = a_hi + 2 * A_REGION, b_lo = b_hi + B_REGION;
#pragma unroll
                    for (int j = 0; j < TFK / 8; ++j) {                   // 8 pixels (K rows) per MMA
                        const uint32_t ao = j * 8 * p.cbA * 4, bo = j * 8 * p.cbB * 4;
                        mma_tf32_ss(dcol, desc_mn_f32(a_lo + ao, p.cbA, blkA_bytes), desc_mn_f32(b_hi + bo, p.cbB, blkB_bytes), idesc, (it > k_beg || j > 0) ? 1u : 0u);
                        mma_tf32_ss(dcol, desc_mn_f32(a_hi + ao, p.cbA, blkA_bytes), desc_mn_f32(b_lo + bo, p.cbB, blkB_bytes), idesc, 1u);
                        mma_tf32_ss(dcol, desc_mn_f32(a_hi + ao, p.cbA, blkA_bytes), desc_mn_f32(b_hi + bo, p.cbB, blkB_bytes), idesc, 1u);
                    }
                    mma_commit(empty_bar + 8 * s);
                    if (it == k_end - 1) mma_commit(tmem_full + 8 * buf);
                }
                __syncwarp();
            }
        }
        if (n_steps == 0 && lane == 0) mbar_arrive(tmem_full);
        __syncwarp();
    } else {
        const int q = warp & 3, chalf = (warp - 2) >> 2;
        float part[4][32];                                        // this thread's 128 columns, summed over the chunks so far
#pragma unroll
        for (int cb = 0; cb < 4; ++cb)
#pragma unroll
            for (int e = 0; e < 32; ++e) part[cb][e] = 0.f;
        bool ok = true;
        for (int c = 0; c + 1 < n_chunks && ok; ++c) {
            const int buf = c & 1, use = c >> 1;
            ok = mbar_wait_bounded(tmem_full + 8 * buf, use & 1, status, ST_T_EPILOGUE);
            ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) {
                if (chalf * 128 + cb * 32 < p.n_tile_cols) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * TN + chalf * 128 + cb * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) part[cb][e] += __uint_as_float(v[e]);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty + 8 * buf);
        }
        const int last = n_chunks > 0 ? n_chunks - 1 : 0, lbuf = last & 1;
        if (ok) {
            ok = mbar_wait_bounded(tmem_full + 8 * lbuf, (last >> 1) & 1, status, ST_T_EPILOGUE);
            ok = __all_sync(0xffffffffu, ok && (*reinterpret_cast<volatile int*>(status) == 0));
        }
        tc_fence_after_sync();
        if (ok && n_steps > 0) {
            const int row = q * 32 + lane;
            const int blk = blockA0 + row / p.cbA;
            const int d = blk / bpcA, co = (blk % bpcA) * p.cbA + row % p.cbA;
            const bool row_ok = d < p.nc && co < p.Co;
            const size_t comp_stride = (size_t)p.Co * p.Ci;
            float* tap_base = dw32 + (size_t)tap * p.nc * comp_stride;
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) {
                const int col0 = chalf * 128 + cb * 32;
                if (col0 >= p.n_tile_cols) break;
                uint32_t v[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + lbuf * TN + col0, v);
                tmem_ld_wait();
                if (!row_ok) continue;
#pragma unroll
                for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) + part[cb][e]);
#pragma unroll
                for (int g4 = 0; g4 < 8; ++g4) {
                    const int col = col0 + g4 * 4;
                    if (col >= p.n_tile_cols) continue;
                    const int nblk = blockB0 + col / p.cbB;
                    const int l = nblk / bpcB, ci = (nblk % bpcB) * p.cbB + col % p.cbB;
                    if (l >= p.nc || ci >= p.Ci) continue;
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

// scratch [tap][r][co][ci] -> dw [r][co][ci][tap], or [r][ci][co] for dense layers (input-major, one tap)
__global__ void unpack_filter_grad_f32_kernel(const float* __restrict__ src, float* __restrict__ dw, int taps, int Co, int Ci, int dw_io, int nc) {
    const size_t per_tap = (size_t)nc * Co * Ci, total = per_tap * taps;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        if (dw_io) {
            const int co = (int)(idx % Co);
            const int ci = (int)((idx / Co) % Ci);
            const int r = (int)(idx / ((size_t)Co * Ci));
            dw[idx] = src[((size_t)r * Co + co) * Ci + ci];
        } else {
            const int tap = (int)(idx % taps);
            dw[idx] = src[(size_t)tap * per_tap + idx / taps];
        }
    }
}

struct Plan32 {
    int Cin, Cout, Hin, Win, Hout, Wout, pad_top, pad_left, SH, SW, ins_h, ins_w, Cp, Hp, Wp, Mp, Kp, LK;
    size_t xp_bytes, w_bytes;      // one of (hi, lo)
};

Plan32 make_plan32(Pass pass, const Geom& g) {
    Plan32 pl;
    if (pass == PASS_FWD) {
        pl.Cin = g.Ci; pl.Cout = g.Co; pl.Hin = g.H; pl.Win = g.W; pl.Hout = g.HO; pl.Wout = g.WO;
        pl.pad_top = g.PT; pl.pad_left = g.PL; pl.SH = g.SH; pl.SW = g.SW; pl.ins_h = pl.ins_w = 1;
    } else {
        pl.Cin = g.Co; pl.Cout = g.Ci; pl.Hin = g.HO; pl.Win = g.WO; pl.Hout = g.H; pl.Wout = g.W;
        pl.pad_top = (g.KH - 1) * g.DH - g.PT; pl.pad_left = (g.KW - 1) * g.DW - g.PL; pl.SH = 1; pl.SW = 1;
        pl.ins_h = g.SH; pl.ins_w = g.SW;
    }
    pl.LK = (pass == PASS_FWD && g.real_in) ? 1 : g.nc;
    pl.Cp = round_up(pl.Cin, 16);
    pl.Hp = (pl.Hout - 1) * pl.SH + (g.KH - 1) * g.DH + 1;
    pl.Wp = (pl.Wout - 1) * pl.SW + (g.KW - 1) * g.DW + 1;
    pl.Mp = round_up(g.nc * pl.Cout, TM);
    pl.Kp = pl.LK * pl.Cp;
    pl.xp_bytes = ((size_t)pl.LK * g.Nb * pl.Hp * pl.Wp * pl.Cp * 4 + 1023) / 1024 * 1024;
    pl.w_bytes = ((size_t)g.KH * g.KW * pl.Mp * pl.Kp * 4 + 1023) / 1024 * 1024;
    return pl;
}

struct FilterPlan32 {
    int Cop, Cip, Hp, Wp;
    size_t xp_bytes, dyp_bytes, acc_bytes;
};

FilterPlan32 make_filter_plan32(const Geom& g) {
    FilterPlan32 f;
    f.Cop = round_up(g.Co, 32);
    f.Cip = round_up(g.Ci, 32);
    f.Hp = (g.HO - 1) * g.SH + (g.KH - 1) * g.DH + 1;
    f.Wp = (g.WO - 1) * g.SW + (g.KW - 1) * g.DW + 1;
    f.xp_bytes = ((size_t)g.nc * g.Nb * f.Hp * f.Wp * f.Cip * 4 + 1023) / 1024 * 1024;
    f.dyp_bytes = ((size_t)g.nc * g.Nb * g.HO * g.WO * f.Cop * 4 + 1023) / 1024 * 1024;
    f.acc_bytes = ((size_t)g.nc * g.Co * g.Ci * g.KH * g.KW * 4 + 1023) / 1024 * 1024;
    return f;
}

bool common_ok(int dtype, int variant, const Geom& g) {
    if (dtype != PCB_F32 || variant != PCB_VARIANT_16_PRODUCT) return false;
    if (g.SH > 2 || g.SW > 2) return false;
    if (g.w_io && g.KH * g.KW != 1) return false;
    return true;
}

}  // namespace

bool conv_tf32_supported(Pass pass, int dtype, int variant, const Geom& g) {
    if (!common_ok(dtype, variant, g)) return false;
    if (pass == PASS_BWD_FILTER) {
        if (g.real_in) return false;
        const FilterPlan32 f = make_filter_plan32(g);
        return f.Hp <= 65535 && f.Wp <= 65535 && 2 * (f.xp_bytes + f.dyp_bytes) <= ((size_t)16 << 30);
    }
    if (g.real_in && pass != PASS_FWD) return false;
    if (pass == PASS_BWD_DATA && ((g.KH - 1) * g.DH < g.PT || (g.KW - 1) * g.DW < g.PL)) return false;
    const Plan32 pl = make_plan32(pass, g);
    return pl.Hp <= 65535 && pl.Wp <= 65535 && 2 * pl.xp_bytes <= ((size_t)16 << 30);
}

size_t conv_tf32_scratch_bytes(Pass pass, const Geom& g) {
    if (pass == PASS_BWD_FILTER) {
        const FilterPlan32 f = make_filter_plan32(g);
        return 2 * (f.xp_bytes + f.dyp_bytes) + f.acc_bytes;
    }
    const Plan32 pl = make_plan32(pass, g);
    return 2 * (pl.xp_bytes + pl.w_bytes);
}

static int conv_tf32_filter_launch(const Geom& g, const float* dy, const float* x, float* dw, void* scratch, int* status, cudaStream_t stream) {
    const FilterPlan32 f = make_filter_plan32(g);
    const int taps = g.KH * g.KW;
    uint8_t* s8 = static_cast<uint8_t*>(scratch);
    float* x_hi = reinterpret_cast<float*>(s8);
    float* x_lo = reinterpret_cast<float*>(s8 + f.xp_bytes);
    float* y_hi = reinterpret_cast<float*>(s8 + 2 * f.xp_bytes);
    float* y_lo = reinterpret_cast<float*>(s8 + 2 * f.xp_bytes + f.dyp_bytes);
    float* acc = reinterpret_cast<float*>(s8 + 2 * f.xp_bytes + 2 * f.dyp_bytes);
    stage_activations_f32(x, x_hi, x_lo, g.nc * g.Nb, g.Ci, g.H, g.W, f.Hp, f.Wp, f.Cip, g.PT, g.PL, 1, 1, 32, g.Nb, stream);
    stage_activations_f32(dy, y_hi, y_lo, g.nc * g.Nb, g.Co, g.HO, g.WO, g.HO, g.WO, f.Cop, 0, 0, 1, 1, 32, g.Nb, stream);
    PCB_CUDA_TRY(cudaGetLastError());
    PCB_CUDA_TRY(cudaMemsetAsync(acc, 0, (size_t)g.nc * g.Co * g.Ci * taps * sizeof(float), stream));

    TFParams p;
    p.nc = g.nc; p.ga = g.ga; p.neg = g.neg;
    p.Nb = g.Nb; p.Co = g.Co; p.Ci = g.Ci; p.HO = g.HO; p.WO = g.WO; p.Cop = f.Cop; p.Cip = f.Cip;
    p.cbA = 32; p.cbB = 32;
    p.KH = g.KH; p.KW = g.KW; p.SH = g.SH; p.SW = g.SW; p.DH = g.DH; p.DW = g.DW;
    {
        long long best = -1;
        for (int pw = 1; pw <= TFK; pw *= 2)
            for (int ph = 1; ph * pw <= TFK; ph *= 2) {
                const int pn = TFK / (pw * ph);
                const long long vol = (long long)round_up(g.WO, pw) * round_up(g.HO, ph) * round_up(g.Nb, pn);
                if (best < 0 || vol < best || (vol == best && pw > p.PW)) { best = vol; p.PW = pw; p.PH = ph; p.PN = pn; }
            }
    }
    p.tiles_w = (g.WO + p.PW - 1) / p.PW; p.tiles_h = (g.HO + p.PH - 1) / p.PH; p.tiles_n = (g.Nb + p.PN - 1) / p.PN;
    const int m_cols = g.nc * f.Cop, n_cols = g.nc * f.Cip;
    p.m_tiles = (m_cols + TM - 1) / TM;
    p.n_tiles = (n_cols + TN - 1) / TN;
    p.n_tile_cols = n_cols < TN ? n_cols : TN;
    const int steps_total = p.tiles_w * p.tiles_h * p.tiles_n;
    const int items = taps * p.m_tiles * p.n_tiles;
    int splits = split_count(items, sm_count());
    if (splits > steps_total) splits = steps_total;
    if (splits < 1) splits = 1;
    p.steps_per_split = (steps_total + splits - 1) / splits;
    p.splits = (steps_total + p.steps_per_split - 1) / p.steps_per_split;

    auto swz = [](int) { return CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B; };
    alignas(64) CUtensorMap m_dy_hi, m_dy_lo, m_x_hi, m_x_lo;
    {
        // staged tensors: [component * blocks per component + channel block][image][h][w][32 channels]; the last box extent
        // is the number of channel blocks of a tile (blocks past the end read as zeros)
        const cuuint64_t dims[5] = {(cuuint64_t)p.cbA, (cuuint64_t)g.WO, (cuuint64_t)g.HO, (cuuint64_t)g.Nb, (cuuint64_t)(g.nc * (f.Cop / p.cbA))};
        const cuuint64_t strides[4] = {(cuuint64_t)p.cbA * 4, (cuuint64_t)g.WO * p.cbA * 4, (cuuint64_t)g.HO * g.WO * p.cbA * 4,
                                       (cuuint64_t)g.Nb * g.HO * g.WO * p.cbA * 4};
        const cuuint32_t box[5] = {(cuuint32_t)p.cbA, (cuuint32_t)p.PW, (cuuint32_t)p.PH, (cuuint32_t)p.PN, (cuuint32_t)(TM / p.cbA)};
        int rc = make_tensor_map(&m_dy_hi, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, y_hi, 5, dims, strides, box, nullptr, swz(p.cbA), "dy hi");
        if (rc == PCB_OK) rc = make_tensor_map(&m_dy_lo, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, y_lo, 5, dims, strides, box, nullptr, swz(p.cbA), "dy lo");
        if (rc != PCB_OK) return rc;
    }
    {
        const cuuint64_t dims[5] = {(cuuint64_t)p.cbB, (cuuint64_t)f.Wp, (cuuint64_t)f.Hp, (cuuint64_t)g.Nb, (cuuint64_t)(g.nc * (f.Cip / p.cbB))};
        const cuuint64_t strides[4] = {(cuuint64_t)p.cbB * 4, (cuuint64_t)f.Wp * p.cbB * 4, (cuuint64_t)f.Hp * f.Wp * p.cbB * 4,
                                       (cuuint64_t)g.Nb * f.Hp * f.Wp * p.cbB * 4};
        const cuuint32_t box[5] = {(cuuint32_t)p.cbB, (cuuint32_t)((p.PW - 1) * g.SW + 1), (cuuint32_t)((p.PH - 1) * g.SH + 1), (cuuint32_t)p.PN,
                                   (cuuint32_t)(p.n_tile_cols / p.cbB)};
        const cuuint32_t es[5] = {1, (cuuint32_t)g.SW, (cuuint32_t)g.SH, 1, 1};
        int rc = make_tensor_map(&m_x_hi, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, x_hi, 5, dims, strides, box, es, swz(p.cbB), "x hi");
        if (rc == PCB_OK) rc = make_tensor_map(&m_x_lo, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, x_lo, 5, dims, strides, box, es, swz(p.cbB), "x lo");
        if (rc != PCB_OK) return rc;
    }
    constexpr size_t smem = 1024 + T_STAGES * TF_STAGE + 512;
    PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_filter_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    qconv_filter_tf32_kernel<<<items * p.splits, T_THREADS, smem, stream>>>(m_dy_hi, m_dy_lo, m_x_hi, m_x_lo, p, acc, status);
    PCB_CUDA_TRY(cudaGetLastError());
    unpack_filter_grad_f32_kernel<<<grid_cap((size_t)g.nc * g.Co * g.Ci * taps, 256, 16), 256, 0, stream>>>(acc, dw, taps, g.Co, g.Ci, g.dw_io, g.nc);
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

int conv_tf32_launch(Pass pass, const Geom& g, const void* a, const void* b, const void* bias, void* out, void* scratch, int* status,
                     cudaStream_t stream) {
    // operand roles as for the other launchers: forward/backward-data a = filters, b = activations; backward-filter a = dy, b = x
    if (pass == PASS_BWD_FILTER) return conv_tf32_filter_launch(g, (const float*)a, (const float*)b, (float*)out, scratch, status, stream);
    const Plan32 pl = make_plan32(pass, g);
    const int taps = g.KH * g.KW;
    uint8_t* s8 = static_cast<uint8_t*>(scratch);
    float* x_hi = reinterpret_cast<float*>(s8);
    float* x_lo = reinterpret_cast<float*>(s8 + pl.xp_bytes);
    float* w_hi = reinterpret_cast<float*>(s8 + 2 * pl.xp_bytes);
    float* w_lo = reinterpret_cast<float*>(s8 + 2 * pl.xp_bytes + pl.w_bytes);
    stage_activations_f32((const float*)b, x_hi, x_lo, pl.LK * g.Nb, pl.Cin, pl.Hin, pl.Win, pl.Hp, pl.Wp, pl.Cp, pl.pad_top, pl.pad_left, pl.ins_h,
                          pl.ins_w, 0, 1, stream);
    pack_filters_f32_kernel<<<grid_cap((size_t)taps * pl.Mp, 1, 8), pl.Kp >= 256 ? 256 : 128, 0, stream>>>(
        (const float*)a, w_hi, w_lo, g.Co, g.Ci, taps, pl.Mp, pl.Kp, pl.Cp, pass == PASS_BWD_DATA ? 1 : 0, g.w_io, g.nc, g.ga, g.neg);
    PCB_CUDA_TRY(cudaGetLastError());

    TParams p;
    {
        long long best = -1;
        for (int pw = 1; pw <= 128; pw *= 2)
            for (int ph = 1; ph * pw <= 256; ph *= 2) {
                const int pn = 256 / (pw * ph);
                if (pn > 256 || (pw - 1) * pl.SW + 1 > 256 || (ph - 1) * pl.SH + 1 > 256) continue;
                if (pw < 8 && pl.Wout >= 8) continue;                      // narrow boxes only for narrow planes
                const long long vol = (long long)round_up(pl.Wout, pw) * round_up(pl.Hout, ph) * round_up(g.Nb, pn);
                if (best < 0 || vol < best || (vol == best && pw > p.PW)) { best = vol; p.PW = pw; p.PH = ph; p.PN = pn; }
            }
    }
    p.Nb = g.Nb; p.Cout = pl.Cout; p.Mvalid = g.nc * pl.Cout; p.HO = pl.Hout; p.WO = pl.Wout; p.Cp = pl.Cp;
    p.KH = g.KH; p.KW = g.KW; p.SH = pl.SH; p.SW = pl.SW; p.DH = g.DH; p.DW = g.DW;
    p.tiles_w = (pl.Wout + p.PW - 1) / p.PW; p.tiles_h = (pl.Hout + p.PH - 1) / p.PH; p.tiles_n = (g.Nb + p.PN - 1) / p.PN;
    p.tiles_m = pl.Mp / TM;
    p.has_bias = (pass == PASS_FWD && g.has_bias) ? 1 : 0;
    p.LK = pl.LK;
    p.store_vec = 1;
    while (p.store_vec < 8 && pl.Wout % (p.store_vec * 2) == 0 && (reinterpret_cast<uintptr_t>(out) % (size_t)(p.store_vec * 8)) == 0) p.store_vec *= 2;

    alignas(64) CUtensorMap m_w_hi, m_w_lo, m_x_hi, m_x_lo;
    {
        const cuuint64_t dims[3] = {(cuuint64_t)pl.Kp, (cuuint64_t)pl.Mp, (cuuint64_t)taps};
        const cuuint64_t strides[2] = {(cuuint64_t)pl.Kp * 4, (cuuint64_t)pl.Mp * pl.Kp * 4};
        const cuuint32_t box[3] = {TKS, TM, 1};
        int rc = make_tensor_map(&m_w_hi, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, w_hi, 3, dims, strides, box, nullptr, CU_TENSOR_MAP_SWIZZLE_64B, "filters hi");
        if (rc == PCB_OK) rc = make_tensor_map(&m_w_lo, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, w_lo, 3, dims, strides, box, nullptr, CU_TENSOR_MAP_SWIZZLE_64B, "filters lo");
        if (rc != PCB_OK) return rc;
    }
    {
        const cuuint64_t dims[5] = {(cuuint64_t)pl.Cp, (cuuint64_t)pl.Wp, (cuuint64_t)pl.Hp, (cuuint64_t)g.Nb, (cuuint64_t)pl.LK};
        const cuuint64_t strides[4] = {(cuuint64_t)pl.Cp * 4, (cuuint64_t)pl.Wp * pl.Cp * 4, (cuuint64_t)pl.Hp * pl.Wp * pl.Cp * 4,
                                       (cuuint64_t)g.Nb * pl.Hp * pl.Wp * pl.Cp * 4};
        const cuuint32_t box[5] = {TKS, (cuuint32_t)((p.PW - 1) * pl.SW + 1), (cuuint32_t)((p.PH - 1) * pl.SH + 1), (cuuint32_t)p.PN, 1};
        const cuuint32_t es[5] = {1, (cuuint32_t)pl.SW, (cuuint32_t)pl.SH, 1, 1};
        int rc = make_tensor_map(&m_x_hi, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, x_hi, 5, dims, strides, box, es, CU_TENSOR_MAP_SWIZZLE_64B, "activations hi");
        if (rc == PCB_OK) rc = make_tensor_map(&m_x_lo, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, x_lo, 5, dims, strides, box, es, CU_TENSOR_MAP_SWIZZLE_64B, "activations lo");
        if (rc != PCB_OK) return rc;
    }
    const int n_tiles = p.tiles_w * p.tiles_h * p.tiles_n * p.tiles_m;
    const int n_k = taps * pl.LK * (pl.Cp / TKS);
    // Too few tiles for the SMs (dense layers, small planes): cut the K loop of every tile into work items of at least one chunk
    // each; their partial sums meet in the output, zeroed first, by fp32 reductions (the order of which is not fixed).
    p.splits = 1;
    if (2 * n_tiles <= sm_count() && n_k >= 2 * T_CHUNK) {
        p.splits = sm_count() / n_tiles;
        if (p.splits > n_k / T_CHUNK) p.splits = n_k / T_CHUNK;
        while (n_k % p.splits != 0) --p.splits;                      // equal work items: every chunk of every item holds stages
    }
    p.k_per_split = n_k / p.splits;
    if (p.splits > 1) PCB_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)g.nc * g.Nb * pl.Cout * pl.Hout * pl.Wout * sizeof(float), stream));
    const int n_items = n_tiles * p.splits;
    const int grid = n_items < sm_count() ? n_items : sm_count();
    p.n_chunks = (p.k_per_split + T_CHUNK - 1) / T_CHUNK;
    p.chunk_len = (p.k_per_split + p.n_chunks - 1) / p.n_chunks;
    if (p.n_chunks > 1) {
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_general_tf32_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T_SMEM));
        qconv_general_tf32_kernel<true><<<grid, T_THREADS, T_SMEM, stream>>>(m_w_hi, m_w_lo, m_x_hi, m_x_lo, p, (const float*)bias, (float*)out, status);
    } else {
        PCB_CUDA_TRY(cudaFuncSetAttribute(qconv_general_tf32_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T_SMEM));
        qconv_general_tf32_kernel<false><<<grid, T_THREADS, T_SMEM, stream>>>(m_w_hi, m_w_lo, m_x_hi, m_x_lo, p, (const float*)bias, (float*)out, status);
    }
    PCB_CUDA_TRY(cudaGetLastError());
    return PCB_OK;
}

}  // namespace pcb
