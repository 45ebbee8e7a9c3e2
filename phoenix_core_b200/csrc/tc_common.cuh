// Helpers shared by the TMA-fed tcgen05 kernels: TMA load wrappers, wide stores, the tensor-map encoder
// (fetched from the driver at run time, so the library does not link against libcuda), small host utilities.
#pragma once
#include <cstdlib>

#include <cuda.h>

#include "common.cuh"
#include "umma.cuh"

namespace pcb {
extern int g_sm_margin;      // defined in api.cu
namespace tc {

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar) : "memory");
}

// TMA store of one shared-memory box (written by ordinary stores, then fence_proxy_async) to global memory; elements of
// the box that fall outside the tensor are not written. Completion is tracked per thread in bulk groups.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// Bulk copy of a contiguous shared-memory range to global memory (both 16-byte aligned, size a multiple of 16 bytes).
__device__ __forceinline__ void bulk_store_1d(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until the bulk stores committed so far by this thread have finished READING shared memory (the buffer may be reused).
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_u16(uint32_t addr, uint16_t v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// 32-byte store: one full sector per thread and half as many store instructions as 16-byte stores.
__device__ __forceinline__ void st_global_v8(void* addr, const uint32_t* v) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}
__device__ __forceinline__ void red_add_f32x4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Staging copy of NCHW activations for the TMA-fed kernels, fast form (no zero insertion, W a multiple of PX = 4 or 2,
// rows aligned to PX elements): one thread moves 8 channels x PX pixels -- eight loads of 2 PX bytes and PX 16-byte stores. Destination: channels-last xp[plane][hp][wp][Cp] (planar == 0),
// planar xp[plane][c / 8][hp][wp][8] (planar == 1), or -- cb > 0 -- blocks of cb channels with the block index outermost,
// xp[comp * (Cp / cb) + c / cb][img][hp][wp][cb] where plane = comp * Nb + img (one TMA box can then span the channel
// blocks of several components). Zero outside the image and for c >= C. The threads at the ends of a row also write
// the padding columns.
template <typename T, int PX>
__global__ void pack_rows_kernel(const T* __restrict__ x, T* __restrict__ xp, int planes, int C, int H, int W, int Hp, int Wp, int groups,
                                 int pad_top, int pad_left, int planar, int cb = 0, int Nb = 1) {
    const int Wq = W / PX;
    const unsigned total = (unsigned)planes * groups * Hp * Wq;         // 32-bit indices: staged copies stay below 2^32 / 8 threads
    const int Cp = groups * 8;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        // The channel group runs fastest across threads: the lanes of a warp that share a pixel group then write the channel
        // groups of a pixel side by side (whole 32- to 128-byte runs per pixel instead of one 16-byte piece per lane and
        // 32 half-filled sectors per store), while every load instruction still fetches full 32-byte sectors (PX * 2 bytes
        // from each of the neighbouring pixel groups of one channel row).
        const int grp = (int)(idx % groups);
        unsigned rest = idx / groups;
        const int q = (int)(rest % Wq); rest /= Wq;
        const int hp = (int)(rest % Hp);
        const int plane = (int)(rest / Hp);
        const int ih = hp - pad_top;
        const bool row_in = ih >= 0 && ih < H;
        alignas(8) T v[8][PX];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int c = grp * 8 + e;
            if (PX == 4) {
                uint2 raw = make_uint2(0u, 0u);
                if (row_in && c < C) raw = __ldg(reinterpret_cast<const uint2*>(x + (((size_t)plane * C + c) * H + ih) * W + 4 * q));
                *reinterpret_cast<uint2*>(v[e]) = raw;
            } else {
                uint32_t raw = 0u;
                if (row_in && c < C) raw = __ldg(reinterpret_cast<const uint32_t*>(x + (((size_t)plane * C + c) * H + ih) * W + 2 * q));
                *reinterpret_cast<uint32_t*>(v[e]) = raw;
            }
        }
        size_t blk_plane = 0;                       // (block, image) index and channel offset inside the block
        int c_lo = 0;
        if (cb > 0) {
            const int comp = plane / Nb, img = plane - comp * Nb, b = (grp * 8) / cb;
            c_lo = grp * 8 - b * cb;
            blk_plane = ((size_t)comp * (Cp / cb) + b) * Nb + img;
        }
        auto dst = [&](int wp) {
            if (cb > 0) return xp + ((blk_plane * Hp + hp) * Wp + wp) * cb + c_lo;
            return planar ? xp + ((((size_t)plane * groups + grp) * Hp + hp) * Wp + wp) * 8 : xp + (((size_t)plane * Hp + hp) * Wp + wp) * Cp + grp * 8;
        };
#pragma unroll
        for (int j = 0; j < PX; ++j) {
            alignas(16) T o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = v[e][j];
            *reinterpret_cast<uint4*>(dst(pad_left + PX * q + j)) = *reinterpret_cast<const uint4*>(o);
        }
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        if (q == 0)
            for (int wp = 0; wp < pad_left && wp < Wp; ++wp) *reinterpret_cast<uint4*>(dst(wp)) = zero;
        if (q == Wq - 1)
            for (int wp = pad_left + W; wp < Wp; ++wp) *reinterpret_cast<uint4*>(dst(wp)) = zero;
    }
}
// A side stream per host thread and device, for a prologue kernel that is independent of its neighbour: the filter matrix
// is packed beside the staging of the activations instead of after it (both are short, one bound by memory, the other by
// latency). fork() orders the side stream after everything enqueued so far on the caller's stream and returns it; join()
// makes the caller's stream wait for it. Where the side stream cannot be made the caller's stream is returned and join()
// does nothing. The fork / join pattern is also what stream capture expects.
struct SideStream {
    cudaStream_t side = nullptr;
    cudaEvent_t forked = nullptr, joined = nullptr;
    bool tried = false;
    cudaStream_t fork(cudaStream_t main) {
        if (!tried) {
            tried = true;
            const char* off = getenv("PCB_NO_SIDE_STREAM");      // escape hatch: everything on the caller's stream
            if (off && off[0] && off[0] != '0') return main;
            if (cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking) != cudaSuccess) side = nullptr;
            if (side && (cudaEventCreateWithFlags(&forked, cudaEventDisableTiming) != cudaSuccess ||
                         cudaEventCreateWithFlags(&joined, cudaEventDisableTiming) != cudaSuccess)) side = nullptr;
            if (!side) (void)cudaGetLastError();
        }
        if (!side) return main;
        if (cudaEventRecord(forked, main) != cudaSuccess || cudaStreamWaitEvent(side, forked, 0) != cudaSuccess) { (void)cudaGetLastError(); return main; }
        return side;
    }
    void join(cudaStream_t main, cudaStream_t used) {
        if (used == main) return;
        cudaEventRecord(joined, used);
        cudaStreamWaitEvent(main, joined, 0);
    }
};
inline SideStream& side_stream() {
    static thread_local SideStream per_device[16];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) dev = 0;
    return per_device[dev];
}

// Pixels per thread pack_rows_kernel can take for this tensor: 4, 2, or 0 (the general staging kernel must run).
inline int pack_rows_px(const void* x, int W, int Wp, int pad_left, int ins_h, int ins_w) {
    if (ins_h != 1 || ins_w != 1 || pad_left < 0 || pad_left + W > Wp) return 0;
    if (W % 4 == 0 && W >= 4 && reinterpret_cast<uintptr_t>(x) % 8 == 0) return 4;
    if (W % 2 == 0 && W >= 2 && reinterpret_cast<uintptr_t>(x) % 4 == 0) return 2;
    return 0;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// Encodes a tiled tensor map with zero out-of-bounds fill; returns a pcb_status.
inline int make_tensor_map(CUtensorMap* map, CUtensorMapDataType dt, const void* ptr, int rank, const cuuint64_t* dims,
                           const cuuint64_t* strides_bytes, const cuuint32_t* box, const cuuint32_t* elem_strides,
                           CUtensorMapSwizzle swizzle, const char* what) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return PCB_ERR_CUDA; }
    const cuuint32_t ones[5] = {1, 1, 1, 1, 1};
    const CUresult r = fn(map, dt, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides_bytes, box, elem_strides ? elem_strides : ones,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (%s) failed with code %d", what, (int)r); return PCB_ERR_CUDA; }
    return PCB_OK;
}

// SMs the persistent kernels size their grids for: the device's count minus the margin set through pcb_set_sm_margin (SMs left
// free so that another kernel, e.g. a collective's, can run beside them), never fewer than two.
inline int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    const int left = sms - pcb::g_sm_margin;
    return left < 2 ? 2 : left;
}

inline int round_up(int v, int m) { return (v + m - 1) / m * m; }
// Number of slices to cut each of `items` work items into when every CTA occupies a whole SM: the CTAs must fill
// one, two or three rounds of the machine as exactly as possible (one CTA more than a round costs a whole round). A further
// round also costs every CTA's fixed part again (tensor-memory allocation, pipeline fill, the atomic fold of its
// accumulator), so it has to fill the machine at least 5 % better to be taken.
inline int split_count(int items, int sms) {
    int best = 1;
    double best_util = 0.0;
    for (int waves = 1; waves <= 3; ++waves) {
        const int splits = waves * sms / items;
        if (splits < 1) continue;
        const double util = (double)items * splits / ((double)waves * sms);
        if (util > best_util + (best_util > 0.0 ? 0.05 : 0.0)) { best_util = util; best = splits; }
    }
    return best;
}
inline int grid_cap(size_t work_items, int per_block, int blocks_per_sm) {
    const size_t want = (work_items + per_block - 1) / per_block, cap = (size_t)sm_count() * blocks_per_sm;
    return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace tc
}  // namespace pcb
