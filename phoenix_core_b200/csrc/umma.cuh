// Thin inline-PTX layer over the Blackwell (sm_100a) primitives the tensor-core kernels use:
// mbarriers with BOUNDED waits, tensor memory (TMEM) allocation, tcgen05.mma / commit / ld, proxy fences,
// and the 64-bit shared-memory matrix descriptors and 32-bit instruction descriptor of tcgen05.mma.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace pcb {
namespace umma {

// ---------------------------------------------------------------------------------------------------
// Shared-memory operand layouts (16-bit element types; 8 elements per 16-byte chunk).
//
// K-major, 128-byte swizzle: a tile is R rows (M or N index) by 64 K-elements. Row r occupies the 128
// bytes at r*128; its 16-byte chunk c (K elements 8c..8c+7) is stored at chunk position c ^ (r % 8).
// Groups of 8 rows (1024 bytes) follow each other: stride-byte-offset = 1024. One MMA consumes 16
// K-elements = 32 bytes, so the descriptor start address advances by 32 bytes per K step.
//
// MN-major, 128-byte swizzle: a tile is 64 K-rows by blocks of 64 M/N-elements. Within a block, K-row k
// occupies the 128 bytes at k*128 and its chunk c (M/N elements 8c..8c+7) sits at position c ^ (k % 8).
// Groups of 8 K-rows are 1024 bytes apart (stride-byte-offset), blocks of 64 M/N elements are
// `block_bytes` apart (leading-byte-offset). One MMA consumes 16 K-rows = 2048 bytes.
//
// Tiles must start on a 1024-byte boundary: the swizzle is a function of the shared-memory address bits.
// ---------------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint32_t kmajor_sw128_offset(int row, int chunk) {
    return (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}
__host__ __device__ __forceinline__ uint32_t mnmajor_sw128_offset(int k, int mn_chunk, uint32_t block_bytes) {
    return (uint32_t)(mn_chunk >> 3) * block_bytes + (uint32_t)k * 128u + (uint32_t)(((mn_chunk & 7) ^ (k & 7)) << 4);
}

constexpr uint64_t DESC_VERSION_SM100 = 1ull << 46;
constexpr uint64_t DESC_SWIZZLE_128B = 2ull << 61;

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | DESC_VERSION_SM100 | DESC_SWIZZLE_128B;
}
// K-major SW128 tile at `smem_addr`; the leading offset is not used by the hardware for this layout.
__device__ __forceinline__ uint64_t make_desc_kmajor(uint32_t smem_addr) { return make_desc(smem_addr, 16, 1024); }
// MN-major SW128 tile at `smem_addr` whose 64-element blocks are `block_bytes` apart.
__device__ __forceinline__ uint64_t make_desc_mnmajor(uint32_t smem_addr, uint32_t block_bytes) {
    return make_desc(smem_addr, block_bytes, 1024);
}

// Instruction descriptor of tcgen05.mma.kind::f16 with fp32 accumulation.
//   fmt: 0 = f16, 1 = bf16, 2 = tf32 (with kind::tf32).  a_mn / b_mn: operand is MN-major.  a_neg / b_neg: negate the operand.
__host__ __device__ __forceinline__ uint32_t make_idesc_f16(int fmt, int M, int N, bool a_mn, bool b_mn,
                                                           bool a_neg = false, bool b_neg = false) {
    return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)a_neg << 13) | ((uint32_t)b_neg << 14) |
           ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier --------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity to complete, for at most `limit` SM clocks (default ~2^31, about a
// second). On expiry ORs `code` into *status and returns false; the caller then skips its remaining work and
// proceeds to the common teardown, so a lost signal can never hang the GPU. Kernels only ever OR into the status
// word: it is cleared once per API call by the host, so an expiry in an earlier launch of the call stays visible
// (and makes the later launches of that call give up at their first slow wait).
constexpr long long WAIT_LIMIT_CLOCKS = 1ll << 31;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int* status, int code,
                                                  long long limit = WAIT_LIMIT_CLOCKS) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*reinterpret_cast<volatile int*>(status) != 0) return false;   // another wait of this launch already expired
        if (clock64() - t0 > limit) {
            atomicOr(status, code);
            return false;
        }
    }
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// Makes generic-proxy shared-memory writes visible to the async proxy (tcgen05.mma, TMA).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- tensor memory ---------------------------------------------------------------------------------
// Allocates `cols` (power of two >= 32) TMEM columns; executed by one full warp. The base address is
// written to *slot in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem_addr, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem_addr), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t tmem_addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread. accumulate == 0 overwrites D.
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same instruction with each 64-bit descriptor given as its two 32-bit words, so that the issuing thread can step the
// address field (low word) of a prebuilt descriptor with one 32-bit addition.
__device__ __forceinline__ void mma_f16_ss_words(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
// Same with fp32 operands read as TF32 (the 13 low mantissa bits are not used), 8 K-elements per instruction.
__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Loads 32 consecutive fp32 columns of this thread's TMEM lane (lane = 32 * (warp % 4) + lane id).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
// Loads 16 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
}
// Loads 64 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld_32x32b_x64(uint32_t taddr, uint32_t (&v)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]), "=r"(v[32]), "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]), "=r"(v[40]), "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]), "=r"(v[48]), "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]), "=r"(v[56]), "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The registers written by a tcgen05.ld hold data only after tcgen05.wait::ld, a dependency the compiler cannot see
// when other work sits between the two. This empty statement is ordered after the wait (both are volatile) and
// "rewrites" every register, so no use of the values can move above the wait.
template <int N>
__device__ __forceinline__ void tmem_regs_ready(uint32_t (&v)[N]) {
#pragma unroll
    for (int i = 0; i < N; ++i) asm volatile("" : "+r"(v[i]));
}

}  // namespace umma
}  // namespace pcb
