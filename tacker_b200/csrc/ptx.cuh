// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (bulk tensor copies without
// any cluster broadcast), tcgen05 (TMEM allocation, UMMA issue, commit, TMEM loads)
// and named barriers.  Every wait is bounded: it gives up after a clock budget or
// when another role of the CTA has raised the abort flag, and reports why.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tk {

// ---- device status word ------------------------------------------------------
// 0 = ok.  The first bounded wait that expires stores its code below (and nothing else: a later expiry does not
// overwrite it); the host reads and clears the word.
enum : unsigned {
    DEV_OK = 0,
    DEV_TIMEOUT_EMPTY = 1,      // producer waited for a free smem stage
    DEV_TIMEOUT_FULL = 2,       // MMA issuer waited for TMA bytes
    DEV_TIMEOUT_TMEM_EMPTY = 3, // MMA issuer waited for the epilogue to drain an accumulator
    DEV_TIMEOUT_TMEM_FULL = 4,  // epilogue waited for the accumulator
    DEV_TMEM_ALLOC = 5,
};

// Clock budget of every bounded wait: about one second at 2 GHz unless the host stores another value (a test
// shortens it to make a wait run out quickly).
__device__ long long g_wait_budget_cycles = 2000000000ll;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
    uint32_t l;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
    return l;
}

// ---- named barriers ------------------------------------------------------------
// Each role of a fused CTA synchronises only its own threads (the idea behind the
// reference's `bar.sync id, nthreads`, src/mix_kernel/tzgemm_stencil.cu:113,203).
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- mbarrier -------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_inval(uint32_t bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the budget ran out or `abort_flag` (shared
// memory, written by any role that gave up) is set; on expiry the first failing
// site is recorded in *status and the abort flag is raised for the other roles.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          unsigned* status, unsigned code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 63u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > *const_cast<volatile long long*>(&g_wait_budget_cycles)) {
                *abort_flag = 1u;
                atomicCAS(status, 0u, code);
                return false;
            }
        }
    }
}

// ---- TMA: 2-D tiled load global -> shared, completion on an mbarrier -------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tmap, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// operand tiles of the GEMM: tensor maps are {K, rows, batch}, the box is one K-block x rows x 1
__device__ __forceinline__ void tma_load_tile(uint32_t dst_smem, const void* tmap, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// L2 eviction-priority policies for bulk loads: operands that are re-read by other CTAs (GEMM tiles) are
// kept, data that is streamed once (stencil planes) is marked to go first.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma_load_tile_hint(uint32_t dst_smem, const void* tmap, uint32_t bar, int x, int y,
                                                   int z, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4, %5}], [%2], %6;"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z), "l"(policy)
        : "memory");
}

// C += partial for the K-split GEMM: one 16-byte reduction, no value returned
__device__ __forceinline__ void red_add_v4(float* addr, const float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}

// ---- tcgen05 ---------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t result_slot_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_slot_smem),
                 "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem], fp16 inputs, fp32 accumulate, issued by one thread.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The mbarrier gets one arrival once every UMMA issued so far by this thread has retired.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane
// (lane base + t), columns [col, col + 32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- UMMA descriptors ---------------------------------------------------------------
// Shared-memory operand descriptor for a K-major tile whose rows are 128 bytes
// (64 fp16) stored with the 128-byte swizzle TMA writes: 8-row groups are 1024
// bytes apart (stride byte offset), the leading byte offset is unused.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);       // bits 0-13: start address / 16
    d |= static_cast<uint64_t>(1024u >> 4) << 32;                   // bits 32-45: stride byte offset / 16
    d |= 1ull << 46;                                                // bits 46-48: descriptor version (sm_100)
    d |= 2ull << 61;                                                // bits 61-63: 128-byte swizzle
    return d;
}

// Instruction descriptor, kind::f16: fp16 A and B (both K-major), fp32 accumulator.
__host__ __device__ constexpr uint32_t umma_idesc_f16_f32(uint32_t m, uint32_t n) {
    return (1u << 4)            // bits 4-5: accumulator format, 1 = fp32
           | (0u << 7)          // bits 7-9: A format, 0 = fp16
           | (0u << 10)         // bits 10-12: B format, 0 = fp16
           | (0u << 15)         // bit 15: A major, 0 = K
           | (0u << 16)         // bit 16: B major, 0 = K
           | ((n >> 3) << 17)   // bits 17-22: N / 8
           | ((m >> 4) << 24);  // bits 24-28: M / 16
}

}  // namespace tk
