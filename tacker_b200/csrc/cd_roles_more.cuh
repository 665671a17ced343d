// Four more CUDA-core roles with the persistent-thread-block contract of cd_roles.cuh: the Parboil kernels the
// reference pairs with tzgemm besides stencil / cp / mriq / mrif --
//   sgemm  C = 2 C + 2 A B, fp32          (src/gptb_kernel/sgemm_kernel.cu:3-64)
//   lbm    one D3Q19 lattice-Boltzmann step (src/gptb_kernel/lbm_kernel.cu:3-177, src/header/lbm_header.h)
//   fft    batches of 256-point transforms (src/gptb_kernel/fft_kernel.cu:3-80, src/header/fft_header.h)
//   cutcp  cutoff Coulomb potential, binned atoms (src/gptb_kernel/cutcp_kernel.cu:12-183)
// Each takes the block range [start, end) of the ORIGINAL launch and produces, block for block, what the
// reference's kernel writes for it.  The work unit is a warp, not a 128-thread block: a role may be given any
// number of warps (solo: the whole CTA; fused: the warps behind the tensor role), warps never meet on a barrier
// except once at the start of the FFT role, and every role runs on 64 .. 128 registers.
//
// Arithmetic follows the reference expression by expression, so that the same compiler contracts the same
// multiply-adds: the results are the reference's to the last bit wherever the order of operations is fixed by the
// algorithm (all four are: no reductions across threads).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "cd_roles.cuh"
#include "ptx.cuh"

namespace tk {

// role-wide barrier: `count` threads on hardware barrier `id` (0 = the CTA's own barrier when the role is the CTA)
__device__ __forceinline__ void role_sync(uint32_t id, uint32_t count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// =====================================================================================
// sgemm.  Layouts of the reference: A [K][M], B [K][N], C [N][M].  Original block (bx, by) of the (M / 128, N / 16)
// grid = rows 128 bx .., columns 16 by ...  A warp computes half a block (64 rows x 16 columns): lane l holds rows
// 2 l, 2 l + 1 of all 16 columns (32 accumulators).  The warp streams its slices of the A and B panels through a ring
// of its own in shared memory, eight k-steps (2 KB of A, 512 bytes of B) per slot, filled by asynchronous copies
// (cp.async) that run S - 1 slots ahead: no register holds data in flight, and no warp ever waits for another.
// Per k-step a lane reads its two A values (8 bytes) and the 16 B values (four 16-byte broadcasts) and issues 32
// fused multiply-adds.  The warps of a CTA take the same rows and consecutive by, so the A panel they stream is
// shared through L1 / L2.  Every output accumulates k = 0 .. K - 1 in order with one fused multiply-add per step, as
// the reference's thread does.
// =====================================================================================
struct SgemmArgs {
    const float* A;
    const float* B;
    float* C;
    int M, N, K;
    int gx, gy;      // M / 128, N / 16
    int start, end;  // original blocks, bx fastest
    // 0: a work item is half a block over the whole K (the reference's order of additions, bit for bit).
    // > 0 (a multiple of 8): a work item covers that many k-steps and adds 2 x its partial sums to C with reductions;
    // C must already hold 2 x its old value (sgemm_scale_c_kernel) -- half a block of K = 4064 is 280 us of one warp,
    // far too long a unit to share an SM with a GEMM of tens of microseconds.
    int k_per_item;
    // 1: the warps of a CTA work as a group on one (bx, half) and up to `nw` consecutive by, and share the A slices
    // in shared memory (sgemm_group below); k_per_item then cuts the groups' work.  For launches that cover many by per
    // bx; a short block range keeps the per-warp form.
    int coop;
};

constexpr int kSgemmChunk = 8;                                       // k-steps per ring slot
constexpr int kSgemmSlotBytes = kSgemmChunk * (64 + 16) * 4;         // 2560
__host__ __device__ constexpr int sgemm_role_smem(int warps, int slots) { return warps * slots * kSgemmSlotBytes; }

__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// rows 64 * half .. + 63 of block (bx, by); ring: this warp's S slots
template <int S>
__device__ __forceinline__ void sgemm_half_block(const SgemmArgs& g, const int bx, const int by, const int half,
                                                 uint8_t* ring, const int lane, const int k_begin, const int k_end,
                                                 const bool partial) {
    float c[2][16];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int j = 0; j < 16; ++j) c[r][j] = 0.0f;
    const int m0 = bx * 128 + half * 64;
    const size_t lda = static_cast<size_t>(g.M), ldb = static_cast<size_t>(g.N);
    const float* __restrict__ a_ptr = g.A + m0 + static_cast<size_t>(k_begin) * lda;
    const float* __restrict__ b_ptr = g.B + by * 16 + static_cast<size_t>(k_begin) * ldb;
    const int K = k_end - k_begin;  // k-steps of this item
    const int nchunks = (K + kSgemmChunk - 1) / kSgemmChunk;
    const uint32_t ring_u32 = smem_u32(ring);
    // slot layout: A [8][64] floats, then B [8][16] floats
    auto issue = [&](int ch) {
        if (ch < nchunks) {
            const uint32_t slot = ring_u32 + (ch % S) * kSgemmSlotBytes;
            const int k0 = ch * kSgemmChunk;
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // 8 x 256 bytes of A: 128 pieces of 16 bytes
                const int idx = lane + 32 * j, kl = idx >> 4, seg = idx & 15;
                if (k0 + kl < K) cp_async_16(slot + (kl * 64 + seg * 4) * 4, a_ptr + (k0 + kl) * lda + seg * 4);
            }
            const int kl = lane >> 2, seg = lane & 3;  // 8 x 64 bytes of B: 32 pieces
            if (k0 + kl < K) cp_async_16(slot + (kSgemmChunk * 64 + kl * 16 + seg * 4) * 4, b_ptr + (k0 + kl) * ldb + seg * 4);
        }
        cp_async_commit();  // also when nothing was issued: the group count stays in step with the chunk count
    };
#pragma unroll
    for (int s = 0; s < S - 1; ++s) issue(s);
    for (int ch = 0; ch < nchunks; ++ch) {
        issue(ch + S - 1);
        cp_async_wait<S - 1>();  // this lane's copies of chunk ch have landed
        __syncwarp();            // ... and so have the other lanes'
        const float* slot = reinterpret_cast<const float*>(ring + (ch % S) * kSgemmSlotBytes);
        const int steps = min(kSgemmChunk, K - ch * kSgemmChunk);
#pragma unroll
        for (int kk = 0; kk < kSgemmChunk; ++kk) {
            if (kk < steps) {  // the same in every lane; only the last chunk of a K that is no multiple of 8 is short
                const float2 av = *reinterpret_cast<const float2*>(slot + kk * 64 + 2 * lane);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 b = *reinterpret_cast<const float4*>(slot + kSgemmChunk * 64 + kk * 16 + 4 * q);
                    c[0][4 * q + 0] = fmaf(av.x, b.x, c[0][4 * q + 0]);
                    c[0][4 * q + 1] = fmaf(av.x, b.y, c[0][4 * q + 1]);
                    c[0][4 * q + 2] = fmaf(av.x, b.z, c[0][4 * q + 2]);
                    c[0][4 * q + 3] = fmaf(av.x, b.w, c[0][4 * q + 3]);
                    c[1][4 * q + 0] = fmaf(av.y, b.x, c[1][4 * q + 0]);
                    c[1][4 * q + 1] = fmaf(av.y, b.y, c[1][4 * q + 1]);
                    c[1][4 * q + 2] = fmaf(av.y, b.z, c[1][4 * q + 2]);
                    c[1][4 * q + 3] = fmaf(av.y, b.w, c[1][4 * q + 3]);
                }
            }
        }
        __syncwarp();  // the slot may be refilled by the next issue
    }
    cp_async_wait<0>();
    // C = C * beta + alpha * c with alpha = beta = 2 (src/gptb_kernel/sgemm_kernel.cu:12-13, 59-62)
    float* c_ptr = g.C + static_cast<size_t>(by) * 16 * lda + m0 + 2 * lane;
    if (partial) {  // C already holds 2 x its old value
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            red_add_f32(c_ptr + j * lda, 2.0f * c[0][j]);
            red_add_f32(c_ptr + j * lda + 1, 2.0f * c[1][j]);
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        float2* p = reinterpret_cast<float2*>(c_ptr + j * lda);
        float2 o = *p;
        o.x = o.x * 2.0f + 2.0f * c[0][j];
        o.y = o.y * 2.0f + 2.0f * c[1][j];
        *p = o;
    }
}

// The warps of the role as one group: all 128 rows of bx, warp w takes column block `by` (inactive warps only help
// to fetch); lane l holds rows 4 l .. 4 l + 3 of the 16 columns (64 accumulators).  The A slice of a k-chunk
// (16 x 128 floats) is fetched once for all warps, every warp fetches its own B slice; slot = A [16][128], then
// B [nw][16][16].  One role-wide barrier per chunk: it publishes chunk ch and retires chunk ch - 1, whose slot the copies
// issued right after it overwrite.  Per k-step a lane reads 16 bytes of A and four 16-byte broadcasts of B for 64
// fused multiply-adds: half the shared-memory traffic per multiply-add of sgemm_half_block, whose reads and ring
// fills together keep the shared-memory pipe as busy as the FMA pipe.  The arithmetic per output is the same sequence
// of fused multiply-adds.  Needs nw >= 8 (the slots use the ring space of sgemm_role_smem).
constexpr int kSgemmGroupChunk = 16;  // k-steps per ring slot of the group form
template <int S>
__device__ __forceinline__ void sgemm_group(const SgemmArgs& g, const int bx, const int by, const bool active,
                                            uint8_t* ring, const int w, const int nw, const int lane, const int k_begin,
                                            const int k_end, const bool partial, const uint32_t bar_id) {
    static_assert(S >= 2, "the ring needs two slots");
    float c[4][16];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int j = 0; j < 16; ++j) c[r][j] = 0.0f;
    const int t = 32 * w + lane, nt = 32 * nw;
    const int m0 = bx * 128;
    const size_t lda = static_cast<size_t>(g.M), ldb = static_cast<size_t>(g.N);
    const float* __restrict__ a_ptr = g.A + m0 + static_cast<size_t>(k_begin) * lda;
    const float* __restrict__ b_ptr = g.B + (active ? by : 0) * 16 + static_cast<size_t>(k_begin) * ldb;
    const int K = k_end - k_begin;
    const int nchunks = (K + kSgemmGroupChunk - 1) / kSgemmGroupChunk;
    const uint32_t slot_bytes = (kSgemmGroupChunk * 128 + nw * kSgemmGroupChunk * 16) * 4;
    const uint32_t ring_u32 = smem_u32(ring);
    auto issue = [&](int ch) {
        if (ch < nchunks) {
            const uint32_t slot = ring_u32 + (ch % S) * slot_bytes;
            const int k0 = ch * kSgemmGroupChunk;
            for (int idx = t; idx < kSgemmGroupChunk * 32; idx += nt) {  // 16 x 512 bytes of A: 512 pieces of 16 bytes
                const int kl = idx >> 5, seg = idx & 31;
                if (k0 + kl < K) cp_async_16(slot + (kl * 128 + seg * 4) * 4, a_ptr + (k0 + kl) * lda + seg * 4);
            }
#pragma unroll
            for (int j = 0; j < kSgemmGroupChunk / 8; ++j) {  // this warp's 16 x 64 bytes of B
                const int kl = (lane >> 2) + 8 * j, seg = lane & 3;
                if (active && k0 + kl < K)
                    cp_async_16(slot + (kSgemmGroupChunk * 128 + (w * kSgemmGroupChunk + kl) * 16 + seg * 4) * 4,
                                b_ptr + (k0 + kl) * ldb + seg * 4);
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int q = 0; q < S - 1; ++q) issue(q);
    for (int ch = 0; ch < nchunks; ++ch) {
        cp_async_wait<S - 2>();  // this thread's copies of chunk ch have landed
        role_sync(bar_id, nt);   // ... and everybody's; everybody is done with chunk ch - 1
        issue(ch + S - 1);       // into the slot of chunk ch - 1
        if (!active) continue;
        const float* slot = reinterpret_cast<const float*>(ring + (ch % S) * slot_bytes);
        const float* bs = slot + kSgemmGroupChunk * 128 + w * kSgemmGroupChunk * 16;
        const int steps = min(kSgemmGroupChunk, K - ch * kSgemmGroupChunk);
        auto k_step = [&](const float4 av, const float4 (&b)[4]) {
            const float a4[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    c[r][4 * q + 0] = fmaf(a4[r], b[q].x, c[r][4 * q + 0]);
                    c[r][4 * q + 1] = fmaf(a4[r], b[q].y, c[r][4 * q + 1]);
                    c[r][4 * q + 2] = fmaf(a4[r], b[q].z, c[r][4 * q + 2]);
                    c[r][4 * q + 3] = fmaf(a4[r], b[q].w, c[r][4 * q + 3]);
                }
        };
        auto fetch = [&](const int kk, float4& av, float4 (&b)[4]) {
            av = *reinterpret_cast<const float4*>(slot + kk * 128 + 4 * lane);
#pragma unroll
            for (int q = 0; q < 4; ++q) b[q] = *reinterpret_cast<const float4*>(bs + kk * 16 + 4 * q);
        };
        if (steps == kSgemmGroupChunk) {
            // whole chunk, no predicates: the operands of step kk + 1 are read while step kk multiplies
            float4 av, b[4];
            fetch(0, av, b);
#pragma unroll
            for (int kk = 0; kk < kSgemmGroupChunk; ++kk) {
                float4 avn = av, bn[4] = {b[0], b[1], b[2], b[3]};
                if (kk + 1 < kSgemmGroupChunk) fetch(kk + 1, avn, bn);
                k_step(av, b);
                av = avn;
#pragma unroll
                for (int q = 0; q < 4; ++q) b[q] = bn[q];
            }
        } else {
            for (int kk = 0; kk < steps; ++kk) {  // the ragged end of a K that is no multiple of 16
                float4 av, b[4];
                fetch(kk, av, b);
                k_step(av, b);
            }
        }
    }
    cp_async_wait<0>();
    role_sync(bar_id, nt);  // the next group's first copies may overwrite any slot
    if (!active) return;
    // C = C * beta + alpha * c with alpha = beta = 2 (src/gptb_kernel/sgemm_kernel.cu:12-13, 59-62)
    float* c_ptr = g.C + static_cast<size_t>(by) * 16 * lda + m0 + 4 * lane;
    if (partial) {  // C already holds 2 x its old value
#pragma unroll
        for (int j = 0; j < 16; ++j)
#pragma unroll
            for (int r = 0; r < 4; ++r) red_add_f32(c_ptr + j * lda + r, 2.0f * c[r][j]);
        return;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        float4* p = reinterpret_cast<float4*>(c_ptr + j * lda);
        float4 o = *p;
        o.x = o.x * 2.0f + 2.0f * c[0][j];
        o.y = o.y * 2.0f + 2.0f * c[1][j];
        o.z = o.z * 2.0f + 2.0f * c[2][j];
        o.w = o.w * 2.0f + 2.0f * c[3][j];
        *p = o;
    }
}

// warp `w` of `nw` in CTA `cta` of `ncta`; smem: sgemm_role_smem(nw, S) bytes, 16-byte aligned; counter: the CTA's
// item counter (zero on entry; used when the items are split in k)
template <int S>
__device__ __forceinline__ void sgemm_role(const SgemmArgs& g, uint8_t* smem, int* counter, const int w, const int nw,
                                           const int lane, const int cta, const int ncta, const uint32_t bar_id = 0) {
    if (g.coop) {
        // items: bx fastest, so that the CTAs running together share B rows; then the group of by; then the k-chunk.
        // Only the by the block range touches are grouped, and they are spread evenly over the groups (258 on 16
        // warps: groups of 15 and 16, not 16 x 16 + 2).
        const int by_lo = g.start / g.gx, nby = (g.end + g.gx - 1) / g.gx - by_lo;
        const int ygroups = (nby + nw - 1) / nw;
        const int nk = g.k_per_item > 0 ? (g.K + g.k_per_item - 1) / g.k_per_item : 1;
        const long long nitems = static_cast<long long>(g.gx) * ygroups * nk;
        for (long long item = cta; item < nitems; item += ncta) {
            const int bx = static_cast<int>(item % g.gx);
            const int yg = static_cast<int>((item / g.gx) % ygroups);
            const int kc = static_cast<int>(item / (static_cast<long long>(g.gx) * ygroups));
            const int b0 = by_lo + static_cast<int>(static_cast<long long>(yg) * nby / ygroups);
            const int b1 = by_lo + static_cast<int>(static_cast<long long>(yg + 1) * nby / ygroups);
            const int by = b0 + w, pos = by * g.gx + bx;
            const bool active = by < b1 && pos >= g.start && pos < g.end;
            const bool split = g.k_per_item > 0;  // C then holds 2 x its old value already (sgemm_scale_c)
            const int k0 = split ? kc * g.k_per_item : 0, k1 = split ? min(k0 + g.k_per_item, g.K) : g.K;
            sgemm_group<S>(g, bx, by, active, smem, w, nw, lane, k0, k1, split, bar_id);
        }
        return;
    }
    uint8_t* ring = smem + w * (S * kSgemmSlotBytes);
    if (g.k_per_item > 0) {
        const int nchunks = (g.K + g.k_per_item - 1) / g.k_per_item;
        const long long nitems = 2ll * (g.end - g.start) * nchunks;
        for (long long item = claim_item(counter, lane, cta, ncta); item < nitems; item = claim_item(counter, lane, cta, ncta)) {
            const int chunk = static_cast<int>(item % nchunks);
            const long long hb = item / nchunks;
            const int pos = g.start + static_cast<int>(hb >> 1);
            const int k0 = chunk * g.k_per_item;
            sgemm_half_block<S>(g, pos % g.gx, (pos / g.gx) % g.gy, static_cast<int>(hb & 1), ring, lane, k0,
                                min(k0 + g.k_per_item, g.K), true);
        }
        return;
    }
    // groups of nw consecutive by at one (bx, half); (bx, half) fastest so that neighbouring CTAs share B rows
    const int ygroups = (g.gy + nw - 1) / nw;
    const int ngroups = 2 * g.gx * ygroups;
    for (int grp = cta; grp < ngroups; grp += ncta) {
        const int xh = grp % (2 * g.gx), by = (grp / (2 * g.gx)) * nw + w;
        if (by >= g.gy) continue;
        const int pos = by * g.gx + (xh >> 1);
        if (pos < g.start || pos >= g.end) continue;
        sgemm_half_block<S>(g, xh >> 1, by, xh & 1, ring, lane, 0, g.K, false);
    }
}

// C *= 2 on the blocks of [start, end): the first half of C = 2 C + 2 A B when the items are split in k
__device__ __forceinline__ void sgemm_scale_c(const SgemmArgs& g, const int t, const int nt, const int cta, const int ncta) {
    for (int pos = g.start + cta; pos < g.end; pos += ncta) {
        const int bx = pos % g.gx, by = (pos / g.gx) % g.gy;
        float* c = g.C + static_cast<size_t>(by) * 16 * g.M + bx * 128;
        for (int i = t; i < 16 * 32; i += nt) {
            float4* p = reinterpret_cast<float4*>(c + static_cast<size_t>(i >> 5) * g.M) + (i & 31);
            float4 v = *p;
            v.x *= 2.0f, v.y *= 2.0f, v.z *= 2.0f, v.w *= 2.0f;
            *p = v;
        }
    }
}

// =====================================================================================
// lbm.  Layout of the reference: element e of cell (x, y, z) at e * cells + x + y nx + z nx ny with the 20 elements
// C N S E W T B NE NW SE SW NT NB ST SB ET EB WT WB FLAGS; the pointers address cell (0, 0, 0) and two z-planes of
// margin lie on either side (src/header/lbm_header.h:52-53, 246-247).  Original block p of the (ny, nz) grid is the
// row y = p % ny, z = p / ny.  A warp takes 32 consecutive cells of a row, one per lane: 20 loads of a full 128-byte
// line each, the collision in registers (about 60 of them, so that 32 warps per SM keep 80 KB of loads in flight),
// and 19 stores to the neighbours by flat index (so rows at the faces write into the next row or the margin, as in
// the reference).  The kernel moves 156 bytes per cell and does nothing else of note: it is bound by HBM.
// =====================================================================================
struct LbmArgs {
    const float* src;
    float* dst;
    int nx, ny, nz;  // nx a multiple of 32
    int start, end;  // original blocks (rows), y fastest
};

enum LbmEntry { LB_C, LB_N, LB_S, LB_E, LB_W, LB_T, LB_B, LB_NE, LB_NW, LB_SE, LB_SW, LB_NT, LB_NB, LB_ST, LB_SB, LB_ET,
                LB_EB, LB_WT, LB_WB, LB_FLAGS };

// the relaxation of one cell; f[0..18] in, f[0..18] out (src/gptb_kernel/lbm_kernel.cu:70-146)
__device__ __forceinline__ void lbm_collide(float (&f)[19], const unsigned flags) {
    float tempC = f[LB_C], tempN = f[LB_N], tempS = f[LB_S], tempE = f[LB_E], tempW = f[LB_W], tempT = f[LB_T],
          tempB = f[LB_B], tempNE = f[LB_NE], tempNW = f[LB_NW], tempSE = f[LB_SE], tempSW = f[LB_SW], tempNT = f[LB_NT],
          tempNB = f[LB_NB], tempST = f[LB_ST], tempSB = f[LB_SB], tempET = f[LB_ET], tempEB = f[LB_EB], tempWT = f[LB_WT],
          tempWB = f[LB_WB];
    if (flags & 1u) {  // obstacle: everything that came in goes back where it came from
        float temp_swp;
        temp_swp = tempN; tempN = tempS; tempS = temp_swp;
        temp_swp = tempE; tempE = tempW; tempW = temp_swp;
        temp_swp = tempT; tempT = tempB; tempB = temp_swp;
        temp_swp = tempNE; tempNE = tempSW; tempSW = temp_swp;
        temp_swp = tempNW; tempNW = tempSE; tempSE = temp_swp;
        temp_swp = tempNT; tempNT = tempSB; tempSB = temp_swp;
        temp_swp = tempNB; tempNB = tempST; tempST = temp_swp;
        temp_swp = tempET; tempET = tempWB; tempWB = temp_swp;
        temp_swp = tempEB; tempEB = tempWT; tempWT = temp_swp;
    } else {
        constexpr float OMEGA = 1.95f, DFL1 = 1.0f / 3.0f, DFL2 = 1.0f / 18.0f, DFL3 = 1.0f / 36.0f;
        float ux, uy, uz, rho, u2;
        float temp1, temp2, temp_base;
        rho = tempC + tempN + tempS + tempE + tempW + tempT + tempB + tempNE + tempNW + tempSE + tempSW + tempNT + tempNB +
              tempST + tempSB + tempET + tempEB + tempWT + tempWB;
        ux = +tempE - tempW + tempNE - tempNW + tempSE - tempSW + tempET + tempEB - tempWT - tempWB;
        uy = +tempN - tempS + tempNE + tempNW - tempSE - tempSW + tempNT + tempNB - tempST - tempSB;
        uz = +tempT - tempB + tempNT - tempNB + tempST - tempSB + tempET - tempEB + tempWT - tempWB;
        ux /= rho;
        uy /= rho;
        uz /= rho;
        if (flags & 2u) {  // accelerated cell
            ux = 0.005f;
            uy = 0.002f;
            uz = 0.000f;
        }
        u2 = 1.5f * (ux * ux + uy * uy + uz * uz) - 1.0f;
        temp_base = OMEGA * rho;
        temp1 = DFL1 * temp_base;
        temp2 = 1.0f - OMEGA;
        tempC = temp2 * tempC + temp1 * (-u2);
        temp1 = DFL2 * temp_base;
        tempN = temp2 * tempN + temp1 * (uy * (4.5f * uy + 3.0f) - u2);
        tempS = temp2 * tempS + temp1 * (uy * (4.5f * uy - 3.0f) - u2);
        tempT = temp2 * tempT + temp1 * (uz * (4.5f * uz + 3.0f) - u2);
        tempB = temp2 * tempB + temp1 * (uz * (4.5f * uz - 3.0f) - u2);
        tempE = temp2 * tempE + temp1 * (ux * (4.5f * ux + 3.0f) - u2);
        tempW = temp2 * tempW + temp1 * (ux * (4.5f * ux - 3.0f) - u2);
        temp1 = DFL3 * temp_base;
        tempNT = temp2 * tempNT + temp1 * ((+uy + uz) * (4.5f * (+uy + uz) + 3.0f) - u2);
        tempNB = temp2 * tempNB + temp1 * ((+uy - uz) * (4.5f * (+uy - uz) + 3.0f) - u2);
        tempST = temp2 * tempST + temp1 * ((-uy + uz) * (4.5f * (-uy + uz) + 3.0f) - u2);
        tempSB = temp2 * tempSB + temp1 * ((-uy - uz) * (4.5f * (-uy - uz) + 3.0f) - u2);
        tempNE = temp2 * tempNE + temp1 * ((+ux + uy) * (4.5f * (+ux + uy) + 3.0f) - u2);
        tempSE = temp2 * tempSE + temp1 * ((+ux - uy) * (4.5f * (+ux - uy) + 3.0f) - u2);
        tempET = temp2 * tempET + temp1 * ((+ux + uz) * (4.5f * (+ux + uz) + 3.0f) - u2);
        tempEB = temp2 * tempEB + temp1 * ((+ux - uz) * (4.5f * (+ux - uz) + 3.0f) - u2);
        tempNW = temp2 * tempNW + temp1 * ((-ux + uy) * (4.5f * (-ux + uy) + 3.0f) - u2);
        tempSW = temp2 * tempSW + temp1 * ((-ux - uy) * (4.5f * (-ux - uy) + 3.0f) - u2);
        tempWT = temp2 * tempWT + temp1 * ((-ux + uz) * (4.5f * (-ux + uz) + 3.0f) - u2);
        tempWB = temp2 * tempWB + temp1 * ((-ux - uz) * (4.5f * (-ux - uz) + 3.0f) - u2);
    }
    f[LB_C] = tempC; f[LB_N] = tempN; f[LB_S] = tempS; f[LB_E] = tempE; f[LB_W] = tempW; f[LB_T] = tempT; f[LB_B] = tempB;
    f[LB_NE] = tempNE; f[LB_NW] = tempNW; f[LB_SE] = tempSE; f[LB_SW] = tempSW; f[LB_NT] = tempNT; f[LB_NB] = tempNB;
    f[LB_ST] = tempST; f[LB_SB] = tempSB; f[LB_ET] = tempET; f[LB_EB] = tempEB; f[LB_WT] = tempWT; f[LB_WB] = tempWB;
}

__device__ __forceinline__ void lbm_role(const LbmArgs& g, int* counter, const int lane, const int cta, const int ncta) {
    const size_t cells = static_cast<size_t>(g.nx) * g.ny * g.nz;
    const int segs = g.nx / 32;
    const long long nitems = static_cast<long long>(g.end - g.start) * segs;
    const long long plane = static_cast<long long>(g.nx) * g.ny;
    // Items are dealt to a CTA in runs of 16: its warps work on 16 consecutive 32-cell pieces at a time, i.e. on 2 KB
    // of each of the 39 arrays, instead of on pieces 128 bytes long that lie ncta pieces apart.
    constexpr long long kRun = 16;
    const long long nitems_padded = (nitems + kRun * ncta - 1) / (kRun * ncta) * (kRun * ncta);
    for (long long raw = claim_item(counter, lane, cta, ncta); raw < nitems_padded; raw = claim_item(counter, lane, cta, ncta)) {
        const long long k = raw / ncta;  // this CTA's k-th claim
        const long long item = ((k / kRun) * ncta + cta) * kRun + k % kRun;
        if (item >= nitems) continue;
        const int p = g.start + static_cast<int>(item / segs), seg = static_cast<int>(item % segs);
        const int y = p % g.ny, z = (p / g.ny) % g.nz;
        const long long cell = seg * 32 + lane + static_cast<long long>(y) * g.nx + z * plane;
        float f[19];
#pragma unroll
        for (int e = 0; e < 19; ++e) f[e] = __ldcs(g.src + e * cells + cell);
        const unsigned flags = __float_as_uint(__ldcs(g.src + LB_FLAGS * cells + cell));
        lbm_collide(f, flags);
        float* d = g.dst + cell;
        const long long nx = g.nx;
        // value e goes to the neighbour in direction e, by flat index (dx, dy, dz of the 19 directions)
        __stcs(d + LB_C * cells, f[LB_C]);
        __stcs(d + LB_N * cells + nx, f[LB_N]);
        __stcs(d + LB_S * cells - nx, f[LB_S]);
        __stcs(d + LB_E * cells + 1, f[LB_E]);
        __stcs(d + LB_W * cells - 1, f[LB_W]);
        __stcs(d + LB_T * cells + plane, f[LB_T]);
        __stcs(d + LB_B * cells - plane, f[LB_B]);
        __stcs(d + LB_NE * cells + 1 + nx, f[LB_NE]);
        __stcs(d + LB_NW * cells - 1 + nx, f[LB_NW]);
        __stcs(d + LB_SE * cells + 1 - nx, f[LB_SE]);
        __stcs(d + LB_SW * cells - 1 - nx, f[LB_SW]);
        __stcs(d + LB_NT * cells + nx + plane, f[LB_NT]);
        __stcs(d + LB_NB * cells + nx - plane, f[LB_NB]);
        __stcs(d + LB_ST * cells - nx + plane, f[LB_ST]);
        __stcs(d + LB_SB * cells - nx - plane, f[LB_SB]);
        __stcs(d + LB_ET * cells + 1 + plane, f[LB_ET]);
        __stcs(d + LB_EB * cells + 1 - plane, f[LB_EB]);
        __stcs(d + LB_WT * cells - 1 + plane, f[LB_WT]);
        __stcs(d + LB_WB * cells - 1 - plane, f[LB_WB]);
    }
}

// =====================================================================================
// fft.  A warp transforms one batch entry of 256 complex points in place with the reference's radix-2 Stockham
// schedule (src/gptb_kernel/fft_kernel.cu:27-41): in pass Ns = 1, 2, .., 128 butterfly j = 0 .. 127 reads points j
// and j + 128, multiplies the second by w = (cos a, sin a), a = float(-2 pi (j % Ns) / (2 Ns)) with the quotient in
// binary64, and writes sum and difference to expand(j, Ns, 2) and + Ns.  a only takes the values float(-2 pi t / 256),
// t = 0 .. 127 (the binary64 quotients agree exactly because Ns is a power of two), so the role fills a 128-entry
// table (per pass) with the same cosf / sinf calls once and every pass reads w from it.
//
// A pass takes the top bit of the point index as the butterfly dimension and re-inserts the result bit at position
// log2 Ns, so three consecutive passes only combine points that differ in the top three index bits: the eight points
// lane + 32 q that a lane holds anyway.  The eight passes therefore run as 3 + 3 + 2 passes in registers with two
// exchanges through a warp-private buffer in shared memory (instead of eight round trips), the points come from
// global memory straight into registers and leave from registers.  Every butterfly is the reference's, operation for
// operation (the product is spelled with the contractions nvcc applies to it), so the result is bit-identical.
// =====================================================================================
struct FftArgs {
    float2* data;
    int nfft;        // batch entries = original blocks
    int start, end;
};

// twiddles per pass, packed: entry (Ns - 1) + lo is w for j % Ns = lo, so that the lanes of a warp read neighbouring
// entries in every pass (one table of 128 angles would be read with strides of up to 128 bytes)
constexpr int kFftTwiddleBytes = 256 * 8;
constexpr int kFftWarpBytes = 256 * 8;
__host__ __device__ constexpr int fft_role_smem(int warps) { return kFftTwiddleBytes + warps * kFftWarpBytes; }

// where point p lives in the warp's exchange buffer: the low four bits are mixed with bits 4..6 so that the writes
// of both exchanges (strides of 8 points between lanes) and the reads (consecutive points) are free of bank conflicts
__device__ __forceinline__ int fft_slot(const int p) { return p ^ ((p >> 4) & 7) ^ ((p >> 3) & 8); }
__device__ __forceinline__ int fft_rev3(const int i) { return ((i & 1) << 2) | (i & 2) | (i >> 2); }

// (a, b) <- (a + w b, a - w b)
__device__ __forceinline__ void fft_bfly(float2& a, float2& b, const float2 w) {
    // the two contractions nvcc applies to the reference's a.x*b.x - a.y*b.y and a.x*b.y + a.y*b.x (src/header/fft_header.h:20),
    // found by comparing the four possible pairs with the reference's output bit for bit
    const float tr = __fmaf_rn(b.x, w.x, -__fmul_rn(b.y, w.y));
    const float ti = __fmaf_rn(b.y, w.x, __fmul_rn(b.x, w.y));
    const float2 sum = make_float2(__fadd_rn(a.x, tr), __fadd_rn(a.y, ti));
    b = make_float2(__fsub_rn(a.x, tr), __fsub_rn(a.y, ti));
    a = sum;
}

// Passes Ns = 2^S, 2^(S+1), 2^(S+2) on the points e[q] = (index bits 7..5 = q, the rest fixed); lo0 = the low S index
// bits.  Afterwards slot i = (tA tB tC) holds the point whose three new index bits above lo0 are (tC tB tA).
template <int S>
__device__ __forceinline__ void fft_passes3(float2 (&e)[8], const float2* __restrict__ tw, const int lo0) {
    {
        const float2 w = tw[(1 << S) - 1 + lo0];
#pragma unroll
        for (int i = 0; i < 4; ++i) fft_bfly(e[i], e[i + 4], w);
    }
#pragma unroll
    for (int tA = 0; tA < 2; ++tA) {
        const float2 w = tw[(2 << S) - 1 + tA * (1 << S) + lo0];
        fft_bfly(e[4 * tA], e[4 * tA + 2], w);
        fft_bfly(e[4 * tA + 1], e[4 * tA + 3], w);
    }
#pragma unroll
    for (int tA = 0; tA < 2; ++tA)
#pragma unroll
        for (int tB = 0; tB < 2; ++tB) {
            const float2 w = tw[(4 << S) - 1 + tB * (2 << S) + tA * (1 << S) + lo0];
            fft_bfly(e[4 * tA + 2 * tB], e[4 * tA + 2 * tB + 1], w);
        }
}

// smem: fft_role_smem(nw) bytes, 16-byte aligned.  t / nt: thread index within the role and its thread count.
__device__ __forceinline__ void fft_role(const FftArgs& g, uint8_t* smem, const int t, const int nt, const int cta,
                                         const int ncta, const uint32_t bar_id) {
    float2* tw = reinterpret_cast<float2*>(smem);
    const int w = t >> 5, lane = t & 31, nw = nt >> 5;
    float2* buf = reinterpret_cast<float2*>(smem + kFftTwiddleBytes) + w * (kFftWarpBytes / 8);
    for (int i = t; i < 255; i += nt) {
        const int Ns = 1 << (31 - __clz(i + 1)), lo = i + 1 - Ns;
        const float angle = -2 * M_PI * (lo * (128 / Ns)) / 256;  // binary64 quotient rounded to binary32, as in the reference
        tw[i] = make_float2(cosf(angle), sinf(angle));
    }
    role_sync(bar_id, nt);
    for (int p = g.start + cta * nw + w; p < g.end; p += ncta * nw) {
        float2* d = g.data + static_cast<size_t>(p % g.nfft) * 256;
        float2 e[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) e[q] = d[lane + 32 * q];
        // passes 1, 2, 4: afterwards the point of slot i sits at index 8 lane + rev3(i)
        fft_passes3<0>(e, tw, 0);
#pragma unroll
        for (int i = 0; i < 8; ++i) buf[fft_slot(8 * lane + fft_rev3(i))] = e[i];
        __syncwarp();
#pragma unroll
        for (int q = 0; q < 8; ++q) e[q] = buf[fft_slot(lane + 32 * q)];
        __syncwarp();
        // passes 8, 16, 32: index bits (4 3 | new three | 2 1 0)
        fft_passes3<3>(e, tw, lane & 7);
#pragma unroll
        for (int i = 0; i < 8; ++i) buf[fft_slot(((lane >> 3) << 6) | (fft_rev3(i) << 3) | (lane & 7))] = e[i];
        __syncwarp();
#pragma unroll
        for (int q = 0; q < 8; ++q) e[q] = buf[fft_slot(lane + 32 * q)];
        __syncwarp();
        // passes 64 and 128 on the two sets q & 1 = 0, 1 (index bit 5)
#pragma unroll
        for (int y5 = 0; y5 < 2; ++y5) {
            const float2 wv = tw[63 + y5 * 32 + lane];
            fft_bfly(e[y5], e[4 + y5], wv);
            fft_bfly(e[2 + y5], e[6 + y5], wv);
        }
#pragma unroll
        for (int tA = 0; tA < 2; ++tA)
#pragma unroll
            for (int y5 = 0; y5 < 2; ++y5) fft_bfly(e[4 * tA + y5], e[4 * tA + 2 + y5], tw[127 + tA * 64 + y5 * 32 + lane]);
        // slot (tA tB y5) is point 128 tB + 64 tA + 32 y5 + lane
#pragma unroll
        for (int i = 0; i < 8; ++i) d[lane + 32 * (((i & 2) << 1) | ((i & 4) >> 1) | (i & 1))] = e[i];
    }
}

// =====================================================================================
// cutcp.  Atoms lie in bins of 4 A, eight float4 {x, y, z, q} each, q = 0 ending a bin; `bins` addresses the bin at the
// lattice origin, `c` margin bins surround the lattice.  Original block p of the (gx, gy, gz) grid is the region
// x = p / (gy gz), y = (p / gz) % gy, z = p % gz of 8 x 8 x 8 lattice points, stored at ((z gy + y) gx + x) * 512 in
// the order [z][y][x].  A warp computes a quarter of a region: lane l of quarter q is the reference's thread
// tid = 32 q + l, i.e. the column x = tid % 8, z = tid / 16 and the four points y = (tid / 8) % 2 + 2 s, s = 0 .. 3,
// which it steps through the way that thread does (dy -= 2 h, src/gptb_kernel/cutcp_kernel.cu:134-160); it walks the
// neighbour bins in list order and the atoms in bin order: per point the same sequence of operations as in the
// reference.  The eight atoms of a bin are the same addresses in every lane: eight broadcast loads issued together
// instead of the reference's staging of bins through shared memory.
// =====================================================================================
struct CutcpArgs {
    int bin_dim_x, bin_dim_y;
    const float4* bins;   // bin at the lattice origin
    float h, cutoff2, inv_cutoff2;
    float* regions;
    int gx, gy, gz;
    const int4* nbr;      // neighbour offsets {dx, dy, dz, 0}
    int nbrlen;
    int start, end;
    // 0: a work item is a quarter region over the whole neighbour list (the reference's order of additions, bit for
    // bit).  > 0: a work item covers that many neighbour bins and adds its partial sums to the region with reductions;
    // the region must be zero before (cutcp_zero) -- a quarter region over 335 bins is 370 us of one warp.
    int nbr_per_item;
};

__device__ __forceinline__ void cutcp_quarter(const CutcpArgs& g, const int rx, const int ry, const int rz, const int quarter,
                                              const int lane, const int nb_begin, const int nb_end, const bool partial) {
    constexpr float kBinInvLen = 1.f / 4.f;
    const int tid = 32 * quarter + lane;
    const int tx = tid & 7, ty = (tid >> 3) & 1, tz = tid >> 4;
    const float x = (8 * rx + tx) * g.h;
    const float y = (8 * ry + ty) * g.h;
    const float z = (8 * rz + tz) * g.h;
    const int cx = static_cast<int>(floorf((8 * rx + 4) * g.h * kBinInvLen));
    const int cy = static_cast<int>(floorf((8 * ry + 4) * g.h * kBinInvLen));
    const int cz = static_cast<int>(floorf((8 * rz + 4) * g.h * kBinInvLen));
    float e0 = 0.f, e1 = 0.f, e2 = 0.f, e3 = 0.f;
    const float h2 = 2.0f * g.h, cutoff2 = g.cutoff2, inv_cutoff2 = g.inv_cutoff2;
    for (int nb = nb_begin; nb < nb_end; ++nb) {
        const int4 o = __ldg(g.nbr + nb);
        const float4* bin = g.bins + ((static_cast<long long>(cz + o.z) * g.bin_dim_y + (cy + o.y)) * g.bin_dim_x + (cx + o.x)) * 8;
        float4 atom[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) atom[i] = __ldg(bin + i);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float aq = atom[i].w;
            if (0.f == aq) break;  // no more atoms in this bin (the same in every lane)
            // the fused operations are spelled out so that the last bit does not depend on what else the compiler sees
            const float dx = atom[i].x - x;
            const float dz = atom[i].z - z;
            const float dxdz2 = __fmaf_rn(dx, dx, __fmul_rn(dz, dz));
            float dy = atom[i].y - y;
            float r2 = __fmaf_rn(dy, dy, dxdz2);
            if (r2 < cutoff2) {
                const float sw = __fmaf_rn(-r2, inv_cutoff2, 1.f);
                e0 = __fmaf_rn(__fmul_rn(__fmul_rn(aq, rsqrtf(r2)), sw), sw, e0);
            }
            dy -= h2;
            r2 = __fmaf_rn(dy, dy, dxdz2);
            if (r2 < cutoff2) {
                const float sw = __fmaf_rn(-r2, inv_cutoff2, 1.f);
                e1 = __fmaf_rn(__fmul_rn(__fmul_rn(aq, rsqrtf(r2)), sw), sw, e1);
            }
            dy -= h2;
            r2 = __fmaf_rn(dy, dy, dxdz2);
            if (r2 < cutoff2) {
                const float sw = __fmaf_rn(-r2, inv_cutoff2, 1.f);
                e2 = __fmaf_rn(__fmul_rn(__fmul_rn(aq, rsqrtf(r2)), sw), sw, e2);
            }
            dy -= h2;
            r2 = __fmaf_rn(dy, dy, dxdz2);
            if (r2 < cutoff2) {
                const float sw = __fmaf_rn(-r2, inv_cutoff2, 1.f);
                e3 = __fmaf_rn(__fmul_rn(__fmul_rn(aq, rsqrtf(r2)), sw), sw, e3);
            }
        }
    }
    float* out = g.regions + ((static_cast<size_t>(rz) * g.gy + ry) * g.gx + rx) * 512 + (tid >> 4) * 64 + (tid & 15);
    if (partial) {
        red_add_f32(out, e0);
        red_add_f32(out + 16, e1);
        red_add_f32(out + 32, e2);
        red_add_f32(out + 48, e3);
        return;
    }
    out[0] = e0;
    out[16] = e1;
    out[32] = e2;
    out[48] = e3;
}

__device__ __forceinline__ void cutcp_role(const CutcpArgs& g, int* counter, const int lane, const int cta, const int ncta) {
    const bool split = g.nbr_per_item > 0 && g.nbr_per_item < g.nbrlen;
    const int per = split ? g.nbr_per_item : g.nbrlen;
    const int nchunks = split ? (g.nbrlen + per - 1) / per : 1;
    const long long nitems = 4ll * (g.end - g.start) * nchunks;
    for (long long item = claim_item(counter, lane, cta, ncta); item < nitems; item = claim_item(counter, lane, cta, ncta)) {
        const int chunk = static_cast<int>(item % nchunks);
        const long long q = item / nchunks;
        const int p = g.start + static_cast<int>(q >> 2);
        cutcp_quarter(g, p / (g.gy * g.gz), (p / g.gz) % g.gy, p % g.gz, static_cast<int>(q & 3), lane, chunk * per,
                      min(chunk * per + per, g.nbrlen), split);
    }
}

// zero the regions of [start, end): the starting point of the partial sums when the items are split
__device__ __forceinline__ void cutcp_zero(const CutcpArgs& g, const int t, const int nt, const int cta, const int ncta) {
    for (int p = g.start + cta; p < g.end; p += ncta) {
        const int rx = p / (g.gy * g.gz), ry = (p / g.gz) % g.gy, rz = p % g.gz;
        float4* region = reinterpret_cast<float4*>(g.regions + ((static_cast<size_t>(rz) * g.gy + ry) * g.gx + rx) * 512);
        for (int i = t; i < 128; i += nt) region[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

}  // namespace tk
