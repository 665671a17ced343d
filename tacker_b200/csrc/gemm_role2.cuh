// tzgemm on CTA pairs: tcgen05.mma.cta_group::2 over a cluster of two CTAs.
//
// Same contract as gemm_role (gemm_role.cuh): C = alpha * A * B^T on the 64x64 tiles of [start, end).  One
// cluster of two CTAs (two SMs) computes a 256 x 256 pair tile: CTA r of the pair owns rows 128 r .. 128 r + 127,
// loads its own 128 x 64 A tile and ONE HALF of the B tile (128 of the 256 B rows) per K-block, and the MMA
// of the pair reads each B half from the shared memory of the CTA that loaded it.  Per K-block a CTA therefore
// brings in 32 KB for 128 x 256 outputs instead of the 48 KB of the single-CTA role: a third less operand
// traffic from L2 and a third less shared-memory fill, with two accumulator buffers kept (the 256 x 256
// single-CTA form has the same traffic but no room in tensor memory for a second buffer).
//
//   CTA 0 (leader) warp 0   TMA producer of its own A tile and B half
//                  warp 1   MMA issuer of the pair: one thread issues tcgen05.mma.cta_group::2 256x256x16
//                  warps 2..5 epilogue of its 128 rows
//   CTA 1          warp 0   TMA producer of its A tile and B half; its loads complete on the LEADER's barrier
//                  warp 1   takes part in the tensor-memory allocation only
//                  warps 2..5 epilogue of its 128 rows
//
// Signals.  full[s] lives in the leader: one arrival (the leader's producer, which also announces the bytes of
// BOTH CTAs) plus the bytes of both CTAs' loads.  empty[s] exists in both CTAs: the MMA thread signals the
// leader's with one tcgen05.commit per K-block, and the leader's producer, once it has seen that arrival, passes
// it on to the peer's barrier with a plain remote arrive -- the MMA thread is the one serial instruction stream
// the whole pair waits for (about 60 cycles per tcgen05 instruction against 128 cycles of tensor pipe per MMA),
// so everything that can be is kept out of it.  tfull[a] exists in both CTAs (two commits per tile).  tempty[a]
// lives in the leader and counts the eight epilogue warps of the pair.
// No load is a cluster broadcast: every CTA fetches what it needs itself.  Every wait is bounded as in gemm_role.
// The two CTAs never leave while the other may still touch them: everything a CTA sends to its peer is awaited
// by a role of the peer before that role ends (see the tails of the producer and the MMA issuer).
#pragma once
#include "gemm_role_m256.cuh"

namespace tk {

// ---- cluster helpers ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}

// Every thread of the cluster arrives once at kernel start; only the threads that need the peer's barriers to be
// initialised wait.
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Arrival on a barrier of this CTA or of its peer that orders nothing but the barrier itself.  The epilogue uses
// it to hand an accumulator buffer back: what it read from tensor memory is already in registers
// (tcgen05.wait::ld), and a release at cluster scope would make the warp wait for all its stores to C first.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// non-blocking probe of a barrier phase
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// operand tile load of a CTA pair: the data lands in this CTA, the bytes are counted on the barrier at
// `bar_cluster_addr`, which may belong to the peer CTA
__device__ __forceinline__ void tma_load_tile_pair(uint32_t dst_smem, const void* tmap, uint32_t bar_cluster_addr,
                                                   int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t result_slot_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_slot_smem),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// one arrival on the barrier at `bar_cluster_addr` (this CTA's or the peer's) once every MMA issued so far by
// this thread has retired in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}

// ---- optional phase trace (diagnostic builds with -DTK_TRACE only) ------------------------------------------
// Per CTA 16 values: [0] globaltimer at role entry, [1] clock at role entry, [2] clock after set-up, [3] clock when the
// first operand stage had landed (leader), [4] clock after the last commit (leader), [5] clock when the last accumulator
// was complete, [6] clock at the end of the last epilogue, [7] cycles spent in epilogues, [8] tiles, [9] clock at role
// exit, [10] globaltimer at role exit, [11] cycles the MMA thread waited for operands after the first stage, [12] cycles
// it waited for a free accumulator, [13] cycles the producer waited for free stages.  tk_debug_trace() copies them out.
#ifdef TK_TRACE
__device__ long long g_tk_trace[512 * 16];
__device__ __forceinline__ long long tk_gtime() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TK_TR(slot, val) (g_tk_trace[(blockIdx.x & 511) * 16 + (slot)] = (val))
#define TK_TRACE_ONLY(...) __VA_ARGS__
#else
#define TK_TR(slot, val) ((void)0)
#define TK_TRACE_ONLY(...)
#endif

// ---- the role ------------------------------------------------------------------------------------------
constexpr int kGemm2BN = 256;          // columns of a pair tile
constexpr int kGemm2Threads = 6 * 32;  // per CTA, as in gemm_role

template <int STAGES>
struct Gemm2Smem {
    static constexpr int kABytes = kGemmBM * kGemmBK * 2;          // 128 rows of A
    static constexpr int kBBytes = (kGemm2BN / 2) * kGemmBK * 2;   // this CTA's half of the B tile
    static constexpr int kStageBytes = kABytes + kBBytes;          // 32 KB
    static constexpr int kBarOffset = STAGES * kStageBytes;
    static constexpr int kNumBars = 2 * STAGES + 4;
    static constexpr int kTmemSlotOffset = kBarOffset + kNumBars * 8;
    static constexpr int kAbortOffset = kTmemSlotOffset + 4;
    static constexpr int kEpiPitch = 36;
    static constexpr int kEpiWarpBytes = 32 * kEpiPitch * 4;
    static constexpr int kEpiOffset = ((kAbortOffset + 4 + 127) / 128) * 128;
    static constexpr int kBytes = kEpiOffset + 4 * kEpiWarpBytes;
};

// The pair tiles of a launch as every role of a pair walks them.  Whole waves of 256 x 256 tiles first; when the
// last wave would leave at least half of the pairs idle (and the launcher supplied the 64-row B map), its tiles
// are cut into two 256 x 128 halves so that twice as many pairs share it: 256 tiles on 74 pairs take 3.5 tile
// times instead of 4.
struct PairTileList {
    int nfull;    // candidates walked as whole tiles: cand = pair, pair + npairs, ... < nfull
    int nhalves;  // half tiles after them: pair p < nhalves takes half (p & 1) of candidate nfull + p / 2
    __device__ __forceinline__ void init(const SuperTileWalk256& w, const GemmArgs& g, int npairs, bool can_split) {
        nfull = w.ncand;
        nhalves = 0;
        const bool whole = w.start == 0 && w.end == w.nt * w.mt && w.mt % 4 == 0 && w.nt % 4 == 0;
        const int rem = w.ncand % npairs;
        if (can_split && whole && rem > 0 && 2 * rem <= npairs) {
            nfull = w.ncand - rem;
            nhalves = 2 * rem;
        }
        (void)g;
    }
    // step k of pair `pair`: false when its list is exhausted; half = -1 for a whole tile, else 0 / 1
    __device__ __forceinline__ bool get(int k, int pair, int npairs, int& cand, int& half) const {
        const int nw = nfull > pair ? (nfull - pair + npairs - 1) / npairs : 0;
        half = -1;
        if (k < nw) {
            cand = pair + k * npairs;
            return true;
        }
        if (k == nw && pair < nhalves) {
            cand = nfull + pair / 2;
            half = pair & 1;
            return true;
        }
        return false;
    }
};

// `pair`/`npairs`: index of this cluster and number of clusters of the launch.  All 192 tensor-role threads of
// both CTAs call this; every OTHER thread of the two CTAs must have executed cluster_arrive() once.
// tmap_a: box 64 x 128 rows; tmap_b: box 64 x 128 rows (a half of the pair's B tile); tmap_bh: box 64 x 64 rows
// (a quarter: this CTA's share of a half tile) or null, in which case no tile is ever cut.
template <int STAGES>
__device__ __forceinline__ void gemm_role2(const CUtensorMap* __restrict__ tmap_a,
                                           const CUtensorMap* __restrict__ tmap_b, const GemmArgs g, uint8_t* smem,
                                           const int warp, const int lane, const int pair, const int npairs,
                                           const CUtensorMap* __restrict__ tmap_bh = nullptr) {
    using L = Gemm2Smem<STAGES>;
    constexpr uint32_t kTmemCols = 512;  // two 256-column accumulator buffers
    constexpr uint32_t kIdesc = umma_idesc_f16_f32(256, kGemm2BN);
    constexpr uint32_t kIdescHalf = umma_idesc_f16_f32(256, kGemm2BN / 2);

    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + L::kBarOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemSlotOffset);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kAbortOffset);

    SuperTileWalk256 walk;
    walk.init(g);
    PairTileList list;
    list.init(walk, g, npairs, tmap_bh != nullptr);
    const int kblocks = g.K / kGemmBK;
    TK_TRACE_ONLY(if (warp == 2 && lane == 0) { TK_TR(0, tk_gtime()); TK_TR(1, clock64()); } long long tr_a = 0, tr_b = 0;
                  bool tr_first = true;)

    // ---- set-up ----
    if (warp == 0 && lane == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);   // used in the leader only
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 8);  // used in the leader only: four epilogue warps of each CTA
        }
        fence_mbar_init();
        tma_prefetch_desc(tmap_a);
        tma_prefetch_desc(tmap_b);
    }
    __syncwarp();
    cluster_arrive();  // publishes the barrier initialisation to the peer
    cluster_wait();
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    named_bar_sync(kGemmBarrierId, kGemm2Threads);
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    TK_TRACE_ONLY(if (warp == 2 && lane == 0) TK_TR(2, clock64());)

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int cand, half;
            // The leader's wait number i (counted over the whole launch) sees the commit of K-block i - STAGES; the
            // first STAGES waits pass without any arrival, in both CTAs.  Every later one is passed on to the peer with
            // a relaxed arrive: no data travels with it, the MMAs' reads of the peer's stage ended before the commit
            // arrived here, and a release at cluster scope would stall this thread for a memory fence per K-block.
            int waits = 0;
            const uint32_t empty_peer0 = mapa_shared(empty_bar(0), 1u);
            for (int step = 0; ok && list.get(step, pair, npairs, cand, half); ++step) {
                int R, Cc;
                if (walk.mask(cand, R, Cc) == 0u) continue;
                // this CTA's share of the B tile: 128 of 256 rows, or 64 of the 128 rows of a half tile
                const uint32_t b_bytes = half < 0 ? L::kBBytes : L::kBBytes / 2;
                const int b_row = half < 0 ? Cc * kGemm2BN + static_cast<int>(rank) * (kGemm2BN / 2)
                                           : Cc * kGemm2BN + half * (kGemm2BN / 2) + static_cast<int>(rank) * (kGemm2BN / 4);
                for (int kb = 0; kb < kblocks; ++kb) {
                    TK_TRACE_ONLY(const long long tw = clock64();)
                    ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, g.status, DEV_TIMEOUT_EMPTY);
                    TK_TRACE_ONLY(tr_a += clock64() - tw;)
                    if (!ok) break;
                    if (leader && waits >= STAGES) mbar_arrive_cluster_relaxed(empty_peer0 + 8u * stage);
                    ++waits;
                    if (leader) mbar_arrive_expect_tx(full_bar(stage), 2u * (L::kABytes + b_bytes));
                    const uint32_t full_leader = mapa_shared(full_bar(stage), 0u);
                    const uint32_t a_dst = smem_base + stage * L::kStageBytes;
                    tma_load_tile_pair(a_dst, tmap_a, full_leader, kb * kGemmBK, R * 256 + static_cast<int>(rank) * 128, 0);
                    tma_load_tile_pair(a_dst + L::kABytes, half < 0 ? tmap_b : tmap_bh, full_leader, kb * kGemmBK, b_row, 0);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            // tail: the last commits arrive on this CTA's empty barriers asynchronously (from the leader's MMA thread);
            // do not let the CTA retire before they have landed and the MMAs have stopped reading its stages
            for (int s = 0; s < STAGES && ok; ++s) {
                ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, g.status, DEV_TIMEOUT_EMPTY);
                if (ok && leader && waits >= STAGES) mbar_arrive_cluster_relaxed(empty_peer0 + 8u * stage);
                ++waits;
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            TK_TR(13, tr_a);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader only) ----------------
        if (leader && lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t it = 0;
            bool ok = true;
            bool ready = false;  // the full barrier of `stage` was already seen complete
            int cand, half;
            for (int step = 0; ok && list.get(step, pair, npairs, cand, half); ++step) {
                int R, Cc;
                if (walk.mask(cand, R, Cc) == 0u) continue;
                const uint32_t as = it & 1u, aphase = (it >> 1) & 1u;
                TK_TRACE_ONLY(const long long tw = clock64();)
                ok = mbar_wait(tempty_bar(as), aphase ^ 1u, abort_flag, g.status, DEV_TIMEOUT_TMEM_EMPTY);
                TK_TRACE_ONLY(tr_b += clock64() - tw;)
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + as * kGemm2BN;
                const uint32_t idesc = half < 0 ? kIdesc : kIdescHalf;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!ready) {
                        TK_TRACE_ONLY(const long long tw = clock64();)
                        ok = mbar_wait(full_bar(stage), phase, abort_flag, g.status, DEV_TIMEOUT_FULL);
                        TK_TRACE_ONLY(if (tr_first) TK_TR(3, clock64()); else tr_a += clock64() - tw;)
                        if (!ok) break;
                    }
                    TK_TRACE_ONLY(tr_first = false;)
                    tc_fence_after_sync();
                    const uint32_t a_src = smem_base + stage * L::kStageBytes;
                    const uint64_t a_desc = umma_smem_desc_sw128(a_src);
                    const uint64_t b_desc = umma_smem_desc_sw128(a_src + L::kABytes);
                    const uint32_t this_empty = empty_bar(stage);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                    // probe the next stage now: the answer arrives while the MMAs below are being issued
                    ready = mbar_test_wait(full_bar(stage), phase);
#pragma unroll
                    for (int k = 0; k < kGemmBK / 16; ++k)
                        umma_f16_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, (kb > 0 || k != 0) ? 1u : 0u);
                    // the stage is free in both CTAs once these MMAs have read it (the leader's producer tells the peer)
                    umma_commit_pair(this_empty);
                }
                if (!ok) break;
                umma_commit_pair(tfull_bar(as));  // accumulator complete: tell both epilogues
                umma_commit_pair(mapa_shared(tfull_bar(as), 1u));
                ++it;
            }
            TK_TRACE_ONLY(TK_TR(4, clock64()); TK_TR(11, tr_a); TK_TR(12, tr_b);)
            // tail: the peer's epilogue warps arrive on this CTA's tempty barriers; wait until the last two accumulators
            // have been released by all eight warps before this CTA may retire
            for (int j = 0; j < 2 && ok; ++j) {
                const uint32_t as = it & 1u, aphase = (it >> 1) & 1u;
                ok = mbar_wait(tempty_bar(as), aphase ^ 1u, abort_flag, g.status, DEV_TIMEOUT_TMEM_EMPTY);
                ++it;
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
        const int q = warp & 3;  // the TMEM lane quarter this warp is allowed to read
        const int h = q >> 1;    // which 64-row half of this CTA's 128 rows those lanes are
        const uint32_t tempty_leader0 = mapa_shared(tempty_bar(0), 0u);
        uint32_t it = 0;
        bool ok = true;
        int cand, half;
        for (int step = 0; ok && list.get(step, pair, npairs, cand, half); ++step) {
            int R, Cc;
            const uint32_t m16 = walk.mask(cand, R, Cc);
            if (m16 == 0u) continue;
            const uint32_t as = it & 1u, aphase = (it >> 1) & 1u;
            ok = mbar_wait(tfull_bar(as), aphase, abort_flag, g.status, DEV_TIMEOUT_TMEM_FULL);
            if (!ok) break;
            tc_fence_after_sync();
            TK_TRACE_ONLY(const long long tw = clock64();)
            // the 4 mask bits of this warp's 64-row quarter of the pair tile
            uint32_t m = (m16 >> ((2 * static_cast<int>(rank) + h) * 4)) & 0xFu;
            const int row0 = R * 256 + static_cast<int>(rank) * 128 + q * 32;
            float* cbase = g.C + static_cast<size_t>(row0) * g.N + static_cast<size_t>(Cc) * kGemm2BN;
            int nchunks = kGemm2BN / 32;
            if (half >= 0) {  // a half tile: accumulator columns 0 .. 127 are C columns 128 half .. 128 half + 127
                cbase += half * (kGemm2BN / 2);
                m >>= 2 * half;
                nchunks = kGemm2BN / 64;
            }
            const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * kGemm2BN;
            float* stage = reinterpret_cast<float*>(smem + L::kEpiOffset) + (warp - 2) * (32 * L::kEpiPitch);
#pragma unroll 1
            for (int c = 0; c < nchunks; ++c) {
                if (((m >> (c >> 1)) & 1u) == 0u) continue;  // warp-uniform
                uint32_t r[32];
                tmem_ld_32x32(t_lane + c * 32, r);
                tmem_ld_wait();
                float4* srow = reinterpret_cast<float4*>(stage + lane * L::kEpiPitch);
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    float4 o;
                    o.x = g.alpha * __uint_as_float(r[4 * v + 0]);
                    o.y = g.alpha * __uint_as_float(r[4 * v + 1]);
                    o.z = g.alpha * __uint_as_float(r[4 * v + 2]);
                    o.w = g.alpha * __uint_as_float(r[4 * v + 3]);
                    srow[v] = o;
                }
                __syncwarp();
                float* cchunk = cbase + c * 32 + (lane & 7) * 4;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rr = 4 * i + (lane >> 3);
                    const float4 o = *reinterpret_cast<const float4*>(stage + rr * L::kEpiPitch + (lane & 7) * 4);
                    // C is written once and not read by this launch: streaming stores leave the operands in L2
                    __stcs(reinterpret_cast<float4*>(cchunk + static_cast<size_t>(rr) * g.N), o);
                }
                __syncwarp();
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster_relaxed(tempty_leader0 + 8u * as);
            ++it;
            TK_TRACE_ONLY(tr_a += clock64() - tw; if (warp == 2 && lane == 0) { TK_TR(5, tw); TK_TR(6, clock64()); TK_TR(7, tr_a);
                              TK_TR(8, static_cast<long long>(it)); })
        }
    }

    // ---- teardown: every role gets here, also after a bounded wait gave up ----
    __syncwarp();
    if (*abort_flag) __nanosleep(1000000u);  // let bulk copies still in flight land before smem is released
    tc_fence_before_sync();
    named_bar_sync(kGemmBarrierId, kGemm2Threads);
    tc_fence_after_sync();
    if (warp == 1) tmem_dealloc_pair(tmem_base, kTmemCols);
    TK_TRACE_ONLY(if (warp == 2 && lane == 0) { TK_TR(9, clock64()); TK_TR(10, tk_gtime()); })
}

}  // namespace tk
