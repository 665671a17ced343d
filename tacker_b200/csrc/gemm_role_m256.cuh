// tzgemm with 256 x 256 super-tiles: the solo kernel for large problems.
//
// Same contract as gemm_role (gemm_role.cuh): C = alpha * A * B^T on the 64x64 tiles of [start, end).  The
// 128 x 256 role is bound by the operand stream from L2 (768 KB per super-tile); here one CTA computes two
// 128-row halves against the same B tile, so a K-block of 64 brings 32 KB of A and 32 KB of B for twice the
// output: one third less operand traffic per flop.  The price is the tensor memory: two 128 x 256 fp32
// accumulators fill all 512 columns, so there is no second buffer and the epilogue of a super-tile does not
// overlap the MMAs of the next one (about 2 us against a main loop of 9 us and more); the TMA producer keeps
// prefetching the next super-tile meanwhile.
//
//   warp 0      TMA producer : A 256x64 and B 256x64 fp16 tiles, 128-byte swizzle, 3 stages of 64 KB
//   warp 1      MMA issuer   : per 16-deep step two tcgen05.mma 128x256x16 (upper / lower A half)
//   warps 2..5  epilogue     : warp w drains TMEM lanes 32 (w % 4) .. +31 of both accumulators
#pragma once
#include "gemm_role.cuh"

namespace tk {

constexpr int kGemm256Warps = 6;
constexpr int kGemm256Threads = kGemm256Warps * 32;
constexpr int kGemm256Stages = 3;
constexpr uint32_t kGemm256BarrierId = 1;

struct Gemm256Smem {
    static constexpr int kABytes = 256 * kGemmBK * 2;
    static constexpr int kBBytes = 256 * kGemmBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarOffset = kGemm256Stages * kStageBytes;
    static constexpr int kNumBars = 2 * kGemm256Stages + 2;  // full, empty per stage; accumulators full / empty
    static constexpr int kTmemSlotOffset = kBarOffset + kNumBars * 8;
    static constexpr int kAbortOffset = kTmemSlotOffset + 4;
    static constexpr int kEpiPitch = 36;
    static constexpr int kEpiWarpBytes = 32 * kEpiPitch * 4;
    static constexpr int kEpiOffset = ((kAbortOffset + 4 + 127) / 128) * 128;
    static constexpr int kBytes = kEpiOffset + 4 * kEpiWarpBytes;
};

// Super-tiles (256 x 256) that intersect [start, end); bit (rh * 4 + cb) of the mask = 64x64 sub-tile
// (row quarter rh, column quarter cb) is inside the range.
struct SuperTileWalk256 {
    int nt, mt, sc, r0, ncand, start, end;

    __host__ __device__ __forceinline__ void init(const GemmArgs& g) {
        nt = g.N / 64;
        mt = g.M / 64;
        sc = (g.N + 255) / 256;
        start = g.start < 0 ? 0 : g.start;
        end = g.end > nt * mt ? nt * mt : g.end;
        r0 = 0;
        ncand = 0;
        if (start >= end) return;
        r0 = (start / nt) / 4;
        const int r1 = ((end - 1) / nt) / 4;
        ncand = (r1 - r0 + 1) * sc;
    }
    __host__ __device__ __forceinline__ uint32_t mask(int cand, int& R, int& Cc) const {
        R = r0 + cand / sc;
        Cc = cand % sc;
        uint32_t m = 0;
#pragma unroll
        for (int rh = 0; rh < 4; ++rh) {
            const int row = 4 * R + rh;
            if (row >= mt) continue;
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) {
                const int col = 4 * Cc + cb;
                const int id = row * nt + col;
                if (col < nt && id >= start && id < end) m |= 1u << (rh * 4 + cb);
            }
        }
        return m;
    }
};

// all 192 threads of the CTA call this; tmap_a has a 64 x 256 box, tmap_b a 64 x 256 box
__device__ __forceinline__ void gemm_role_m256(const CUtensorMap* __restrict__ tmap_a,
                                               const CUtensorMap* __restrict__ tmap_b, const GemmArgs g, uint8_t* smem,
                                               const int warp, const int lane) {
    using L = Gemm256Smem;
    constexpr int STAGES = kGemm256Stages;
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kIdesc = umma_idesc_f16_f32(128, 256);

    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + L::kBarOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    const uint32_t tfull_bar = bar_base + 8u * (2 * STAGES);
    const uint32_t tempty_bar = bar_base + 8u * (2 * STAGES + 1);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemSlotOffset);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kAbortOffset);

    SuperTileWalk256 walk;
    walk.init(g);
    const int kblocks = g.K / kGemmBK;

    if (warp == 0 && lane == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tfull_bar, 1);
        mbar_init(tempty_bar, 4);  // one arrival per epilogue warp
        fence_mbar_init();
        tma_prefetch_desc(tmap_a);
        tma_prefetch_desc(tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    named_bar_sync(kGemm256BarrierId, kGemm256Threads);
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {  // ---------------- TMA producer ----------------
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int cand = blockIdx.x; cand < walk.ncand && ok; cand += gridDim.x) {
                int R, Cc;
                if (walk.mask(cand, R, Cc) == 0u) continue;
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, g.status, DEV_TIMEOUT_EMPTY);
                    if (!ok) break;
                    mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
                    const uint32_t a_dst = smem_base + stage * L::kStageBytes;
                    tma_load_tile(a_dst, tmap_a, full_bar(stage), kb * kGemmBK, R * 256, 0);
                    tma_load_tile(a_dst + L::kABytes, tmap_b, full_bar(stage), kb * kGemmBK, Cc * 256, 0);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            for (int s = 0; s < STAGES && ok; ++s) {  // tail: let the last commits land before the CTA retires
                ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, g.status, DEV_TIMEOUT_EMPTY);
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {  // ---------------- MMA issuer ----------------
            int stage = 0;
            uint32_t phase = 0, it = 0;
            bool ok = true;
            for (int cand = blockIdx.x; cand < walk.ncand && ok; cand += gridDim.x) {
                int R, Cc;
                if (walk.mask(cand, R, Cc) == 0u) continue;
                // both accumulators must have been drained by the epilogue of the previous super-tile
                ok = mbar_wait(tempty_bar, (it & 1u) ^ 1u, abort_flag, g.status, DEV_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after_sync();
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = mbar_wait(full_bar(stage), phase, abort_flag, g.status, DEV_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_src = smem_base + stage * L::kStageBytes;
                    const uint64_t a_lo = umma_smem_desc_sw128(a_src);
                    const uint64_t a_hi = umma_smem_desc_sw128(a_src + 128 * kGemmBK * 2);  // rows 128..255 of the A tile
                    const uint64_t b_desc = umma_smem_desc_sw128(a_src + L::kABytes);
#pragma unroll
                    for (int k = 0; k < kGemmBK / 16; ++k) {
                        const uint32_t acc = (kb | k) != 0 ? 1u : 0u;
                        umma_f16(tmem_base, a_lo + 2u * k, b_desc + 2u * k, kIdesc, acc);
                        umma_f16(tmem_base + 256u, a_hi + 2u * k, b_desc + 2u * k, kIdesc, acc);
                    }
                    umma_commit(empty_bar(stage));
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                umma_commit(tfull_bar);
                ++it;
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        uint32_t it = 0;
        bool ok = true;
        float* stage_buf = reinterpret_cast<float*>(smem + L::kEpiOffset) + (warp - 2) * (32 * L::kEpiPitch);
        for (int cand = blockIdx.x; cand < walk.ncand && ok; cand += gridDim.x) {
            int R, Cc;
            const uint32_t m = walk.mask(cand, R, Cc);
            if (m == 0u) continue;
            ok = mbar_wait(tfull_bar, it & 1u, abort_flag, g.status, DEV_TIMEOUT_TMEM_FULL);
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {  // accumulator 0 = rows 0..127, 1 = rows 128..255 of the super-tile
                const int rh = 2 * half + (q >> 1);  // 64-row quarter of the super-tile these lanes belong to
                const int row0 = R * 256 + half * 128 + q * 32;
                float* cbase = g.C + static_cast<size_t>(row0) * g.N + static_cast<size_t>(Cc) * 256;
                const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + half * 256;
#pragma unroll 1
                for (int c = 0; c < 8; ++c) {
                    if (((m >> (rh * 4 + (c >> 1))) & 1u) == 0u) continue;  // warp-uniform
                    uint32_t r[32];
                    tmem_ld_32x32(t_lane + c * 32, r);
                    tmem_ld_wait();
                    float4* srow = reinterpret_cast<float4*>(stage_buf + lane * L::kEpiPitch);
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
                        const float4 o =
                            *reinterpret_cast<const float4*>(stage_buf + rr * L::kEpiPitch + (lane & 7) * 4);
                        *reinterpret_cast<float4*>(cchunk + static_cast<size_t>(rr) * g.N) = o;
                    }
                    __syncwarp();
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar);
            ++it;
        }
    }

    __syncwarp();
    if (*abort_flag) __nanosleep(1000000u);
    tc_fence_before_sync();
    named_bar_sync(kGemm256BarrierId, kGemm256Threads);
    tc_fence_after_sync();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace tk
