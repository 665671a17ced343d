// tzgemm as a persistent, warp-specialised tcgen05 role.
//
// Computes C[M][N] (fp32, row-major) = alpha * A[M][K] (fp16, row-major) * B[N][K]^T (fp16, K
// contiguous) on the 64x64 output tiles whose row-major tile index lies in [start, end) --
// the operand layout, scaling and virtual-block unit of the reference kernel
// (src/gptb_kernel/tzgemm_kernel.cu:247-253, 284-287, 375, 391).  The reference computes each
// 64x64 tile with 4 wmma warps; here one CTA per SM owns 128 x BN super-tiles:
//
//   warp 0      TMA producer : A 128x64 and B BNx64 fp16 tiles, 128-byte swizzle, STAGES deep
//   warp 1      MMA issuer   : one thread issues tcgen05.mma 128xBNx16, accumulators in TMEM,
//                              two accumulator buffers so tile i+1 starts while tile i drains
//   warps 2..5  epilogue     : tcgen05.ld -> scale by alpha -> transpose through shared memory -> 128-bit
//                              global stores of whole rows, masked per 64x64 sub-tile so that exactly the
//                              tiles in [start, end) are written
//
// The six warps synchronise among themselves on named barrier 1 only, so other warps of the
// same CTA (the CUDA-core role of a fused kernel) are never involved.
#pragma once
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace tk {

constexpr int kGemmWarps = 6;
constexpr int kGemmThreads = kGemmWarps * 32;
constexpr int kGemmBM = 128;
constexpr int kGemmBK = 64;
constexpr uint32_t kGemmBarrierId = 1;

struct GemmArgs {
    float* C;
    int M, N, K;
    float alpha;
    int start, end;      // 64x64 tiles, row-major over (M/64) x (N/64)
    unsigned* status;    // device status word (bounded-wait expiries)
    int batch;           // independent problems of the same shape (1 for the reference's tzgemm)
    long long stride_c;  // elements between consecutive C matrices of a batch
    int l2_hints;        // 1: operand tiles are loaded with the evict-last L2 priority
    int splitk;          // > 1: K is cut into that many ranges handled by different CTAs, C += partial (red.add)
    // Implicit-GEMM convolution (CONV form of the role; 3 x 3, stride 1, padding 1): A is not a matrix in memory but
    // the zero-bordered NHWC fp16 image X[(H + 2)][(W + 2)][C].  GEMM row m stands for the pixel (m / (W + 2),
    // m % (W + 2)) of the bordered grid, so that K-block kb = (tap (i, j), channels c0 .. c0 + 63) of that row is the
    // image row m + i (W + 2) + j: every operand tile is one plain tile load at a shifted row.  The rows with
    // m % (W + 2) >= W are computed and dropped.  The epilogue adds the bias, applies the activation and writes fp16
    // into the bordered output image at row m + (W + 2) + 1.
    int conv_c;          // input channels (a multiple of 64); 0 in the plain GEMM
    int conv_w;          // image width W
    int conv_oh;         // output rows (= H)
    int conv_act;        // 0 none, 1 ReLU
    const float* conv_bias;  // [N] or null
    __half* conv_out;    // bordered fp16 output image [(H + 2)][(W + 2)][N]
    int test_skip_loads; // test hook (single-CTA role only): the producer issues no loads, so the MMA issuer's bounded
                         // wait for operand bytes runs out and the launch ends with DEV_TIMEOUT_FULL in the status word
};

// STAGED = the epilogue transposes through shared memory (coalesced row stores, 18 KB); the unstaged form writes
// 16 bytes per lane and row straight from registers and leaves that memory to a co-running role.
template <int BN, int STAGES, bool STAGED = true>
struct GemmSmem {
    static constexpr int kABytes = kGemmBM * kGemmBK * 2;
    static constexpr int kBBytes = BN * kGemmBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarOffset = STAGES * kStageBytes;
    static constexpr int kNumBars = 2 * STAGES + 4;
    static constexpr int kTmemSlotOffset = kBarOffset + kNumBars * 8;
    static constexpr int kAbortOffset = kTmemSlotOffset + 4;
    // epilogue staging: each of the four epilogue warps transposes its 32 x 32 chunk here so that its global
    // stores cover whole rows (pitch 36 floats keeps both the row-wise writes and the 4-row reads conflict free)
    static constexpr int kEpiPitch = 36;
    static constexpr int kEpiWarpBytes = 32 * kEpiPitch * 4;
    static constexpr int kEpiOffset = ((kAbortOffset + 4 + 127) / 128) * 128;
    // rounded so that whatever follows (a CUDA-core role's scratch) starts 128-byte aligned
    static constexpr int kBytes = kEpiOffset + (STAGED ? 4 * kEpiWarpBytes : 0);
};

// Enumeration of the super-tiles that intersect [start, end); identical in every role.
template <int BN>
struct SuperTileWalk {
    int nt;     // 64-wide tiles per C row
    int sc;     // super-tile columns
    int r0;     // first super-tile row touched
    int ncand;  // candidates = batch x touched super-tile rows x sc
    int per;    // candidates per batch entry (before the K split)
    int nsplit; // K ranges per super-tile
    int start, end, mt;

    __host__ __device__ __forceinline__ void init(const GemmArgs& g) {
        nt = g.N / 64;
        mt = g.M / 64;
        sc = (g.N + BN - 1) / BN;
        start = g.start < 0 ? 0 : g.start;
        end = g.end > nt * mt ? nt * mt : g.end;
        per = 1;
        nsplit = 1;
        if (start >= end) {
            ncand = 0;
            r0 = 0;
            return;
        }
        r0 = (start / nt) / 2;
        const int r1 = ((end - 1) / nt) / 2;
        per = (r1 - r0 + 1) * sc;
        nsplit = g.splitk > 1 ? g.splitk : 1;
        ncand = per * (g.batch > 0 ? g.batch : 1) * nsplit;
    }

    // K-block range [kb0, kb1) of candidate `cand` (the split index is the fastest-varying part of it)
    __host__ __device__ __forceinline__ void krange(int cand, int kblocks, int& kb0, int& kb1) const {
        const int sp = cand % nsplit;
        kb0 = static_cast<int>(static_cast<long long>(kblocks) * sp / nsplit);
        kb1 = static_cast<int>(static_cast<long long>(kblocks) * (sp + 1) / nsplit);
    }

    // bit (h * (BN/64) + cb) set <=> sub-tile (64-row half h, 64-column block cb) is in range
    __host__ __device__ __forceinline__ uint32_t mask(int cand, int& R, int& Cc, int& b) const {
        cand /= nsplit;
        b = cand / per;
        cand -= b * per;
        R = r0 + cand / sc;
        Cc = cand % sc;
        uint32_t m = 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = 2 * R + h;
            if (row >= mt) continue;
#pragma unroll
            for (int cb = 0; cb < BN / 64; ++cb) {
                const int col = Cc * (BN / 64) + cb;
                const int id = row * nt + col;
                if (col < nt && id >= start && id < end) m |= 1u << (h * (BN / 64) + cb);
            }
        }
        return m;
    }
};

// `warp` is the warp index inside the role (0..5); all 192 threads of the role must call this.
// CONV: the implicit-GEMM convolution described at GemmArgs (tmap_a then describes the bordered image as
// {C, (H + 2)(W + 2)} with a 64 x 128 box); needs STAGED.
template <int BN, int STAGES, bool STAGED = true, bool CONV = false>
__device__ __forceinline__ void gemm_role(const CUtensorMap* __restrict__ tmap_a,
                                          const CUtensorMap* __restrict__ tmap_b, const GemmArgs g,
                                          uint8_t* smem, const int warp, const int lane) {
    using L = GemmSmem<BN, STAGES, STAGED>;
    constexpr uint32_t kTmemCols = 2 * BN;  // two accumulator buffers (256 or 512: powers of two)
    constexpr uint32_t kIdesc = umma_idesc_f16_f32(kGemmBM, BN);

    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + L::kBarOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemSlotOffset);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kAbortOffset);

    SuperTileWalk<BN> walk;
    walk.init(g);
    const int kblocks = g.K / kGemmBK;

    // ---- set-up: barriers (warp 0) and TMEM (warp 1) ----
    if (warp == 0 && lane == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4);  // one arrival per epilogue warp
        }
        fence_mbar_init();
        tma_prefetch_desc(tmap_a);
        tma_prefetch_desc(tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    named_bar_sync(kGemmBarrierId, kGemmThreads);
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint64_t keep = l2_policy_evict_last();
            for (int cand = blockIdx.x; cand < walk.ncand && ok; cand += gridDim.x) {
                int R, Cc, b;
                if (walk.mask(cand, R, Cc, b) == 0u) continue;
                int kb0, kb1;
                walk.krange(cand, kblocks, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb) {
                    ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, g.status, DEV_TIMEOUT_EMPTY);
                    if (!ok) break;
                    if (g.test_skip_loads) continue;  // nothing will ever arrive on the full barrier
                    mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
                    const uint32_t a_dst = smem_base + stage * L::kStageBytes;
                    int ax = kb * kGemmBK, ay = R * kGemmBM;
                    if (CONV) {  // K-block = one filter tap x 64 channels: the image rows shifted by the tap
                        const int tap = ax / g.conv_c;
                        ax -= tap * g.conv_c;
                        ay += (tap / 3) * (g.conv_w + 2) + tap % 3;
                    }
                    if (g.l2_hints) {
                        tma_load_tile_hint(a_dst, tmap_a, full_bar(stage), ax, ay, b, keep);
                        tma_load_tile_hint(a_dst + L::kABytes, tmap_b, full_bar(stage), kb * kGemmBK, Cc * BN, b, keep);
                    } else {
                        tma_load_tile(a_dst, tmap_a, full_bar(stage), ax, ay, b);
                        tma_load_tile(a_dst + L::kABytes, tmap_b, full_bar(stage), kb * kGemmBK, Cc * BN, b);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            // tail: the last commits arrive on the empty barriers asynchronously; do not let the
            // CTA retire (and its shared memory be handed to another CTA) before they have landed
            for (int s = 0; s < STAGES && ok; ++s) {
                ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, g.status, DEV_TIMEOUT_EMPTY);
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t it = 0;
            bool ok = true;
            for (int cand = blockIdx.x; cand < walk.ncand && ok; cand += gridDim.x) {
                int R, Cc, b;
                if (walk.mask(cand, R, Cc, b) == 0u) continue;
                const uint32_t as = it & 1u, aphase = (it >> 1) & 1u;
                ok = mbar_wait(tempty_bar(as), aphase ^ 1u, abort_flag, g.status, DEV_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + as * BN;
                int kb0, kb1;
                walk.krange(cand, kblocks, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb) {
                    ok = mbar_wait(full_bar(stage), phase, abort_flag, g.status, DEV_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_src = smem_base + stage * L::kStageBytes;
                    const uint64_t a_desc = umma_smem_desc_sw128(a_src);
                    const uint64_t b_desc = umma_smem_desc_sw128(a_src + L::kABytes);
#pragma unroll
                    for (int k = 0; k < kGemmBK / 16; ++k) {
                        // 16 fp16 = 32 bytes further along K inside the swizzled row: +2 in units of 16 B
                        umma_f16(d_tmem, a_desc + 2u * k, b_desc + 2u * k, kIdesc, (kb > kb0 || k != 0) ? 1u : 0u);
                    }
                    umma_commit(empty_bar(stage));  // frees the stage once these UMMAs have read it
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                umma_commit(tfull_bar(as));  // accumulator complete
                ++it;
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        const int q = warp & 3;  // the TMEM lane quarter this warp is allowed to read
        const int h = q >> 1;    // which 64-row half of the super-tile those lanes are
        uint32_t it = 0;
        bool ok = true;
        for (int cand = blockIdx.x; cand < walk.ncand && ok; cand += gridDim.x) {
            int R, Cc, b;
            const uint32_t m = walk.mask(cand, R, Cc, b);
            if (m == 0u) continue;
            const uint32_t as = it & 1u, aphase = (it >> 1) & 1u;
            ok = mbar_wait(tfull_bar(as), aphase, abort_flag, g.status, DEV_TIMEOUT_TMEM_FULL);
            if (!ok) break;
            tc_fence_after_sync();
            // this warp's 32 rows of the super-tile; lane `lane` holds row (row0 + lane) after the TMEM load and
            // writes rows row0 + 4i + lane/8, columns 4 (lane % 8) .. +3 after the transpose
            const int row0 = R * kGemmBM + q * 32;
            float* cbase = g.C + static_cast<size_t>(b) * g.stride_c + static_cast<size_t>(row0) * g.N +
                           static_cast<size_t>(Cc) * BN;
            const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * BN;
            float* stage = reinterpret_cast<float*>(smem + L::kEpiOffset) + (warp - 2) * (32 * L::kEpiPitch);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                if (((m >> (h * (BN / 64) + (c >> 1))) & 1u) == 0u) continue;  // warp-uniform
                uint32_t r[32];
                tmem_ld_32x32(t_lane + c * 32, r);
                tmem_ld_wait();
                if (STAGED) {
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
                    if (CONV) {
                        // bias + activation + fp16, into the bordered output image; rows that stand for border pixels
                        // of the enumeration (or lie below the image) are dropped, so the border stays zero
                        const int col = Cc * BN + c * 32 + (lane & 7) * 4;
                        float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (g.conv_bias) bv = __ldg(reinterpret_cast<const float4*>(g.conv_bias + col));
                        const int wp = g.conv_w + 2;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rr = 4 * i + (lane >> 3);
                            const int m = row0 + rr;
                            const int oh = m / wp, ow = m - oh * wp;
                            if (ow >= g.conv_w || oh >= g.conv_oh) continue;
                            float4 o = *reinterpret_cast<const float4*>(stage + rr * L::kEpiPitch + (lane & 7) * 4);
                            o.x += bv.x, o.y += bv.y, o.z += bv.z, o.w += bv.w;
                            if (g.conv_act == 1) {
                                o.x = fmaxf(o.x, 0.f), o.y = fmaxf(o.y, 0.f), o.z = fmaxf(o.z, 0.f), o.w = fmaxf(o.w, 0.f);
                            }
                            const __half2 lo = __floats2half2_rn(o.x, o.y), hi = __floats2half2_rn(o.z, o.w);
                            uint2 pk;
                            pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                            pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                            *reinterpret_cast<uint2*>(g.conv_out + static_cast<size_t>(m + wp + 1) * g.N + col) = pk;
                        }
                        __syncwarp();
                        continue;
                    }
                    float* cchunk = cbase + c * 32 + (lane & 7) * 4;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = 4 * i + (lane >> 3);
                        const float4 o = *reinterpret_cast<const float4*>(stage + rr * L::kEpiPitch + (lane & 7) * 4);
                        float* dstp = cchunk + static_cast<size_t>(rr) * g.N;
                        if (g.splitk > 1) red_add_v4(dstp, o);
                        else *reinterpret_cast<float4*>(dstp) = o;
                    }
                    __syncwarp();
                } else {
                    float4* dst = reinterpret_cast<float4*>(cbase + static_cast<size_t>(lane) * g.N + c * 32);
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        float4 o;
                        o.x = g.alpha * __uint_as_float(r[4 * v + 0]);
                        o.y = g.alpha * __uint_as_float(r[4 * v + 1]);
                        o.z = g.alpha * __uint_as_float(r[4 * v + 2]);
                        o.w = g.alpha * __uint_as_float(r[4 * v + 3]);
                        if (g.splitk > 1) red_add_v4(reinterpret_cast<float*>(dst + v), o);
                        else dst[v] = o;
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(as));
            ++it;
        }
    }

    // ---- teardown: every role gets here, also after a bounded wait gave up ----
    __syncwarp();
    if (*abort_flag) __nanosleep(1000000u);  // let bulk copies still in flight land before smem is released
    tc_fence_before_sync();
    named_bar_sync(kGemmBarrierId, kGemmThreads);
    tc_fence_after_sync();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace tk
