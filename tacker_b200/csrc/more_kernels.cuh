// Kernels and launchers of the sgemm / lbm / fft / cutcp roles (cd_roles_more.cuh): one solo kernel each and one
// fused kernel each with tzgemm as the tensor role.  Included by tacker_b200.cu after host_launch.cuh.
#pragma once
#include "cd_roles_more.cuh"
#include "host_launch.cuh"

namespace tk {

// -------------------------------------------------------------------------------------------------
// solo kernels
// -------------------------------------------------------------------------------------------------
// 16 warps of 32 accumulators per lane with a ring of S slots each: one CTA per SM
template <int S>
__global__ void __launch_bounds__(512, 1) sgemm_kernel(const SgemmArgs g) {
    extern __shared__ __align__(16) uint8_t more_smem[];
    __shared__ int item_counter;
    if (threadIdx.x == 0) item_counter = 0;
    __syncthreads();
    sgemm_role<S>(g, more_smem, &item_counter, threadIdx.x >> 5, blockDim.x >> 5, threadIdx.x & 31, blockIdx.x, gridDim.x);
}

// the passes that precede a launch with split work items: C *= 2 (sgemm), regions = 0 (cutcp)
__global__ void __launch_bounds__(256) sgemm_scale_c_kernel(const SgemmArgs g) {
    sgemm_scale_c(g, threadIdx.x, blockDim.x, blockIdx.x, gridDim.x);
}
__global__ void __launch_bounds__(128) cutcp_zero_kernel(const CutcpArgs g) {
    cutcp_zero(g, threadIdx.x, blockDim.x, blockIdx.x, gridDim.x);
}

__global__ void __launch_bounds__(512, 2) lbm_kernel(const LbmArgs g) {
    __shared__ int item_counter;
    if (threadIdx.x == 0) item_counter = 0;
    __syncthreads();
    lbm_role(g, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
}

__global__ void __launch_bounds__(512, 2) fft_kernel(const FftArgs g) {
    extern __shared__ __align__(16) uint8_t more_smem[];
    fft_role(g, more_smem, threadIdx.x, blockDim.x, blockIdx.x, gridDim.x, 0);
}

__global__ void __launch_bounds__(512, 2) cutcp_kernel(const CutcpArgs g) {
    __shared__ int item_counter;
    if (threadIdx.x == 0) item_counter = 0;
    __syncthreads();
    cutcp_role(g, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
}

// {dx, dy, dz} triples -> the int4 table the cutcp role reads
__global__ void cutcp_pack_nbr_kernel(const int* __restrict__ xyz, int n, int4* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = make_int4(xyz[3 * i], xyz[3 * i + 1], xyz[3 * i + 2], 0);
}

// -------------------------------------------------------------------------------------------------
// fused kernels: warps 0..5 the tensor role (128-wide super-tiles, 4 stages: 146 KB; CONV = the implicit-GEMM
// convolution), the remaining warps the CUDA-core role, whose shared memory (sgemm rings, FFT buffers) lies behind it
// -------------------------------------------------------------------------------------------------
constexpr int kMoreBN = 128, kMoreStages = 4;
constexpr int kMaxMixThreadsSgemm = 576;  // 192 + 12 warps at up to 113 registers
constexpr int kSgemmSlotsSolo = 4;

template <int S, bool CONV = false>
__global__ void __launch_bounds__(kMaxMixThreadsSgemm, 1)
mix_sgemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmArgs g,
                 const SgemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int item_counter;
    const int warp = threadIdx.x >> 5;
    uint8_t* smem = align_smem_1024(smem_raw);
    if (warp < kGemmWarps) {
        gemm_role<kMoreBN, kMoreStages, true, CONV>(&tmap_a, &tmap_b, g, smem, warp, threadIdx.x & 31);
    } else {
        cd_role_begin(&item_counter);
        sgemm_role<S>(a, smem + GemmSmem<kMoreBN, kMoreStages>::kBytes, &item_counter, warp - kGemmWarps,
                      (blockDim.x >> 5) - kGemmWarps, threadIdx.x & 31, blockIdx.x, gridDim.x);
    }
}

template <bool CONV = false>
__global__ void __launch_bounds__(kMaxMixThreadsSfu, 1)
mix_lbm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmArgs g,
               const LbmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int item_counter;
    const int warp = threadIdx.x >> 5;
    if (warp < kGemmWarps) {
        gemm_role<kMoreBN, kMoreStages, true, CONV>(&tmap_a, &tmap_b, g, align_smem_1024(smem_raw), warp, threadIdx.x & 31);
    } else {
        cd_role_begin(&item_counter);
        lbm_role(a, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
    }
}

template <bool CONV = false>
__global__ void __launch_bounds__(kMaxMixThreadsSfu, 1)
mix_fft_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmArgs g,
               const FftArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5;
    uint8_t* smem = align_smem_1024(smem_raw);
    if (warp < kGemmWarps) {
        gemm_role<kMoreBN, kMoreStages, true, CONV>(&tmap_a, &tmap_b, g, smem, warp, threadIdx.x & 31);
    } else {
        fft_role(a, smem + GemmSmem<kMoreBN, kMoreStages>::kBytes, threadIdx.x - kGemmThreads, blockDim.x - kGemmThreads,
                 blockIdx.x, gridDim.x, kCdBarrierId);
    }
}

template <bool CONV = false>
__global__ void __launch_bounds__(kMaxMixThreadsSfu, 1)
mix_cutcp_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmArgs g,
                 const CutcpArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int item_counter;
    const int warp = threadIdx.x >> 5;
    if (warp < kGemmWarps) {
        gemm_role<kMoreBN, kMoreStages, true, CONV>(&tmap_a, &tmap_b, g, align_smem_1024(smem_raw), warp, threadIdx.x & 31);
    } else {
        cd_role_begin(&item_counter);
        cutcp_role(a, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
    }
}

// -------------------------------------------------------------------------------------------------
// the same pairs with the tensor role on CTA pairs (gemm_role2; launches that hold at least a wave of pair tiles):
// the CUDA-core role is unchanged and works per CTA, its threads only arrive at the cluster barrier the tensor roles
// of the pair wait on at start-up.  sgemm and fft keep their shared memory behind four operand stages, lbm and cutcp
// need none and leave the tensor role its six.
// -------------------------------------------------------------------------------------------------
constexpr int kMorePairStagesSmem = 4;

template <int S>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMaxMixThreadsSgemm, 1)
mix_sgemm2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmArgs g,
                  const SgemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int item_counter;
    const int warp = threadIdx.x >> 5;
    uint8_t* smem = align_smem_1024(smem_raw);
    if (warp < kGemmWarps) {
        gemm_role2<kMorePairStagesSmem>(&tmap_a, &tmap_b, g, smem, warp, threadIdx.x & 31, blockIdx.x >> 1, gridDim.x >> 1);
    } else {
        cluster_arrive();
        cd_role_begin(&item_counter);
        sgemm_role<S>(a, smem + Gemm2Smem<kMorePairStagesSmem>::kBytes, &item_counter, warp - kGemmWarps,
                      (blockDim.x >> 5) - kGemmWarps, threadIdx.x & 31, blockIdx.x, gridDim.x);
    }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMaxMixThreadsSfu, 1)
mix_lbm2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmArgs g,
                const LbmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int item_counter;
    const int warp = threadIdx.x >> 5;
    if (warp < kGemmWarps) {
        gemm_role2<kStagesPair>(&tmap_a, &tmap_b, g, align_smem_1024(smem_raw), warp, threadIdx.x & 31, blockIdx.x >> 1,
                                gridDim.x >> 1);
    } else {
        cluster_arrive();
        cd_role_begin(&item_counter);
        lbm_role(a, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
    }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMaxMixThreadsSfu, 1)
mix_fft2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmArgs g,
                const FftArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5;
    uint8_t* smem = align_smem_1024(smem_raw);
    if (warp < kGemmWarps) {
        gemm_role2<kMorePairStagesSmem>(&tmap_a, &tmap_b, g, smem, warp, threadIdx.x & 31, blockIdx.x >> 1, gridDim.x >> 1);
    } else {
        cluster_arrive();
        fft_role(a, smem + Gemm2Smem<kMorePairStagesSmem>::kBytes, threadIdx.x - kGemmThreads, blockDim.x - kGemmThreads,
                 blockIdx.x, gridDim.x, kCdBarrierId);
    }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMaxMixThreadsSfu, 1)
mix_cutcp2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmArgs g,
                  const CutcpArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int item_counter;
    const int warp = threadIdx.x >> 5;
    if (warp < kGemmWarps) {
        gemm_role2<kStagesPair>(&tmap_a, &tmap_b, g, align_smem_1024(smem_raw), warp, threadIdx.x & 31, blockIdx.x >> 1,
                                gridDim.x >> 1);
    } else {
        cluster_arrive();
        cd_role_begin(&item_counter);
        cutcp_role(a, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
    }
}

// -------------------------------------------------------------------------------------------------
// argument parsing (reference argument order; p = the CUDA-core list, geometry ints at n_solo .. n_solo + 5)
// -------------------------------------------------------------------------------------------------
static bool misaligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

// sgemm: A, B, C, M, N, K (src/gptb_kernel/sgemm_kernel.cu:3-5)
static int parse_sgemm(void** p, int i_start, int i_end, SgemmArgs* g) {
    g->A = arg<const float*>(p, 0);
    g->B = arg<const float*>(p, 1);
    g->C = arg<float*>(p, 2);
    g->M = arg<int>(p, 3);
    g->N = arg<int>(p, 4);
    g->K = arg<int>(p, 5);
    g->gx = arg<int>(p, 6);
    g->gy = arg<int>(p, 7);
    const int bdx = arg<int>(p, 9), bdy = arg<int>(p, 10);
    g->start = arg<int>(p, i_start);
    g->end = arg<int>(p, i_end);
    g->k_per_item = 0;
    g->coop = 0;
    if (g->M <= 0 || g->N <= 0 || g->K <= 0 || g->start < 0) return TK_ERR_ARGS;
    if (g->M % 128 || g->N % 16) return TK_ERR_SHAPE;
    if (g->gx != g->M / 128 || g->gy != g->N / 16 || bdx != 16 || bdy != 8) return TK_ERR_SHAPE;
    if (g->end > g->gx * g->gy) g->end = g->gx * g->gy;
    if (g->start < g->end && (!g->A || !g->B || !g->C)) return TK_ERR_ARGS;
    if (misaligned16(g->A) || misaligned16(g->B) || misaligned16(g->C)) return TK_ERR_ALIGN;
    return TK_OK;
}

// lbm: srcGrid, dstGrid; the grid is (ny, nz), the block nx threads (src/ori_kernel/lbm_kernel.cu:209-213)
static int parse_lbm(void** p, int i_start, int i_end, LbmArgs* g) {
    g->src = arg<const float*>(p, 0);
    g->dst = arg<float*>(p, 1);
    g->ny = arg<int>(p, 2);
    g->nz = arg<int>(p, 3);
    g->nx = arg<int>(p, 5);
    g->start = arg<int>(p, i_start);
    g->end = arg<int>(p, i_end);
    if (g->nx <= 0 || g->ny <= 0 || g->nz <= 0 || g->start < 0) return TK_ERR_ARGS;
    if (g->nx % 32) return TK_ERR_SHAPE;
    if (g->end > g->ny * g->nz) g->end = g->ny * g->nz;
    if (g->start < g->end && (!g->src || !g->dst)) return TK_ERR_ARGS;
    if ((reinterpret_cast<uintptr_t>(g->src) & 3u) || (reinterpret_cast<uintptr_t>(g->dst) & 3u)) return TK_ERR_ALIGN;
    return TK_OK;
}

// fft: data; the grid is the batch, the block 128 threads (src/ori_kernel/fft_kernel.cu:107-110)
static int parse_fft(void** p, int i_start, int i_end, FftArgs* g) {
    g->data = arg<float2*>(p, 0);
    g->nfft = arg<int>(p, 1);
    const int bdx = arg<int>(p, 4);
    g->start = arg<int>(p, i_start);
    g->end = arg<int>(p, i_end);
    if (g->nfft <= 0 || g->start < 0) return TK_ERR_ARGS;
    if (bdx != 128) return TK_ERR_SHAPE;
    if (g->end > g->nfft) g->end = g->nfft;
    if (g->start < g->end && !g->data) return TK_ERR_ARGS;
    if (reinterpret_cast<uintptr_t>(g->data) & 7u) return TK_ERR_ALIGN;
    return TK_OK;
}

// cutcp: binDim_x, binDim_y, binZeroAddr, h, cutoff2, inv_cutoff2, regionZeroAddr, zRegionIndex_t
// (src/gptb_kernel/cutcp_kernel.cu:12-31), then the neighbour table and its length, which the reference keeps in
// __constant__ symbols (src/ori_kernel/cutcp_kernel.cu:12-13); the grid is the regions, the block (8, 2, 8)
static int parse_cutcp(void** p, int i_start, int i_end, CutcpArgs* g) {
    g->bin_dim_x = arg<int>(p, 0);
    g->bin_dim_y = arg<int>(p, 1);
    g->bins = arg<const float4*>(p, 2);
    g->h = arg<float>(p, 3);
    g->cutoff2 = arg<float>(p, 4);
    g->inv_cutoff2 = arg<float>(p, 5);
    g->regions = arg<float*>(p, 6);
    g->nbr = arg<const int4*>(p, 8);
    g->nbrlen = arg<int>(p, 9);
    g->gx = arg<int>(p, 10);
    g->gy = arg<int>(p, 11);
    g->gz = arg<int>(p, 12);
    const int bdx = arg<int>(p, 13), bdy = arg<int>(p, 14), bdz = arg<int>(p, 15);
    g->start = arg<int>(p, i_start);
    g->end = arg<int>(p, i_end);
    g->nbr_per_item = 0;
    if (g->bin_dim_x <= 0 || g->bin_dim_y <= 0 || g->gx <= 0 || g->gy <= 0 || g->gz <= 0 || g->nbrlen < 0 || g->start < 0)
        return TK_ERR_ARGS;
    if (bdx != 8 || bdy != 2 || bdz != 8) return TK_ERR_SHAPE;
    if (g->end > g->gx * g->gy * g->gz) g->end = g->gx * g->gy * g->gz;
    if (g->start < g->end && (!g->bins || !g->regions || (g->nbrlen > 0 && !g->nbr))) return TK_ERR_ARGS;
    if (misaligned16(g->bins) || misaligned16(g->nbr) || misaligned16(g->regions)) return TK_ERR_ALIGN;
    return TK_OK;
}

// -------------------------------------------------------------------------------------------------
// solo launches
// -------------------------------------------------------------------------------------------------
// k-steps / neighbour bins per work item: about eight items per launched warp when the launch has few blocks
// (option > 0: that many; 0: never split, the reference's order of additions; -1: by this rule)
static int sgemm_split_for(const SgemmArgs& g, long long warps) {
    if (g_opt.sgemm_split == 0) return 0;
    if (g_opt.sgemm_split > 0) return (g_opt.sgemm_split + 7) / 8 * 8;
    return cd_pick_split(2ll * (g.end - g.start), warps, g.K, 64);
}
static int cutcp_split_for(const CutcpArgs& g, long long warps) {
    if (g_opt.cutcp_split == 0) return 0;
    if (g_opt.cutcp_split > 0) return g_opt.cutcp_split;
    return cd_pick_split(4ll * (g.end - g.start), warps, g.nbrlen, 8);
}
// the pass a launch with split items needs first (same stream, so it is complete when the items start adding)
static int sgemm_prepass(const SgemmArgs& g, cudaStream_t st) {
    if (g.k_per_item <= 0) return TK_OK;
    const int blocks = g.end - g.start;
    sgemm_scale_c_kernel<<<blocks < 1184 ? blocks : 1184, 256, 0, st>>>(g);
    return launch_error("sgemm_scale_c_kernel launch");
}
static int cutcp_prepass(const CutcpArgs& g, cudaStream_t st) {
    if (g.nbr_per_item <= 0 || g.nbr_per_item >= g.nbrlen) return TK_OK;
    const int blocks = g.end - g.start;
    cutcp_zero_kernel<<<blocks < 1184 ? blocks : 1184, 128, 0, st>>>(g);
    return launch_error("cutcp_zero_kernel launch");
}

static int run_sgemm(SgemmArgs g, unsigned grid0, unsigned block0, cudaStream_t st) {
    if (g.start >= g.end) return TK_OK;
    const unsigned threads = cd_threads(block0, 32, 512);
    if (threads == 0) return TK_ERR_LAUNCH_CONFIG;
    const int nw = static_cast<int>(threads / 32);
    // a range that gives every CTA at least one full group of column blocks: the warps of a CTA share the A slices
    // (sgemm_group; option 2 forces the form for any range with at least half a group per row block)
    const long long nblocks = g.end - g.start;
    g.coop = nw >= 8 && nblocks * 2 >= static_cast<long long>(g.gx) * nw &&
             (g_opt.sgemm_coop == 2 || (g_opt.sgemm_coop == 1 && nblocks >= static_cast<long long>(grid0) * nw));
    if (g.coop) {
        const int nby = (g.end + g.gx - 1) / g.gx - g.start / g.gx;  // column blocks the range touches
        const long long groups = static_cast<long long>(g.gx) * ((nby + nw - 1) / nw);
        g.k_per_item = g_opt.sgemm_split == 0 ? 0
                       : g_opt.sgemm_split > 0 ? (g_opt.sgemm_split + 7) / 8 * 8
                                               : cd_pick_split(groups, grid0, g.K, 64);
    } else {
        g.k_per_item = sgemm_split_for(g, static_cast<long long>(grid0) * nw);
    }
    int prc = sgemm_prepass(g, st);
    if (prc != TK_OK) return prc;
    const int smem = sgemm_role_smem(static_cast<int>(threads / 32), kSgemmSlotsSolo);
    int rc = enable_smem(sgemm_kernel<kSgemmSlotsSolo>, smem);
    if (rc != TK_OK) return rc;
    sgemm_kernel<kSgemmSlotsSolo><<<grid0, threads, smem, st>>>(g);
    return launch_error("sgemm_kernel launch");
}

static int run_lbm(const LbmArgs& g, unsigned grid0, unsigned block0, cudaStream_t st) {
    if (g.start >= g.end) return TK_OK;
    const unsigned threads = cd_threads(block0, 32, 512);
    if (threads == 0) return TK_ERR_LAUNCH_CONFIG;
    lbm_kernel<<<grid0, threads, 0, st>>>(g);
    return launch_error("lbm_kernel launch");
}

static int run_fft(const FftArgs& g, unsigned grid0, unsigned block0, cudaStream_t st) {
    if (g.start >= g.end) return TK_OK;
    const unsigned threads = cd_threads(block0, 32, 512);
    if (threads == 0) return TK_ERR_LAUNCH_CONFIG;
    fft_kernel<<<grid0, threads, fft_role_smem(static_cast<int>(threads / 32)), st>>>(g);
    return launch_error("fft_kernel launch");
}

static int run_cutcp(CutcpArgs g, unsigned grid0, unsigned block0, cudaStream_t st) {
    if (g.start >= g.end) return TK_OK;
    const unsigned threads = cd_threads(block0, 32, 512);
    if (threads == 0) return TK_ERR_LAUNCH_CONFIG;
    g.nbr_per_item = cutcp_split_for(g, static_cast<long long>(grid0) * (threads / 32));
    int prc = cutcp_prepass(g, st);
    if (prc != TK_OK) return prc;
    cutcp_kernel<<<grid0, threads, 0, st>>>(g);
    return launch_error("cutcp_kernel launch");
}

// -------------------------------------------------------------------------------------------------
// fused launches
// -------------------------------------------------------------------------------------------------
enum MoreKind { MORE_SGEMM, MORE_LBM, MORE_FFT, MORE_CUTCP };

struct MoreCall {
    MoreKind kind;
    SgemmArgs sg;
    LbmArgs lb;
    FftArgs ff;
    CutcpArgs cc;
    bool empty() const {
        switch (kind) {
            case MORE_SGEMM: return sg.start >= sg.end;
            case MORE_LBM: return lb.start >= lb.end;
            case MORE_FFT: return ff.start >= ff.end;
            default: return cc.start >= cc.end;
        }
    }
};

static int run_more_solo(const MoreCall& m, unsigned grid0, unsigned threads, cudaStream_t st) {
    switch (m.kind) {
        case MORE_SGEMM: return run_sgemm(m.sg, grid0, threads, st);
        case MORE_LBM: return run_lbm(m.lb, grid0, threads, st);
        case MORE_FFT: return run_fft(m.ff, grid0, threads, st);
        default: return run_cutcp(m.cc, grid0, threads, st);
    }
}

template <bool CONV>
static int launch_mix_more_kernels(const GemmCall& c, const MoreCall& m, const CUtensorMap& ta, const CUtensorMap& tb,
                                   unsigned ctas, unsigned threads, unsigned cdt, cudaStream_t st) {
    constexpr int kGemmBytes = GemmSmem<kMoreBN, kMoreStages>::kBytes + 1024;
    int rc = TK_OK;
    switch (m.kind) {
        case MORE_SGEMM: {  // the deepest ring that fits behind the tensor role's stages
            const int nw = static_cast<int>(cdt / 32), room = kMaxDynSmem - kGemmBytes;
            if (sgemm_role_smem(nw, 4) <= room) {
                const int smem = kGemmBytes + sgemm_role_smem(nw, 4);
                if ((rc = enable_smem(mix_sgemm_kernel<4, CONV>, smem)) != TK_OK) return rc;
                mix_sgemm_kernel<4, CONV><<<ctas, threads, smem, st>>>(ta, tb, c.g, m.sg);
            } else if (sgemm_role_smem(nw, 3) <= room) {
                const int smem = kGemmBytes + sgemm_role_smem(nw, 3);
                if ((rc = enable_smem(mix_sgemm_kernel<3, CONV>, smem)) != TK_OK) return rc;
                mix_sgemm_kernel<3, CONV><<<ctas, threads, smem, st>>>(ta, tb, c.g, m.sg);
            } else {
                const int smem = kGemmBytes + sgemm_role_smem(nw, 2);
                if ((rc = enable_smem(mix_sgemm_kernel<2, CONV>, smem)) != TK_OK) return rc;
                mix_sgemm_kernel<2, CONV><<<ctas, threads, smem, st>>>(ta, tb, c.g, m.sg);
            }
            break;
        }
        case MORE_LBM:
            if ((rc = enable_smem(mix_lbm_kernel<CONV>, kGemmBytes)) != TK_OK) return rc;
            mix_lbm_kernel<CONV><<<ctas, threads, kGemmBytes, st>>>(ta, tb, c.g, m.lb);
            break;
        case MORE_FFT: {
            const int smem = kGemmBytes + fft_role_smem(static_cast<int>(cdt / 32));
            if ((rc = enable_smem(mix_fft_kernel<CONV>, smem)) != TK_OK) return rc;
            mix_fft_kernel<CONV><<<ctas, threads, smem, st>>>(ta, tb, c.g, m.ff);
            break;
        }
        default:
            if ((rc = enable_smem(mix_cutcp_kernel<CONV>, kGemmBytes)) != TK_OK) return rc;
            mix_cutcp_kernel<CONV><<<ctas, threads, kGemmBytes, st>>>(ta, tb, c.g, m.cc);
            break;
    }
    return launch_error("fused kernel launch");
}

// fused launch with the tensor role on CTA pairs
template <typename KernelT, typename ArgsT>
static int launch_more_pair(KernelT k, const GemmCall& c, const ArgsT& a, DeviceInfo* d, unsigned ctas, unsigned threads, int smem,
                            cudaStream_t st) {
    CUtensorMap ta, tb;
    int rc = make_tmap(&ta, c.A, c.g.M, c.g.K, kGemmBM);
    if (rc != TK_OK) return rc;
    if ((rc = make_tmap(&tb, c.B, c.g.N, c.g.K, kGemm2BN / 2)) != TK_OK) return rc;
    if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
    unsigned pairs = 0;
    if ((rc = pairs_for(k, d, ctas, threads, smem, &pairs)) != TK_OK) return rc;
    k<<<2 * pairs, threads, smem, st>>>(ta, tb, c.g, a);
    return launch_error("fused kernel launch (CTA pairs)");
}

static int launch_mix_more_pair(const GemmCall& c, const MoreCall& m, DeviceInfo* d, unsigned ctas, unsigned threads,
                                unsigned cdt, cudaStream_t st) {
    constexpr int kBytes6 = Gemm2Smem<kStagesPair>::kBytes + 1024, kBytes4 = Gemm2Smem<kMorePairStagesSmem>::kBytes + 1024;
    const int nw = static_cast<int>(cdt / 32);
    switch (m.kind) {
        case MORE_SGEMM: {
            const int room = kMaxDynSmem - kBytes4;
            if (sgemm_role_smem(nw, 4) <= room)
                return launch_more_pair(mix_sgemm2_kernel<4>, c, m.sg, d, ctas, threads, kBytes4 + sgemm_role_smem(nw, 4), st);
            if (sgemm_role_smem(nw, 3) <= room)
                return launch_more_pair(mix_sgemm2_kernel<3>, c, m.sg, d, ctas, threads, kBytes4 + sgemm_role_smem(nw, 3), st);
            return launch_more_pair(mix_sgemm2_kernel<2>, c, m.sg, d, ctas, threads, kBytes4 + sgemm_role_smem(nw, 2), st);
        }
        case MORE_LBM: return launch_more_pair(mix_lbm2_kernel, c, m.lb, d, ctas, threads, kBytes6, st);
        case MORE_FFT: return launch_more_pair(mix_fft2_kernel, c, m.ff, d, ctas, threads, kBytes4 + fft_role_smem(nw), st);
        default: return launch_more_pair(mix_cutcp2_kernel, c, m.cc, d, ctas, threads, kBytes6, st);
    }
}

static int run_mix_more(GemmCall& c, const MoreCall& m, unsigned grid0, unsigned block0, cudaStream_t st) {
    DeviceInfo* d = nullptr;
    int rc = device_info(&d);
    if (rc != TK_OK) return rc;
    c.g.status = d->status_ptr;
    c.g.l2_hints = g_opt.l2_hints;
    const bool gemm_empty = c.g.start >= c.g.end;
    if (gemm_empty && m.empty()) return TK_OK;
    if (block0 <= static_cast<unsigned>(kGemmThreads)) return TK_ERR_LAUNCH_CONFIG;
    // The tensor role on CTA pairs pays once the launch holds at least a wave of pair tiles (as for the other pairs).
    const unsigned ctas0 = grid0 < static_cast<unsigned>(d->sm_count) ? grid0 : static_cast<unsigned>(d->sm_count);
    const bool pair_ok = !c.conv && c.g.M >= 256 && c.g.N >= 256 && ctas0 >= 2;
    const bool pair_wins = c.g.N % 256 == 0 && static_cast<long long>(c.g.end - c.g.start) >= 16ll * (ctas0 / 2);
    const bool use_pair = pair_ok && (g_opt.mix_pair > 0 || (g_opt.mix_pair == 0 && pair_wins));
    const int kGemmBytes = use_pair ? Gemm2Smem<kMorePairStagesSmem>::kBytes + 1024 : GemmSmem<kMoreBN, kMoreStages>::kBytes + 1024;
    unsigned cap = (m.kind == MORE_SGEMM ? kMaxMixThreadsSgemm : kMaxMixThreadsSfu) - kGemmThreads;
    if (m.kind == MORE_SGEMM) {  // as many warps as find a ring of two slots behind the tensor role's stages
        const unsigned fit = static_cast<unsigned>((kMaxDynSmem - kGemmBytes) / (2 * kSgemmSlotBytes)) * 32u;
        if (fit < cap) cap = fit;
    }
    if (m.kind == MORE_FFT) {  // as many warps as find a buffer behind the tensor role's stages
        const unsigned fit = static_cast<unsigned>((kMaxDynSmem - kGemmBytes - kFftTwiddleBytes) / kFftWarpBytes) * 32u;
        if (fit < cap) cap = fit;
    }
    const unsigned cdt = cd_threads(block0 - kGemmThreads, 32, cap);
    if (cdt == 0) return TK_ERR_LAUNCH_CONFIG;
    if (gemm_empty) return run_more_solo(m, grid0, cdt, st);
    if (m.empty()) return run_tzgemm(c, grid0, st);
    const unsigned ctas = ctas0;
    const unsigned threads = kGemmThreads + cdt;
    CUtensorMap ta, tb;
    if (!use_pair) {
        if ((rc = make_tmap_a(&ta, c, kGemmBM)) != TK_OK) return rc;
        if ((rc = make_tmap(&tb, c.B, c.g.N, c.g.K, kMoreBN)) != TK_OK) return rc;
    }
    // work items sized for the CUDA-core warps of this launch; what split items need done first goes ahead on the stream
    MoreCall mm = m;
    const long long cd_warps = static_cast<long long>(ctas) * (cdt / 32);
    if (mm.kind == MORE_SGEMM) {
        mm.sg.k_per_item = sgemm_split_for(mm.sg, cd_warps);
        if ((rc = sgemm_prepass(mm.sg, st)) != TK_OK) return rc;
    } else if (mm.kind == MORE_CUTCP) {
        mm.cc.nbr_per_item = cutcp_split_for(mm.cc, cd_warps);
        if ((rc = cutcp_prepass(mm.cc, st)) != TK_OK) return rc;
    }
    if (use_pair) return launch_mix_more_pair(c, mm, d, ctas, threads, cdt, st);
    if (c.conv) return launch_mix_more_kernels<true>(c, mm, ta, tb, ctas, threads, cdt, st);
    return launch_mix_more_kernels<false>(c, mm, ta, tb, ctas, threads, cdt, st);
}

// number of solo arguments of each kind (before the six geometry ints)
static int more_solo_args(MoreKind k) {
    switch (k) {
        case MORE_SGEMM: return 6;
        case MORE_LBM: return 2;
        case MORE_FFT: return 1;
        default: return 10;
    }
}

static int parse_more(MoreKind kind, void** params, MoreCall* m) {
    const int n = more_solo_args(kind);
    m->kind = kind;
    switch (kind) {
        case MORE_SGEMM: return parse_sgemm(params, n + 6, n + 8, &m->sg);
        case MORE_LBM: return parse_lbm(params, n + 6, n + 8, &m->lb);
        case MORE_FFT: return parse_fft(params, n + 6, n + 8, &m->ff);
        default: return parse_cutcp(params, n + 6, n + 8, &m->cc);
    }
}

// gptb_<kind>: solo list + 6 geometry ints + start, step, end, thread_base
static int launch_more_gptb(MoreKind kind, void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                            void* stream) {
    int rc = check_params(params, nparams, more_solo_args(kind) + 10);
    if (rc != TK_OK) return rc;
    if ((rc = validate_grid(grid, block)) != TK_OK) return rc;
    MoreCall m;
    if ((rc = parse_more(kind, params, &m)) != TK_OK) return rc;
    return run_more_solo(m, grid[0], block[0], static_cast<cudaStream_t>(stream));
}

// tzgemm_<kind> / tzconv_<kind>: CUDA-core list (solo + 6 + 3), then tzgemm's (7 + 6 + 3) or tzconv's (12 + 6 + 3)
static int launch_more_mix(MoreKind kind, void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                           void* stream, bool conv = false) {
    const int cd_len = more_solo_args(kind) + 9;
    int rc = check_params(params, nparams, cd_len + (conv ? 21 : 16));
    if (rc != TK_OK) return rc;
    if ((rc = validate_grid(grid, block)) != TK_OK) return rc;
    MoreCall m;
    if ((rc = parse_more(kind, params, &m)) != TK_OK) return rc;
    GemmCall c;
    if (conv) rc = parse_conv(params, cd_len, cd_len + 18, cd_len + 20, &c);
    else rc = parse_gemm(params, cd_len, cd_len + 13, cd_len + 15, &c);
    if (rc != TK_OK) return rc;
    return run_mix_more(c, m, grid[0], block[0], static_cast<cudaStream_t>(stream));
}

// ---- launcher body for kernels of these four roles emitted by the fused-kernel generator -----------------------
// As generated_mix_launch (host_launch.cuh): the module fixes super-tile width, stage count and the number of
// CUDA-core warps at compile time; `role_smem` is what its CUDA-core role needs behind the tensor role's stages
// (sgemm: its rings, fft: its buffers).  `launch` receives everything parsed and encoded.
template <int BN, int STAGES, typename LaunchFn>
static int generated_more_launch(MoreKind kind, int cd_warps, int role_smem, void** params, int nparams,
                                 const unsigned grid[3], void* stream, LaunchFn launch) {
    const int cd_len = more_solo_args(kind) + 9;
    int rc = check_params(params, nparams, cd_len + 16);
    if (rc != TK_OK) return rc;
    if (grid == nullptr || grid[0] == 0) return TK_ERR_LAUNCH_CONFIG;
    MoreCall m;
    if ((rc = parse_more(kind, params, &m)) != TK_OK) return rc;
    GemmCall c;
    if ((rc = parse_gemm(params, cd_len, cd_len + 13, cd_len + 15, &c)) != TK_OK) return rc;
    DeviceInfo* d = nullptr;
    if ((rc = device_info(&d)) != TK_OK) return rc;
    c.g.status = d->status_ptr;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool gemm_empty = c.g.start >= c.g.end;
    if (gemm_empty && m.empty()) return TK_OK;
    if (gemm_empty) return run_more_solo(m, grid[0], 32u * static_cast<unsigned>(cd_warps), st);
    if (m.empty()) return run_tzgemm(c, grid[0], st);
    const unsigned ctas = grid[0] < static_cast<unsigned>(d->sm_count) ? grid[0] : static_cast<unsigned>(d->sm_count);
    const unsigned threads = kGemmThreads + 32u * static_cast<unsigned>(cd_warps);
    const int smem = GemmSmem<BN, STAGES>::kBytes + 1024 + role_smem;
    if (smem > kMaxDynSmem) return TK_ERR_CAPACITY;
    CUtensorMap ta, tb;
    if ((rc = make_tmap(&ta, c.A, c.g.M, c.g.K, kGemmBM)) != TK_OK) return rc;
    if ((rc = make_tmap(&tb, c.B, c.g.N, c.g.K, BN)) != TK_OK) return rc;
    const long long warps = static_cast<long long>(ctas) * cd_warps;
    if (kind == MORE_SGEMM) {
        m.sg.k_per_item = sgemm_split_for(m.sg, warps);
        if ((rc = sgemm_prepass(m.sg, st)) != TK_OK) return rc;
    } else if (kind == MORE_CUTCP) {
        m.cc.nbr_per_item = cutcp_split_for(m.cc, warps);
        if ((rc = cutcp_prepass(m.cc, st)) != TK_OK) return rc;
    }
    rc = launch(ta, tb, c.g, m, ctas, threads, smem, st);
    if (rc != TK_OK) return rc;
    return launch_error("generated mix kernel launch");
}

}  // namespace tk
