// Host side of the launchers: options, per-device state, TMA descriptors, parsing of the reference-order
// argument lists, launch-shape decisions.  Everything is `static`: each shared module that includes this
// file (the library itself, or a module emitted by the fused-kernel generator) gets its own copy.
#pragma once
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>

#include "../../include/tacker_b200.h"
#include "kernels.cuh"

namespace tk {


// -------------------------------------------------------------------------------------------------
// host side
// -------------------------------------------------------------------------------------------------
static thread_local std::string t_last_error;

static int cuda_fail(cudaError_t e, const char* what) {
    t_last_error = std::string(what) + ": " + cudaGetErrorString(e);
    return TK_ERR_CUDA;
}
#define TK_CUDA(call)                                         \
    do {                                                      \
        cudaError_t _e = (call);                              \
        if (_e != cudaSuccess) return cuda_fail(_e, #call);   \
    } while (0)

struct Options {
    int tzgemm_bn = 0;
    int cp_exact = 0;
    int cp_ppt = 8;      // solo kernel: points per thread and work item (8 = the reference's granularity, measured best)
    int mix_cp_ppt = 8;  // fused kernel
    int mriq_accurate = 0;
    int mrif_accurate = 0;
    // (mriq_split, mriq_vpt and mix_mriq_vpt also govern the MRI-FHd kernels, which have the same shape)
    // second dimension of the Coulomb / MRI-Q work items (fast modes only): -1 = the host picks the atoms /
    // samples per item from the launch shape, 0 = never split (deterministic summation order), > 0 = that many
    int cp_split = -1;
    int mriq_split = -1;
    // the same for sgemm (k-steps per work item) and cutcp (neighbour bins per work item)
    int sgemm_split = -1;
    int sgemm_coop = 1;    // 1: large solo sgemm launches share the A slices per CTA (sgemm_group); 2: every launch that can; 0: none
    int cutcp_split = -1;
    int mriq_vpt = 2;      // voxels per thread and work item / 32, solo kernel (2 or 4)
    int mix_mriq_vpt = 4;  // fused kernel: the larger item halves the table reads that compete with the tensor role
    int stencil_prefetch = 0;   // register role: L2 prefetch distance in planes (0 or 8)
    int stencil_tma = 1;        // 1 = TMA-fed role whenever the shape allows, 0 = always the register role
    int stencil_ring = 4;       // ring depth per warp, solo kernel (2 planes in flight per warp measured best)
    int mix_stencil_ring = 12;  // upper bound of the ring depth in the fused kernel (shared memory decides)
    int tzgemm_m256 = 0;        // solo tzgemm with 256 x 256 super-tiles: 0 = by shape, 1 = always, -1 = never
    int tzgemm_pair = 0;        // solo tzgemm on CTA pairs (cta_group::2): 0 = by shape, 1 = whenever possible, -1 = never
    int tzgemm_pair_split = 1;  // solo kernel on CTA pairs: cut the tiles of a short last wave into column halves
    int mix_pair = 0;           // the same for the tensor role of the fused kernels
    int mix_pair_stages = 4;    // operand stages of the fused stencil kernel on CTA pairs (3 .. 5; the rest goes to the rings)
    int l2_hints = 0;           // fused kernels: GEMM tiles evict-last, stencil planes evict-first in L2
    int wait_budget_us = 1000000;  // budget of the bounded device-side waits, microseconds at 2 GHz
    int test_skip_loads = 0;       // test hook: the next n single-CTA tzgemm launches issue no operand loads
    int mix_stencil_cfg = 0;    // tensor-role shape of the fused stencil kernel: 0 auto, 1 = 256x3 stages,
                                // 2 = 128x4, 3 = 128x3, 4 = 128x2
};
static Options g_opt;

struct DeviceInfo {
    int sm_count = 0;
    unsigned* status_ptr = nullptr;
    // per kernel (and launch shape): clusters of two CTAs that can be resident at once
    std::map<std::tuple<const void*, unsigned, int>, int> pair_clusters;
};
static std::mutex g_mutex;
static std::map<int, DeviceInfo> g_devices;

static int device_info(DeviceInfo** out) {
    int dev = 0;
    TK_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_devices.find(dev);
    if (it == g_devices.end()) {
        DeviceInfo d;
        TK_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        TK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status_ptr), g_dev_status));
        it = g_devices.emplace(dev, d).first;
    }
    *out = &it->second;
    return TK_OK;
}

// ---- TMA descriptors (driver entry point fetched through the runtime; libcuda is not linked) ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static int get_encoder() {
    if (g_encode) return TK_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    TK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (q != cudaDriverEntryPointSuccess || fn == nullptr) {
        t_last_error = "cuTensorMapEncodeTiled is not available in this driver";
        return TK_ERR_CUDA;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return TK_OK;
}

// fp16 matrices [batch][rows][k], k contiguous; box = 64 (k) x box_rows x 1, 128-byte swizzle
static int make_tmap(CUtensorMap* m, const void* base, int rows, int k, int box_rows, int batch = 1,
                     long long batch_stride_elems = 0) {
    int rc = get_encoder();
    if (rc != TK_OK) return rc;
    if (batch < 1) batch = 1;
    if (batch_stride_elems <= 0) batch_stride_elems = static_cast<long long>(rows) * k;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(k) * 2, static_cast<cuuint64_t>(batch_stride_elems) * 2};
    cuuint32_t box[3] = {static_cast<cuuint32_t>(kGemmBK), static_cast<cuuint32_t>(box_rows), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        t_last_error = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(r));
        return TK_ERR_CUDA;
    }
    return TK_OK;
}

// fp32 grid [nz][ny][nx]; box = 72 x 6 x 1 (a 64 x 4 bundle plus its halo), no swizzle, zero fill
static int make_tmap_grid(CUtensorMap* m, const float* base, int nx, int ny, int nz) {
    int rc = get_encoder();
    if (rc != TK_OK) return rc;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(nx), static_cast<cuuint64_t>(ny), static_cast<cuuint64_t>(nz)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(nx) * 4, static_cast<cuuint64_t>(nx) * ny * 4};
    cuuint32_t box[3] = {kStTileCols, kStTileRows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        t_last_error = "cuTensorMapEncodeTiled (grid) failed with CUresult " + std::to_string(static_cast<int>(r));
        return TK_ERR_CUDA;
    }
    return TK_OK;
}

static bool stencil_tma_ok(const StencilArgs& s) {
    return g_opt.stencil_tma != 0 && s.nx % 4 == 0 && s.nz >= 3 &&
           (reinterpret_cast<uintptr_t>(s.A0) & 15u) == 0 && (reinterpret_cast<uintptr_t>(s.Anext) & 15u) == 0;
}

constexpr int kMaxDynSmem = 232448;  // 227 KiB per CTA on sm_100

// ---- parameter access ----
template <typename T>
static inline T arg(void** params, int i) {
    T v;
    std::memcpy(&v, params[i], sizeof(T));
    return v;
}

static int check_params(void** params, int nparams, int expected) {
    if (params == nullptr || nparams != expected) return TK_ERR_ARGS;
    for (int i = 0; i < nparams; ++i)
        if (params[i] == nullptr) return TK_ERR_ARGS;
    return TK_OK;
}

struct GemmCall {
    const __half* A;  // the A matrix, or the bordered input image of the implicit-GEMM convolution
    const __half* B;
    GemmArgs g;
    long long stride_a = 0, stride_b = 0;  // elements between batch entries (0 = dense)
    bool conv = false;
    int conv_h = 0;  // image height (rows of the bordered image = conv_h + 2)
};

static void gemm_args_defaults(GemmArgs* g) {
    g->status = nullptr;
    g->batch = 1;
    g->stride_c = 0;
    g->l2_hints = 0;
    g->splitk = 1;
    g->conv_c = 0;
    g->conv_w = 0;
    g->conv_oh = 0;
    g->conv_act = 0;
    g->conv_bias = nullptr;
    g->conv_out = nullptr;
    g->test_skip_loads = 0;
}

// params[base .. base+6] = A, B, C, M, N, K, alpha; start/end at the given indices
static int parse_gemm(void** params, int base, int i_start, int i_end, GemmCall* c) {
    c->A = arg<const __half*>(params, base + 0);
    c->B = arg<const __half*>(params, base + 1);
    c->g.C = arg<float*>(params, base + 2);
    c->g.M = arg<int>(params, base + 3);
    c->g.N = arg<int>(params, base + 4);
    c->g.K = arg<int>(params, base + 5);
    c->g.alpha = arg<float>(params, base + 6);
    c->g.start = arg<int>(params, i_start);
    c->g.end = arg<int>(params, i_end);
    gemm_args_defaults(&c->g);
    const bool empty = c->g.start >= c->g.end;
    if (c->g.M < 128 || c->g.N < 64 || c->g.K < 64) return TK_ERR_SHAPE;
    if (c->g.M % 128 || c->g.N % 64 || c->g.K % 64) return TK_ERR_SHAPE;
    if (!empty && (c->A == nullptr || c->B == nullptr || c->g.C == nullptr)) return TK_ERR_ARGS;
    if ((reinterpret_cast<uintptr_t>(c->A) & 15u) || (reinterpret_cast<uintptr_t>(c->B) & 15u) ||
        (reinterpret_cast<uintptr_t>(c->g.C) & 15u))
        return TK_ERR_ALIGN;
    if (c->g.start < 0) return TK_ERR_ARGS;
    return TK_OK;
}

// params[base .. base+11] = X (bordered NHWC fp16 image), Wt ([N][9 C] fp16), Y (bordered fp16 output image), M, N, K,
// alpha, bias, H, W, C, act; start/end at the given indices.  M = H (W + 2) rounded up to 128.
static int parse_conv(void** params, int base, int i_start, int i_end, GemmCall* c) {
    gemm_args_defaults(&c->g);
    c->conv = true;
    c->A = arg<const __half*>(params, base + 0);
    c->B = arg<const __half*>(params, base + 1);
    c->g.conv_out = arg<__half*>(params, base + 2);
    c->g.C = nullptr;
    c->g.M = arg<int>(params, base + 3);
    c->g.N = arg<int>(params, base + 4);
    c->g.K = arg<int>(params, base + 5);
    c->g.alpha = arg<float>(params, base + 6);
    c->g.conv_bias = arg<const float*>(params, base + 7);
    c->conv_h = arg<int>(params, base + 8);
    c->g.conv_w = arg<int>(params, base + 9);
    c->g.conv_c = arg<int>(params, base + 10);
    c->g.conv_act = arg<int>(params, base + 11);
    c->g.conv_oh = c->conv_h;
    c->g.start = arg<int>(params, i_start);
    c->g.end = arg<int>(params, i_end);
    if (c->conv_h <= 0 || c->g.conv_w <= 0 || c->g.conv_c <= 0 || c->g.conv_act < 0 || c->g.conv_act > 1) return TK_ERR_ARGS;
    if (c->g.conv_c % 64 || c->g.K != 9 * c->g.conv_c || c->g.N < 64 || c->g.N % 64) return TK_ERR_SHAPE;
    if (c->g.M < 128 || c->g.M % 128 || c->g.M < c->conv_h * (c->g.conv_w + 2)) return TK_ERR_SHAPE;
    const bool empty = c->g.start >= c->g.end;
    if (!empty && (c->A == nullptr || c->B == nullptr || c->g.conv_out == nullptr)) return TK_ERR_ARGS;
    if ((reinterpret_cast<uintptr_t>(c->A) & 15u) || (reinterpret_cast<uintptr_t>(c->B) & 15u) ||
        (reinterpret_cast<uintptr_t>(c->g.conv_out) & 15u) || (reinterpret_cast<uintptr_t>(c->g.conv_bias) & 15u))
        return TK_ERR_ALIGN;
    if (c->g.start < 0) return TK_ERR_ARGS;
    return TK_OK;
}

// tensor map of the A operand: the matrix, or the bordered image seen as [(H + 2)(W + 2)][C]
static int make_tmap_a(CUtensorMap* m, const GemmCall& c, int box_rows) {
    if (c.conv) return make_tmap(m, c.A, (c.conv_h + 2) * (c.g.conv_w + 2), c.g.conv_c, box_rows);
    return make_tmap(m, c.A, c.g.M, c.g.K, box_rows, c.g.batch, c.stride_a);
}

static int choose_bn(const GemmArgs& g, int ctas) {
    if (g_opt.tzgemm_bn == 128 || g_opt.tzgemm_bn == 256) return g_opt.tzgemm_bn;
    if (g.N % 256 != 0) return 128;
    // time model: waves x per-tile cost; a 128-wide tile re-reads A from shared memory twice as
    // often per flop, so it is charged a little more than half of a 256-wide one
    const long long t256 = static_cast<long long>(g.M / 128) * (g.N / 256);
    const long long t128 = static_cast<long long>(g.M / 128) * (g.N / 128);
    const double c256 = static_cast<double>((t256 + ctas - 1) / ctas) * 2.0;
    const double c128 = static_cast<double>((t128 + ctas - 1) / ctas) * 1.15;
    return c256 <= c128 ? 256 : 128;
}

constexpr int kStages256 = 4;
constexpr int kStages128 = 6;
template <int BN>
struct StagesFor {
    static constexpr int value = BN == 256 ? kStages256 : kStages128;
};

template <int BN>
static constexpr int gemm_smem_bytes() {
    return GemmSmem<BN, StagesFor<BN>::value>::kBytes + 1024;  // + slack for the 1024-byte alignment
}

template <typename KernelT>
static int enable_smem(KernelT kernel, int bytes) {
    // idempotent and cheap; done on every call so that it holds for every device that is used
    TK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    return TK_OK;
}

static int validate_grid(const unsigned grid[3], const unsigned block[3]) {
    if (grid == nullptr || block == nullptr) return TK_ERR_ARGS;
    if (grid[0] == 0 || grid[1] > 1 || grid[2] > 1) return TK_ERR_LAUNCH_CONFIG;
    if (block[0] == 0 || block[1] > 1 || block[2] > 1) return TK_ERR_LAUNCH_CONFIG;
    return TK_OK;
}

// ---- CUDA-core argument parsing (reference argument order) ----
static int parse_stencil(void** p, int i_start, int i_end, StencilArgs* s) {
    s->c0 = arg<float>(p, 0);
    s->c1 = arg<float>(p, 1);
    s->A0 = arg<const float*>(p, 2);
    s->Anext = arg<float*>(p, 3);
    s->nx = arg<int>(p, 4);
    s->ny = arg<int>(p, 5);
    s->nz = arg<int>(p, 6);
    s->gx = arg<int>(p, 7);
    s->gy = arg<int>(p, 8);
    const int bdx = arg<int>(p, 10), bdy = arg<int>(p, 11);
    s->start = arg<int>(p, i_start);
    s->end = arg<int>(p, i_end);
    s->l2_hints = 0;
    s->slabs = 1;
    s->per = 1;
    if (s->nx <= 0 || s->ny <= 0 || s->nz <= 0 || s->gx <= 0 || s->gy <= 0 || s->start < 0) return TK_ERR_ARGS;
    if (bdx != 32 || bdy != 4) return TK_ERR_SHAPE;  // the 64 x 4 bundle is the virtual-block unit
    if (s->end > s->gx * s->gy) s->end = s->gx * s->gy;  // see the note on ranges in the header
    if (s->start < s->end && (s->A0 == nullptr || s->Anext == nullptr)) return TK_ERR_ARGS;
    if ((reinterpret_cast<uintptr_t>(s->A0) & 3u) || (reinterpret_cast<uintptr_t>(s->Anext) & 3u)) return TK_ERR_ALIGN;
    return TK_OK;
}

static int parse_cp(void** p, int i_start, int i_end, CpArgs* a) {
    a->numatoms = arg<int>(p, 0);
    a->spacing = arg<float>(p, 1);
    a->lattice = arg<float*>(p, 2);
    a->atoms = arg<const float4*>(p, 3);
    a->gx = arg<int>(p, 4);
    a->gy = arg<int>(p, 5);
    const int bdx = arg<int>(p, 7), bdy = arg<int>(p, 8);
    a->start = arg<int>(p, i_start);
    a->end = arg<int>(p, i_end);
    a->atoms_per_item = 0;
    if (a->numatoms < 0 || a->gx <= 0 || a->gy <= 0 || a->start < 0) return TK_ERR_ARGS;
    if (bdx != 16 || bdy != 8) return TK_ERR_SHAPE;
    if (a->end > a->gx * a->gy) a->end = a->gx * a->gy;
    if (a->start < a->end && (a->lattice == nullptr || (a->numatoms > 0 && a->atoms == nullptr))) return TK_ERR_ARGS;
    if ((reinterpret_cast<uintptr_t>(a->atoms) & 15u) || (reinterpret_cast<uintptr_t>(a->lattice) & 3u))
        return TK_ERR_ALIGN;
    return TK_OK;
}

static int parse_mriq(void** p, int i_start, int i_end, MriqArgs* m) {
    m->numK = arg<int>(p, 0);
    m->x = arg<const float*>(p, 2);
    m->y = arg<const float*>(p, 3);
    m->z = arg<const float*>(p, 4);
    m->Qr = arg<float*>(p, 5);
    m->Qi = arg<float*>(p, 6);
    m->kvals = arg<const float4*>(p, 7);
    m->gx = arg<int>(p, 8);
    const int bdx = arg<int>(p, 11);
    m->start = arg<int>(p, i_start);
    m->end = arg<int>(p, i_end);
    m->k_per_item = 0;
    if (m->numK < 0 || m->gx <= 0 || m->start < 0) return TK_ERR_ARGS;
    if (bdx != 256) return TK_ERR_SHAPE;
    if (m->end > m->gx) m->end = m->gx;
    if (m->start < m->end &&
        (!m->x || !m->y || !m->z || !m->Qr || !m->Qi || (m->numK > 0 && m->kvals == nullptr)))
        return TK_ERR_ARGS;
    if (reinterpret_cast<uintptr_t>(m->kvals) & 15u) return TK_ERR_ALIGN;
    return TK_OK;
}

// MRI-FHd has MRI-Q's argument list: numK, kGlobalIndex, x, y, z, outR, outI, packed table
static int parse_mrif(void** p, int i_start, int i_end, MrifArgs* m) {
    MriqArgs q;
    const int rc = parse_mriq(p, i_start, i_end, &q);
    if (rc != TK_OK) return rc;
    m->numK = q.numK;
    m->kvals = q.kvals;
    m->x = q.x;
    m->y = q.y;
    m->z = q.z;
    m->outR = q.Qr;
    m->outI = q.Qi;
    m->gx = q.gx;
    m->start = q.start;
    m->end = q.end;
    m->k_per_item = 0;
    return TK_OK;
}

static int launch_error(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, what);
    return TK_OK;
}

// ---- solo launches ----
template <int BN>
static int launch_tzgemm(const GemmCall& c, unsigned ctas, cudaStream_t st) {
    constexpr int STAGES = StagesFor<BN>::value;
    CUtensorMap ta, tb;
    int rc = make_tmap_a(&ta, c, kGemmBM);
    if (rc != TK_OK) return rc;
    rc = make_tmap(&tb, c.B, c.g.N, c.g.K, BN, c.g.batch, c.stride_b);
    if (rc != TK_OK) return rc;
    if (c.conv) {
        auto ck = tzconv_kernel<BN, STAGES>;
        if ((rc = enable_smem(ck, gemm_smem_bytes<BN>())) != TK_OK) return rc;
        ck<<<ctas, kGemmThreads, gemm_smem_bytes<BN>(), st>>>(ta, tb, c.g);
        return launch_error("tzconv_kernel launch");
    }
    auto kernel = tzgemm_kernel<BN, STAGES>;
    rc = enable_smem(kernel, gemm_smem_bytes<BN>());
    if (rc != TK_OK) return rc;
    GemmArgs g = c.g;
    if (g_opt.test_skip_loads > 0) {
        --g_opt.test_skip_loads;
        g.test_skip_loads = 1;
    }
    kernel<<<ctas, kGemmThreads, gemm_smem_bytes<BN>(), st>>>(ta, tb, g);
    return launch_error("tzgemm_kernel launch");
}

constexpr int kStagesPair = 6;

// How many CTA pairs of `kernel` the device can hold at once (a persistent launch must not exceed it: the
// pairs wait on each other's barriers only inside a pair, but a pair that is not resident would start late).
template <typename KernelT>
static int max_resident_pairs(KernelT kernel, unsigned threads, int smem, int* out) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    TK_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
    *out = n;
    return TK_OK;
}

// number of CTA pairs to launch for a request of `ctas` CTAs: never more than fit at once
template <typename KernelT>
static int pairs_for(KernelT kernel, DeviceInfo* d, unsigned ctas, unsigned threads, int smem, unsigned* pairs) {
    const auto key = std::make_tuple(reinterpret_cast<const void*>(kernel), threads, smem);
    int resident = -1;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        auto it = d->pair_clusters.find(key);
        if (it != d->pair_clusters.end()) resident = it->second;
    }
    if (resident < 0) {
        int rc = max_resident_pairs(kernel, threads, smem, &resident);
        if (rc != TK_OK) return rc;
        std::lock_guard<std::mutex> lock(g_mutex);
        d->pair_clusters[key] = resident;
    }
    unsigned p = ctas / 2;
    if (p > static_cast<unsigned>(resident)) p = static_cast<unsigned>(resident);
    if (p == 0) return TK_ERR_LAUNCH_CONFIG;
    *pairs = p;
    return TK_OK;
}

static int run_tzgemm_pair(const GemmCall& c, DeviceInfo* d, unsigned ctas, cudaStream_t st) {
    constexpr int smem = Gemm2Smem<kStagesPair>::kBytes + 1024;
    auto kernel = tzgemm2_kernel<kStagesPair>;
    int rc = enable_smem(kernel, smem);
    if (rc != TK_OK) return rc;
    unsigned pairs = 0;
    if ((rc = pairs_for(kernel, d, ctas, kGemm2Threads, smem, &pairs)) != TK_OK) return rc;
    CUtensorMap ta, tb, tbh;
    if ((rc = make_tmap(&ta, c.A, c.g.M, c.g.K, kGemmBM)) != TK_OK) return rc;
    if ((rc = make_tmap(&tb, c.B, c.g.N, c.g.K, kGemm2BN / 2)) != TK_OK) return rc;
    if ((rc = make_tmap(&tbh, c.B, c.g.N, c.g.K, kGemm2BN / 4)) != TK_OK) return rc;
    kernel<<<2 * pairs, kGemm2Threads, smem, st>>>(ta, tb, tbh, c.g, g_opt.tzgemm_pair_split);
    return launch_error("tzgemm2_kernel launch");
}

static int run_tzgemm(GemmCall& c, unsigned grid0, cudaStream_t st, bool allow_splitk = false) {
    DeviceInfo* d = nullptr;
    int rc = device_info(&d);
    if (rc != TK_OK) return rc;
    c.g.status = d->status_ptr;
    if (c.g.start >= c.g.end) return TK_OK;
    // one CTA per SM holds the whole tensor memory; more CTAs than SMs would only queue
    const unsigned ctas = grid0 < static_cast<unsigned>(d->sm_count) ? grid0 : static_cast<unsigned>(d->sm_count);
    if (c.conv)  // the convolution form exists for the single-CTA 128-row role only
        return choose_bn(c.g, static_cast<int>(ctas)) == 256 ? launch_tzgemm<256>(c, ctas, st) : launch_tzgemm<128>(c, ctas, st);
    if (allow_splitk) {
        // a skinny problem has fewer super-tiles than SMs: cut K so that every SM gets a share (C was zeroed by
        // the caller and receives the partial products as reductions)
        const int bn = choose_bn(c.g, static_cast<int>(ctas));
        const long long tiles = c.g.end - c.g.start;
        const long long nsuper = (tiles * 64 * 64 + 128ll * bn - 1) / (128ll * bn) * (c.g.batch > 0 ? c.g.batch : 1);
        int split = static_cast<int>(ctas / (nsuper > 0 ? nsuper : 1));
        const int kblocks = c.g.K / kGemmBK;
        if (split > kblocks / 4) split = kblocks / 4;  // at least four K-blocks per share
        if (split > 32) split = 32;
        c.g.splitk = split > 1 ? split : 1;
    }
    // Large dense problems: 256 x 256 super-tiles stream a third less operand data per flop but have no second
    // accumulator buffer.  Measured on B200: +7 % at 4096 x 4096 x 2048 / x 4096 and +5 % at 8192 x 8192 x 1024, no
    // gain at 4096 x 4096 x 1024, a loss when there are fewer super-tiles than SMs.
    const long long full_tiles = static_cast<long long>(c.g.M / 64) * (c.g.N / 64);
    const long long tiles256 = static_cast<long long>((c.g.M + 255) / 256) * (c.g.N / 256);
    const bool big = c.g.N % 256 == 0 && c.g.end - c.g.start == full_tiles && tiles256 >= static_cast<long long>(ctas) &&
                     (c.g.K >= 2048 || tiles256 >= 4ll * ctas);
    // CTA pairs (256 x 256 pair tiles, two accumulator buffers).  Measured on B200 against the forms below: ahead for
    // short K with at least a wave of pair tiles (4096 x 4096 x 1024: 34.2 vs 35.9 us, 8192 x 8192 x 1024: 122.5 vs
    // 125.5 us), behind the single-CTA 256 x 256 form from K = 2048 on and when there are fewer pair tiles than pairs.
    const bool pair_ok = c.g.batch <= 1 && c.g.splitk <= 1 && c.g.M >= 256 && c.g.N >= 256 && ctas >= 2;
    const bool pair_wins = c.g.end - c.g.start == full_tiles && c.g.N % 256 == 0 && c.g.K < 2048 &&
                           tiles256 >= static_cast<long long>(ctas / 2);
    if (pair_ok && (g_opt.tzgemm_pair > 0 || (g_opt.tzgemm_pair == 0 && pair_wins))) return run_tzgemm_pair(c, d, ctas, st);
    if (c.g.batch <= 1 && c.g.splitk <= 1 && (g_opt.tzgemm_m256 > 0 || (g_opt.tzgemm_m256 == 0 && big))) {
        CUtensorMap ta, tb;
        if ((rc = make_tmap(&ta, c.A, c.g.M, c.g.K, 256)) != TK_OK) return rc;
        if ((rc = make_tmap(&tb, c.B, c.g.N, c.g.K, 256)) != TK_OK) return rc;
        constexpr int smem = Gemm256Smem::kBytes + 1024;
        if ((rc = enable_smem(tzgemm256_kernel, smem)) != TK_OK) return rc;
        tzgemm256_kernel<<<ctas, kGemm256Threads, smem, st>>>(ta, tb, c.g);
        return launch_error("tzgemm256_kernel launch");
    }
    return choose_bn(c.g, static_cast<int>(ctas)) == 256 ? launch_tzgemm<256>(c, ctas, st)
                                                        : launch_tzgemm<128>(c, ctas, st);
}

static unsigned cd_threads(unsigned requested, unsigned granule, unsigned cap) {
    unsigned t = requested > cap ? cap : requested;
    t = (t / granule) * granule;
    return t;
}

static int run_stencil(StencilArgs s, unsigned grid0, unsigned block0, cudaStream_t st) {
    if (s.start >= s.end) return TK_OK;
    const unsigned threads = cd_threads(block0, 32, 512);
    if (threads == 0) return TK_ERR_LAUNCH_CONFIG;
    if (stencil_tma_ok(s)) {
        DeviceInfo* d = nullptr;
        int rc = device_info(&d);
        if (rc != TK_OK) return rc;
        const int nwarps = static_cast<int>(threads / 32);
        int ring = g_opt.stencil_ring;
        while (ring > kStMinRing && nwarps * stencil_tma_warp_bytes(ring) + 128 > kMaxDynSmem) --ring;
        const int smem = nwarps * stencil_tma_warp_bytes(ring) + 128;
        CUtensorMap tg;
        if ((rc = make_tmap_grid(&tg, s.A0, s.nx, s.ny, s.nz)) != TK_OK) return rc;
        if ((rc = enable_smem(stencil_tma_kernel, smem)) != TK_OK) return rc;
        stencil_pick_split(s.nz, s.end - s.start, static_cast<long long>(grid0) * nwarps, &s.slabs, &s.per);
        stencil_tma_kernel<<<grid0, threads, smem, st>>>(tg, s, ring, d->status_ptr);
        return launch_error("stencil_tma_kernel launch");
    }
    const unsigned rthreads = cd_threads(threads, kStencilGroup, 512);
    if (rthreads == 0) return TK_ERR_LAUNCH_CONFIG;
    stencil_pick_split(s.nz, s.end - s.start, static_cast<long long>(grid0) * (rthreads / kStencilGroup), &s.slabs,
                       &s.per);
    if (g_opt.stencil_prefetch) stencil_kernel<8><<<grid0, rthreads, 0, st>>>(s);
    else stencil_kernel<0><<<grid0, rthreads, 0, st>>>(s);
    return launch_error("stencil_kernel launch");
}

// atoms per work item for a launch of `warps` warps in total (see CpArgs::atoms_per_item)
static int cp_split_for(const CpArgs& a, int ppt, long long warps) {
    if (g_opt.cp_exact || g_opt.cp_split == 0) return 0;
    if (g_opt.cp_split > 0) return (g_opt.cp_split + kCpChunk - 1) / kCpChunk * kCpChunk;
    return cd_pick_split(static_cast<long long>(a.end - a.start) * 4 * (8 / ppt), warps, a.numatoms, kCpChunk);
}

static int mriq_split_for(const MriqArgs& m, int vpt, long long warps) {
    if (g_opt.mriq_accurate || g_opt.mriq_split == 0) return 0;
    if (g_opt.mriq_split > 0) return g_opt.mriq_split;
    return cd_pick_split(static_cast<long long>(m.end - m.start) * (8 / vpt), warps, m.numK, 64);
}

static int mrif_split_for(const MrifArgs& m, int vpt, long long warps) {
    if (g_opt.mrif_accurate || g_opt.mriq_split == 0) return 0;
    if (g_opt.mriq_split > 0) return g_opt.mriq_split;
    return cd_pick_split(static_cast<long long>(m.end - m.start) * (8 / vpt), warps, m.numK, 64);
}

static int run_mrif(MrifArgs m, unsigned grid0, unsigned block0, cudaStream_t st) {
    if (m.start >= m.end) return TK_OK;
    const unsigned threads = cd_threads(block0, 32, 512);
    if (threads == 0) return TK_ERR_LAUNCH_CONFIG;
    const int vpt = g_opt.mriq_vpt == 4 ? 4 : 2;
    m.k_per_item = mrif_split_for(m, vpt, static_cast<long long>(grid0) * (threads / 32));
    if (g_opt.mrif_accurate) mrif_kernel<true, 2><<<grid0, threads, 0, st>>>(m);
    else if (vpt == 4) mrif_kernel<false, 4><<<grid0, threads, 0, st>>>(m);
    else mrif_kernel<false, 2><<<grid0, threads, 0, st>>>(m);
    return launch_error("mrif_kernel launch");
}

static int run_cp(CpArgs a, unsigned grid0, unsigned block0, cudaStream_t st) {
    if (a.start >= a.end) return TK_OK;
    const unsigned threads = cd_threads(block0, 32, 512);
    if (threads == 0) return TK_ERR_LAUNCH_CONFIG;
    const int ppt = g_opt.cp_ppt;
    a.atoms_per_item = cp_split_for(a, ppt, static_cast<long long>(grid0) * (threads / 32));
    if (g_opt.cp_exact) {
        if (ppt == 2) cp_kernel<2, true><<<grid0, threads, 0, st>>>(a);
        else if (ppt == 4) cp_kernel<4, true><<<grid0, threads, 0, st>>>(a);
        else cp_kernel<8, true><<<grid0, threads, 0, st>>>(a);
    } else {
        if (ppt == 2) cp_kernel<2, false><<<grid0, threads, 0, st>>>(a);
        else if (ppt == 4) cp_kernel<4, false><<<grid0, threads, 0, st>>>(a);
        else cp_kernel<8, false><<<grid0, threads, 0, st>>>(a);
    }
    return launch_error("cp_kernel launch");
}

static int run_mriq(MriqArgs m, unsigned grid0, unsigned block0, cudaStream_t st) {
    if (m.start >= m.end) return TK_OK;
    const unsigned threads = cd_threads(block0, 32, 512);
    if (threads == 0) return TK_ERR_LAUNCH_CONFIG;
    const int vpt = g_opt.mriq_vpt == 4 ? 4 : 2;
    m.k_per_item = mriq_split_for(m, vpt, static_cast<long long>(grid0) * (threads / 32));
    if (g_opt.mriq_accurate) mriq_kernel<true, 2><<<grid0, threads, 0, st>>>(m);
    else if (vpt == 4) mriq_kernel<false, 4><<<grid0, threads, 0, st>>>(m);
    else mriq_kernel<false, 2><<<grid0, threads, 0, st>>>(m);
    return launch_error("mriq_kernel launch");
}

// ---- fused launches ----
enum CdKind { CD_STENCIL, CD_CP, CD_MRIQ, CD_MRIF };

struct CdCall {
    CdKind kind;
    StencilArgs s;
    CpArgs a;
    MriqArgs m;
    MrifArgs f;
    bool empty() const {
        switch (kind) {
            case CD_STENCIL: return s.start >= s.end;
            case CD_CP: return a.start >= a.end;
            case CD_MRIF: return f.start >= f.end;
            default: return m.start >= m.end;
        }
    }
};

// The stencil's rings share the CTA's shared memory with the tensor role's stages, so the fused stencil
// kernel exists in several (super-tile width, stage count) shapes: a launch whose GEMM share is small gives
// most of the shared memory to the rings, a GEMM-heavy launch keeps a deep operand pipeline.
template <int BN, int STAGES, bool STAGED, bool CONV = false>
static int launch_mix_stencil(const GemmCall& c, StencilArgs s, unsigned ctas, unsigned threads, cudaStream_t st) {
    constexpr int kGemmBytes = GemmSmem<BN, STAGES, STAGED>::kBytes + 1024;
    auto k = mix_stencil_kernel<BN, STAGES, STAGED, CONV>;
    CUtensorMap ta, tb, tg;
    std::memset(&tg, 0, sizeof(tg));
    int rc = make_tmap_a(&ta, c, kGemmBM);
    if (rc != TK_OK) return rc;
    if ((rc = make_tmap(&tb, c.B, c.g.N, c.g.K, BN)) != TK_OK) return rc;
    int nwarps = static_cast<int>((threads - kGemmThreads) / 32);
    int ring = 0, smem = kGemmBytes;
    if (stencil_tma_ok(s)) {
        // as many of the requested warps as get at least the minimum ring next to the GEMM's stages
        const int fit = (kMaxDynSmem - kGemmBytes) / stencil_tma_warp_bytes(kStMinRing);
        if (fit >= 1) {
            if (nwarps > fit) nwarps = fit;
            ring = g_opt.mix_stencil_ring;
            while (ring > kStMinRing && kGemmBytes + nwarps * stencil_tma_warp_bytes(ring) > kMaxDynSmem) --ring;
            threads = kGemmThreads + 32u * static_cast<unsigned>(nwarps);
        }
    }
    if (ring > 0) {
        if ((rc = make_tmap_grid(&tg, s.A0, s.nx, s.ny, s.nz)) != TK_OK) return rc;
        smem += nwarps * stencil_tma_warp_bytes(ring);
        stencil_pick_split(s.nz, s.end - s.start, static_cast<long long>(ctas) * nwarps, &s.slabs, &s.per);
    } else {
        const unsigned groups = (threads - kGemmThreads) / kStencilGroup;
        if (groups == 0) return TK_ERR_LAUNCH_CONFIG;
        threads = kGemmThreads + groups * kStencilGroup;
        stencil_pick_split(s.nz, s.end - s.start, static_cast<long long>(ctas) * groups, &s.slabs, &s.per);
    }
    if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
    k<<<ctas, threads, smem, st>>>(ta, tb, c.g, tg, s, ring);
    return launch_error("mix_stencil_kernel launch");
}

static int run_mix_stencil(const GemmCall& c, const StencilArgs& s, unsigned ctas, unsigned threads, cudaStream_t st) {
    if (c.conv) return launch_mix_stencil<128, 4, true, true>(c, s, ctas, threads, st);
    int cfg = g_opt.mix_stencil_cfg;
    if (cfg == 0) {
        // Measured on B200 (config 2; 8 to 18 stencil warps; 64 to 4096 GEMM tiles): the 128-wide super-tile with
        // 4 stages is best up to about one GEMM-time of stencil work per launch -- it leaves ~75 KB to the
        // stencil's rings -- and the 256-wide one with 3 stages once the GEMM dominates the launch.
        const double t_gemm = 2.0 * 4096.0 * (c.g.end - c.g.start) * c.g.K / 1.0e15;
        const double t_cd = 8.0 * 256.0 * (s.end - s.start) * (s.nz > 2 ? s.nz - 2 : 1) / 5.0e12;
        cfg = (t_gemm > 1.2 * t_cd && c.g.N % 256 == 0) ? 1 : 2;
    }
    switch (cfg) {
        case 1: return launch_mix_stencil<256, 3, true>(c, s, ctas, threads, st);
        case 2: return launch_mix_stencil<128, 4, true>(c, s, ctas, threads, st);
        case 3: return launch_mix_stencil<128, 3, true>(c, s, ctas, threads, st);
        default: return launch_mix_stencil<128, 2, true>(c, s, ctas, threads, st);
    }
}

// ---- fused launches on CTA pairs ----
template <int STAGES>
static int launch_mix_stencil_pair(const GemmCall& c, StencilArgs s, DeviceInfo* d, unsigned ctas, unsigned threads,
                                   cudaStream_t st) {
    constexpr int kGemmBytes = Gemm2Smem<STAGES>::kBytes + 1024;
    auto k = mix_stencil2_kernel<STAGES>;
    CUtensorMap ta, tb, tg;
    std::memset(&tg, 0, sizeof(tg));
    int rc = make_tmap(&ta, c.A, c.g.M, c.g.K, kGemmBM);
    if (rc != TK_OK) return rc;
    if ((rc = make_tmap(&tb, c.B, c.g.N, c.g.K, kGemm2BN / 2)) != TK_OK) return rc;
    int nwarps = static_cast<int>((threads - kGemmThreads) / 32);
    int ring = 0, smem = kGemmBytes;
    if (stencil_tma_ok(s)) {
        const int fit = (kMaxDynSmem - kGemmBytes) / stencil_tma_warp_bytes(kStMinRing);
        if (fit >= 1) {
            if (nwarps > fit) nwarps = fit;
            ring = g_opt.mix_stencil_ring;
            while (ring > kStMinRing && kGemmBytes + nwarps * stencil_tma_warp_bytes(ring) > kMaxDynSmem) --ring;
            threads = kGemmThreads + 32u * static_cast<unsigned>(nwarps);
        }
    }
    if (ring > 0) {
        smem += nwarps * stencil_tma_warp_bytes(ring);
    } else {
        const unsigned groups = (threads - kGemmThreads) / kStencilGroup;
        if (groups == 0) return TK_ERR_LAUNCH_CONFIG;
        threads = kGemmThreads + groups * kStencilGroup;
        nwarps = static_cast<int>(groups);
    }
    if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
    unsigned pairs = 0;
    if ((rc = pairs_for(k, d, ctas, threads, smem, &pairs)) != TK_OK) return rc;
    if (ring > 0 && (rc = make_tmap_grid(&tg, s.A0, s.nx, s.ny, s.nz)) != TK_OK) return rc;
    stencil_pick_split(s.nz, s.end - s.start, static_cast<long long>(2 * pairs) * nwarps, &s.slabs, &s.per);
    k<<<2 * pairs, threads, smem, st>>>(ta, tb, c.g, tg, s, ring);
    return launch_error("mix_stencil2_kernel launch");
}

static int run_mix_stencil_pair(const GemmCall& c, const StencilArgs& s, DeviceInfo* d, unsigned ctas, unsigned threads,
                                cudaStream_t st) {
    switch (g_opt.mix_pair_stages) {
        case 3: return launch_mix_stencil_pair<3>(c, s, d, ctas, threads, st);
        case 5: return launch_mix_stencil_pair<5>(c, s, d, ctas, threads, st);
        default: return launch_mix_stencil_pair<4>(c, s, d, ctas, threads, st);
    }
}

template <typename KernelT, typename CdArgsT>
static int launch_mix_pair_kernel(KernelT k, const GemmCall& c, const CdArgsT& cd_args, DeviceInfo* d, unsigned ctas,
                                  unsigned threads, int cd_ppt_or_vpt, cudaStream_t st, CdArgsT (*split)(CdArgsT, int, long long)) {
    constexpr int smem = Gemm2Smem<kStagesPair>::kBytes + 1024;
    CUtensorMap ta, tb;
    int rc = make_tmap(&ta, c.A, c.g.M, c.g.K, kGemmBM);
    if (rc != TK_OK) return rc;
    if ((rc = make_tmap(&tb, c.B, c.g.N, c.g.K, kGemm2BN / 2)) != TK_OK) return rc;
    if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
    unsigned pairs = 0;
    if ((rc = pairs_for(k, d, ctas, threads, smem, &pairs)) != TK_OK) return rc;
    const CdArgsT a = split(cd_args, cd_ppt_or_vpt, static_cast<long long>(2 * pairs) * ((threads - kGemmThreads) / 32));
    k<<<2 * pairs, threads, smem, st>>>(ta, tb, c.g, a);
    return launch_error("fused kernel launch (CTA pairs)");
}

static CpArgs cp_with_split(CpArgs a, int ppt, long long warps) {
    a.atoms_per_item = cp_split_for(a, ppt, warps);
    return a;
}
static MriqArgs mriq_with_split(MriqArgs m, int vpt, long long warps) {
    m.k_per_item = mriq_split_for(m, vpt, warps);
    return m;
}
static MrifArgs mrif_with_split(MrifArgs m, int vpt, long long warps) {
    m.k_per_item = mrif_split_for(m, vpt, warps);
    return m;
}

static int launch_mix_pair(const GemmCall& c, const CdCall& cd, DeviceInfo* d, unsigned ctas, unsigned threads,
                           cudaStream_t st) {
    if (cd.kind == CD_CP) {
        const int ppt = g_opt.mix_cp_ppt;
        if (ppt == 2) return launch_mix_pair_kernel(mix_cp2_kernel<kStagesPair, 2>, c, cd.a, d, ctas, threads, 2, st, cp_with_split);
        if (ppt == 4) return launch_mix_pair_kernel(mix_cp2_kernel<kStagesPair, 4>, c, cd.a, d, ctas, threads, 4, st, cp_with_split);
        return launch_mix_pair_kernel(mix_cp2_kernel<kStagesPair, 8>, c, cd.a, d, ctas, threads, 8, st, cp_with_split);
    }
    if (cd.kind == CD_MRIF) {
        if (g_opt.mix_mriq_vpt == 4)
            return launch_mix_pair_kernel(mix_mrif2_kernel<kStagesPair, 4>, c, cd.f, d, ctas, threads, 4, st, mrif_with_split);
        return launch_mix_pair_kernel(mix_mrif2_kernel<kStagesPair, 2>, c, cd.f, d, ctas, threads, 2, st, mrif_with_split);
    }
    if (g_opt.mix_mriq_vpt == 4)
        return launch_mix_pair_kernel(mix_mriq2_kernel<kStagesPair, 4>, c, cd.m, d, ctas, threads, 4, st, mriq_with_split);
    return launch_mix_pair_kernel(mix_mriq2_kernel<kStagesPair, 2>, c, cd.m, d, ctas, threads, 2, st, mriq_with_split);
}

// fused launches whose tensor role is the implicit-GEMM convolution: one CUDA-core item shape per pair
// (Coulomb 8 points per thread, MRI-Q / MRI-FHd 4 voxels per thread)
template <int BN>
static int launch_mix_conv(const GemmCall& c, CdCall cd, unsigned ctas, unsigned threads, cudaStream_t st) {
    constexpr int STAGES = StagesFor<BN>::value;
    const long long cd_warps = static_cast<long long>(ctas) * ((threads - kGemmThreads) / 32);
    CUtensorMap ta, tb;
    int rc = make_tmap_a(&ta, c, kGemmBM);
    if (rc != TK_OK) return rc;
    if ((rc = make_tmap(&tb, c.B, c.g.N, c.g.K, BN)) != TK_OK) return rc;
    const int smem = gemm_smem_bytes<BN>();
    if (cd.kind == CD_CP) {
        cd.a.atoms_per_item = cp_split_for(cd.a, 8, cd_warps);
        auto k = mix_cp_kernel<BN, STAGES, 8, true>;
        if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
        k<<<ctas, threads, smem, st>>>(ta, tb, c.g, cd.a);
    } else if (cd.kind == CD_MRIF) {
        cd.f.k_per_item = mrif_split_for(cd.f, 4, cd_warps);
        auto k = mix_mrif_kernel<BN, STAGES, 4, true>;
        if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
        k<<<ctas, threads, smem, st>>>(ta, tb, c.g, cd.f);
    } else if (cd.kind == CD_MRIQ) {
        cd.m.k_per_item = mriq_split_for(cd.m, 4, cd_warps);
        auto k = mix_mriq_kernel<BN, STAGES, 4, true>;
        if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
        k<<<ctas, threads, smem, st>>>(ta, tb, c.g, cd.m);
    } else {
        return TK_ERR_ARGS;  // the stencil pair goes through run_mix_stencil
    }
    return launch_error("fused convolution launch");
}

template <int BN>
static int launch_mix(const GemmCall& c, CdCall cd, unsigned ctas, unsigned threads, cudaStream_t st) {
    constexpr int STAGES = StagesFor<BN>::value;
    const long long cd_warps = static_cast<long long>(ctas) * ((threads - kGemmThreads) / 32);
    if (c.conv) return launch_mix_conv<BN>(c, cd, ctas, threads, st);
    if (cd.kind == CD_CP) cd.a.atoms_per_item = cp_split_for(cd.a, g_opt.mix_cp_ppt, cd_warps);
    const int mvpt = g_opt.mix_mriq_vpt == 4 ? 4 : 2;
    if (cd.kind == CD_MRIQ) cd.m.k_per_item = mriq_split_for(cd.m, mvpt, cd_warps);
    if (cd.kind == CD_MRIF) cd.f.k_per_item = mrif_split_for(cd.f, mvpt, cd_warps);
    CUtensorMap ta, tb;
    int rc = make_tmap(&ta, c.A, c.g.M, c.g.K, kGemmBM);
    if (rc != TK_OK) return rc;
    rc = make_tmap(&tb, c.B, c.g.N, c.g.K, BN);
    if (rc != TK_OK) return rc;
    const int smem = gemm_smem_bytes<BN>();
    switch (cd.kind) {
        case CD_STENCIL:
            return TK_ERR_ARGS;  // handled by run_mix_stencil
        case CD_CP: {
            if (g_opt.mix_cp_ppt == 2) {
                auto k = mix_cp_kernel<BN, STAGES, 2>;
                if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
                k<<<ctas, threads, smem, st>>>(ta, tb, c.g, cd.a);
            } else if (g_opt.mix_cp_ppt == 4) {
                auto k = mix_cp_kernel<BN, STAGES, 4>;
                if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
                k<<<ctas, threads, smem, st>>>(ta, tb, c.g, cd.a);
            } else {
                auto k = mix_cp_kernel<BN, STAGES, 8>;
                if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
                k<<<ctas, threads, smem, st>>>(ta, tb, c.g, cd.a);
            }
            break;
        }
        case CD_MRIF: {
            if (mvpt == 4) {
                auto k = mix_mrif_kernel<BN, STAGES, 4>;
                if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
                k<<<ctas, threads, smem, st>>>(ta, tb, c.g, cd.f);
            } else {
                auto k = mix_mrif_kernel<BN, STAGES, 2>;
                if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
                k<<<ctas, threads, smem, st>>>(ta, tb, c.g, cd.f);
            }
            break;
        }
        default: {
            if (mvpt == 4) {
                auto k = mix_mriq_kernel<BN, STAGES, 4>;
                if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
                k<<<ctas, threads, smem, st>>>(ta, tb, c.g, cd.m);
            } else {
                auto k = mix_mriq_kernel<BN, STAGES, 2>;
                if ((rc = enable_smem(k, smem)) != TK_OK) return rc;
                k<<<ctas, threads, smem, st>>>(ta, tb, c.g, cd.m);
            }
            break;
        }
    }
    return launch_error("mix kernel launch");
}

static int run_mix(GemmCall& c, const CdCall& cd_in, unsigned grid0, unsigned block0, cudaStream_t st) {
    DeviceInfo* d = nullptr;
    int rc = device_info(&d);
    if (rc != TK_OK) return rc;
    c.g.status = d->status_ptr;
    CdCall cd = cd_in;
    c.g.l2_hints = g_opt.l2_hints;
    cd.s.l2_hints = g_opt.l2_hints;
    const bool gemm_empty = c.g.start >= c.g.end;
    if (gemm_empty && cd.empty()) return TK_OK;
    if (block0 <= static_cast<unsigned>(kGemmThreads)) return TK_ERR_LAUNCH_CONFIG;
    const unsigned granule = 32;
    const unsigned cap = (cd.kind == CD_STENCIL ? kMaxMixThreads : kMaxMixThreadsSfu) - kGemmThreads;
    const unsigned cdt = cd_threads(block0 - kGemmThreads, granule, cap);
    if (cdt == 0) return TK_ERR_LAUNCH_CONFIG;
    if (gemm_empty) {  // nothing for the tensor role: run the CUDA-core kernel alone
        switch (cd.kind) {
            case CD_STENCIL: return run_stencil(cd.s, grid0, cdt, st);
            case CD_CP: return run_cp(cd.a, grid0, cdt, st);
            case CD_MRIF: return run_mrif(cd.f, grid0, cdt, st);
            default: return run_mriq(cd.m, grid0, cdt, st);
        }
    }
    if (cd.empty()) return run_tzgemm(c, grid0, st);
    const unsigned ctas = grid0 < static_cast<unsigned>(d->sm_count) ? grid0 : static_cast<unsigned>(d->sm_count);
    const unsigned threads = kGemmThreads + cdt;
    // The tensor role on CTA pairs pays once the launch holds at least a wave of pair tiles (measured on the
    // GEMM + stencil pair: 37.3 vs 41.4 us with 2048 tiles, 51.2 vs 55.4 us with 4096; behind by 2 us with 1024 and fewer).
    const bool pair_ok = !c.conv && c.g.M >= 256 && c.g.N >= 256 && ctas >= 2;
    const bool pair_wins = c.g.N % 256 == 0 && static_cast<long long>(c.g.end - c.g.start) >= 16ll * (ctas / 2);
    if (pair_ok && (g_opt.mix_pair > 0 || (g_opt.mix_pair == 0 && pair_wins))) {
        if (cd.kind == CD_STENCIL) return run_mix_stencil_pair(c, cd.s, d, ctas, threads, st);
        return launch_mix_pair(c, cd, d, ctas, threads, st);
    }
    if (cd.kind == CD_STENCIL) return run_mix_stencil(c, cd.s, ctas, threads, st);
    return choose_bn(c.g, static_cast<int>(ctas)) == 256 ? launch_mix<256>(c, cd, ctas, threads, st)
                                                        : launch_mix<128>(c, cd, ctas, threads, st);
}



// ---- launcher body for kernels emitted by the fused-kernel generator -----------------------------------
// A generated module fixes the pair, the super-tile width BN, the stage count and the number of
// CUDA-core warps at compile time (so that the kernel's register budget is the one of that ratio) and
// keeps the argument list of the library's fused launchers.  `launch` receives everything parsed and
// encoded and only has to start its own __global__ kernel.
template <int BN, int STAGES, typename LaunchFn>
static int generated_mix_launch(CdKind kind, int cd_warps, void** params, int nparams, const unsigned grid[3],
                                void* stream, LaunchFn launch) {
    const int n_cd = kind == CD_STENCIL ? 7 : (kind == CD_CP ? 4 : 8);
    const int cd_len = n_cd + 6 + 3;
    int rc = check_params(params, nparams, cd_len + 16);
    if (rc != TK_OK) return rc;
    if (grid == nullptr || grid[0] == 0) return TK_ERR_LAUNCH_CONFIG;
    CdCall cd;
    cd.kind = kind;
    const int i_start = n_cd + 6, i_end = n_cd + 8;
    switch (kind) {
        case CD_STENCIL: rc = parse_stencil(params, i_start, i_end, &cd.s); break;
        case CD_CP: rc = parse_cp(params, i_start, i_end, &cd.a); break;
        case CD_MRIF: rc = parse_mrif(params, i_start, i_end, &cd.f); break;
        default: rc = parse_mriq(params, i_start, i_end, &cd.m); break;
    }
    if (rc != TK_OK) return rc;
    GemmCall c;
    if ((rc = parse_gemm(params, cd_len, cd_len + 13, cd_len + 15, &c)) != TK_OK) return rc;
    DeviceInfo* d = nullptr;
    if ((rc = device_info(&d)) != TK_OK) return rc;
    c.g.status = d->status_ptr;
    // empty ranges as in the library's fused launchers: nothing to do, or the other kernel alone
    const bool gemm_empty = c.g.start >= c.g.end;
    if (gemm_empty && cd.empty()) return TK_OK;
    if (gemm_empty) {
        const unsigned cdt = 32u * static_cast<unsigned>(cd_warps);
        switch (kind) {
            case CD_STENCIL: return run_stencil(cd.s, grid[0], cdt, static_cast<cudaStream_t>(stream));
            case CD_CP: return run_cp(cd.a, grid[0], cdt, static_cast<cudaStream_t>(stream));
            case CD_MRIF: return run_mrif(cd.f, grid[0], cdt, static_cast<cudaStream_t>(stream));
            default: return run_mriq(cd.m, grid[0], cdt, static_cast<cudaStream_t>(stream));
        }
    }
    if (cd.empty()) return run_tzgemm(c, grid[0], static_cast<cudaStream_t>(stream));
    const unsigned ctas = grid[0] < static_cast<unsigned>(d->sm_count) ? grid[0] : static_cast<unsigned>(d->sm_count);
    const unsigned threads = kGemmThreads + 32u * static_cast<unsigned>(cd_warps);
    CUtensorMap ta, tb, tg;
    std::memset(&tg, 0, sizeof(tg));
    if ((rc = make_tmap(&ta, c.A, c.g.M, c.g.K, kGemmBM)) != TK_OK) return rc;
    if ((rc = make_tmap(&tb, c.B, c.g.N, c.g.K, BN)) != TK_OK) return rc;
    int smem = GemmSmem<BN, STAGES>::kBytes + 1024, ring = 0;
    if (kind == CD_STENCIL) {
        if (!stencil_tma_ok(cd.s)) return TK_ERR_SHAPE;  // generated stencil kernels carry the TMA-fed role only
        ring = kStMaxRing;
        while (ring >= kStMinRing && smem + cd_warps * stencil_tma_warp_bytes(ring) > kMaxDynSmem) --ring;
        if (ring < kStMinRing) return TK_ERR_CAPACITY;
        smem += cd_warps * stencil_tma_warp_bytes(ring);
        if ((rc = make_tmap_grid(&tg, cd.s.A0, cd.s.nx, cd.s.ny, cd.s.nz)) != TK_OK) return rc;
        stencil_pick_split(cd.s.nz, cd.s.end - cd.s.start, static_cast<long long>(ctas) * cd_warps, &cd.s.slabs,
                           &cd.s.per);
    }
    const long long cd_warps_total = static_cast<long long>(ctas) * cd_warps;
    if (kind == CD_CP) cd.a.atoms_per_item = cp_split_for(cd.a, 8, cd_warps_total);
    if (kind == CD_MRIQ) cd.m.k_per_item = mriq_split_for(cd.m, 2, cd_warps_total);
    if (kind == CD_MRIF) cd.f.k_per_item = mrif_split_for(cd.f, 2, cd_warps_total);
    rc = launch(ta, tb, c.g, tg, cd, ring, ctas, threads, smem, static_cast<cudaStream_t>(stream));
    if (rc != TK_OK) return rc;
    return launch_error("generated mix kernel launch");
}

}  // namespace tk
