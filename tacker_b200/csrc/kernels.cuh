// Device status word and every __global__ kernel of the library (solo, fused, preparation).
// Included by tacker_b200.cu and by the sources the fused-kernel generator emits.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "cd_roles.cuh"
#include "gemm_role.cuh"
#include "gemm_role_m256.cuh"
#include "gemm_role2.cuh"
#include "stencil_tma.cuh"

namespace tk {

// -------------------------------------------------------------------------------------------------
// device status word (bounded waits report here)
// -------------------------------------------------------------------------------------------------
__device__ unsigned g_dev_status;

// -------------------------------------------------------------------------------------------------
// kernels
// -------------------------------------------------------------------------------------------------
constexpr int kMaxMixThreads = 768;     // stencil pair: 192 tensor-role threads + up to 576 CUDA-core threads (<= 85 registers)
constexpr int kMaxMixThreadsSfu = 1024;  // Coulomb / MRI-Q pairs: their roles need many warps and few registers (<= 64)

__device__ __forceinline__ uint8_t* align_smem_1024(uint8_t* p) {
    const uint32_t a = smem_u32(p);
    return p + ((1024u - (a & 1023u)) & 1023u);
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
tzgemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
              const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    gemm_role<BN, STAGES>(&tmap_a, &tmap_b, g, align_smem_1024(smem_raw), threadIdx.x >> 5, threadIdx.x & 31);
}

// implicit-GEMM convolution (3 x 3, stride 1, padding 1, bordered NHWC fp16 in and out; see GemmArgs)
template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
tzconv_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
              const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    gemm_role<BN, STAGES, true, true>(&tmap_x, &tmap_w, g, align_smem_1024(smem_raw), threadIdx.x >> 5,
                                      threadIdx.x & 31);
}

// 256 x 256 super-tiles (one third less operand traffic per flop): the solo kernel for large problems
__global__ void __launch_bounds__(kGemm256Threads, 1)
tzgemm256_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    gemm_role_m256(&tmap_a, &tmap_b, g, align_smem_1024(smem_raw), threadIdx.x >> 5, threadIdx.x & 31);
}

// CTA pairs (clusters of two): 256 x 256 pair tiles with tcgen05.mma.cta_group::2; the grid must be even
template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemm2Threads, 1)
tzgemm2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_bh, const GemmArgs g, const int split_tail) {
    extern __shared__ uint8_t smem_raw[];
    gemm_role2<STAGES>(&tmap_a, &tmap_b, g, align_smem_1024(smem_raw), threadIdx.x >> 5, threadIdx.x & 31,
                       blockIdx.x >> 1, gridDim.x >> 1, split_tail ? &tmap_bh : nullptr);
}

template <int PF>
__global__ void __launch_bounds__(512) stencil_kernel(const StencilArgs s) {
    stencil_role<PF>(s, threadIdx.x, blockDim.x, blockIdx.x, gridDim.x);
}

__device__ __forceinline__ uint8_t* align_smem_128(uint8_t* p) {
    const uint32_t a = smem_u32(p);
    return p + ((128u - (a & 127u)) & 127u);
}

// TMA-fed form: every warp streams its planes through a private ring of `ring` slots
__global__ void __launch_bounds__(512)
stencil_tma_kernel(const __grid_constant__ CUtensorMap tmap_grid, const StencilArgs s, const int ring,
                   unsigned* status) {
    extern __shared__ uint8_t smem_raw[];
    stencil_role_tma(&tmap_grid, s, align_smem_128(smem_raw), ring, threadIdx.x >> 5, blockDim.x >> 5,
                     threadIdx.x & 31, blockIdx.x, gridDim.x, status);
}

// Two CTAs of 512 threads per SM (<= 64 registers): 32 warps keep the special-function pipe busy.
template <int PPT, bool EXACT>
__global__ void __launch_bounds__(512, 2) cp_kernel(const CpArgs a) {
    __shared__ int item_counter;
    if (threadIdx.x == 0) item_counter = 0;
    __syncthreads();
    cp_role<PPT, EXACT>(a, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
}

template <bool ACCURATE, int VPT>
__global__ void __launch_bounds__(512, 2) mriq_kernel(const MriqArgs m) {
    __shared__ int item_counter;
    if (threadIdx.x == 0) item_counter = 0;
    __syncthreads();
    mriq_role<ACCURATE, VPT>(m, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
}

template <bool ACCURATE, int VPT>
__global__ void __launch_bounds__(512, 2) mrif_kernel(const MrifArgs m) {
    __shared__ int item_counter;
    if (threadIdx.x == 0) item_counter = 0;
    __syncthreads();
    mrif_role<ACCURATE, VPT>(m, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
}

// Fused kernels: warps 0..5 run the tensor role, the remaining warps the CUDA-core role.  The
// two roles share the SM and nothing else (the reference dispatches on threadIdx.x ranges the
// same way, src/mix_kernel/tzgemm_stencil.cu:284-298).
// ring > 0: the stencil warps use the TMA-fed role with their rings placed behind the tensor role's
// shared memory; ring == 0: the register role (shapes TMA cannot describe).
template <int BN, int STAGES, bool STAGED, bool CONV = false>
__global__ void __launch_bounds__(kMaxMixThreads, 1)
mix_stencil_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const GemmArgs g, const __grid_constant__ CUtensorMap tmap_grid, const StencilArgs s,
                   const int ring) {
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5;
    uint8_t* smem = align_smem_1024(smem_raw);
    if (warp < kGemmWarps) {
        gemm_role<BN, STAGES, STAGED, CONV>(&tmap_a, &tmap_b, g, smem, warp, threadIdx.x & 31);
    } else if (ring > 0) {
        stencil_role_tma(&tmap_grid, s, smem + GemmSmem<BN, STAGES, STAGED>::kBytes, ring, warp - kGemmWarps,
                         (blockDim.x >> 5) - kGemmWarps, threadIdx.x & 31, blockIdx.x, gridDim.x, g.status);
    } else {
        stencil_role<0>(s, threadIdx.x - kGemmThreads, blockDim.x - kGemmThreads, blockIdx.x, gridDim.x);
    }
}

// The CUDA-core warps of a fused CTA (threads kGemmThreads .. blockDim.x - 1) zero their item counter and meet
// on a named barrier of their own, so the tensor role is never involved.
constexpr uint32_t kCdBarrierId = 2;
__device__ __forceinline__ void cd_role_begin(int* item_counter) {
    if (threadIdx.x == kGemmThreads) *item_counter = 0;
    named_bar_sync(kCdBarrierId, blockDim.x - kGemmThreads);
}

template <int BN, int STAGES, int PPT, bool CONV = false>
__global__ void __launch_bounds__(kMaxMixThreadsSfu, 1)
mix_cp_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
              const GemmArgs g, const CpArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int item_counter;
    const int warp = threadIdx.x >> 5;
    if (warp < kGemmWarps) {
        gemm_role<BN, STAGES, true, CONV>(&tmap_a, &tmap_b, g, align_smem_1024(smem_raw), warp, threadIdx.x & 31);
    } else {
        cd_role_begin(&item_counter);
        cp_role<PPT, false>(a, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
    }
}

template <int BN, int STAGES, int VPT, bool CONV = false>
__global__ void __launch_bounds__(kMaxMixThreadsSfu, 1)
mix_mriq_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const GemmArgs g, const MriqArgs m) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int item_counter;
    const int warp = threadIdx.x >> 5;
    if (warp < kGemmWarps) {
        gemm_role<BN, STAGES, true, CONV>(&tmap_a, &tmap_b, g, align_smem_1024(smem_raw), warp, threadIdx.x & 31);
    } else {
        cd_role_begin(&item_counter);
        mriq_role<false, VPT>(m, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
    }
}

template <int BN, int STAGES, int VPT, bool CONV = false>
__global__ void __launch_bounds__(kMaxMixThreadsSfu, 1)
mix_mrif_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const GemmArgs g, const MrifArgs m) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int item_counter;
    const int warp = threadIdx.x >> 5;
    if (warp < kGemmWarps) {
        gemm_role<BN, STAGES, true, CONV>(&tmap_a, &tmap_b, g, align_smem_1024(smem_raw), warp, threadIdx.x & 31);
    } else {
        cd_role_begin(&item_counter);
        mrif_role<false, VPT>(m, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
    }
}

// Fused kernels on CTA pairs: the tensor role is gemm_role2 (clusters of two CTAs, 256 x 256 pair tiles), the
// CUDA-core role is unchanged and still works per CTA.  Its threads only arrive at the cluster barrier the tensor
// roles of the pair wait on at start-up.
template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMaxMixThreads, 1)
mix_stencil2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmArgs g, const __grid_constant__ CUtensorMap tmap_grid, const StencilArgs s,
                    const int ring) {
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5;
    uint8_t* smem = align_smem_1024(smem_raw);
    if (warp < kGemmWarps) {
        gemm_role2<STAGES>(&tmap_a, &tmap_b, g, smem, warp, threadIdx.x & 31, blockIdx.x >> 1, gridDim.x >> 1);
    } else {
        cluster_arrive();
        if (ring > 0)
            stencil_role_tma(&tmap_grid, s, smem + Gemm2Smem<STAGES>::kBytes, ring, warp - kGemmWarps,
                             (blockDim.x >> 5) - kGemmWarps, threadIdx.x & 31, blockIdx.x, gridDim.x, g.status);
        else
            stencil_role<0>(s, threadIdx.x - kGemmThreads, blockDim.x - kGemmThreads, blockIdx.x, gridDim.x);
    }
}

template <int STAGES, int PPT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMaxMixThreadsSfu, 1)
mix_cp2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const GemmArgs g, const CpArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int item_counter;
    const int warp = threadIdx.x >> 5;
    if (warp < kGemmWarps) {
        gemm_role2<STAGES>(&tmap_a, &tmap_b, g, align_smem_1024(smem_raw), warp, threadIdx.x & 31, blockIdx.x >> 1,
                           gridDim.x >> 1);
    } else {
        cluster_arrive();
        cd_role_begin(&item_counter);
        cp_role<PPT, false>(a, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
    }
}

template <int STAGES, int VPT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMaxMixThreadsSfu, 1)
mix_mriq2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmArgs g, const MriqArgs m) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int item_counter;
    const int warp = threadIdx.x >> 5;
    if (warp < kGemmWarps) {
        gemm_role2<STAGES>(&tmap_a, &tmap_b, g, align_smem_1024(smem_raw), warp, threadIdx.x & 31, blockIdx.x >> 1,
                           gridDim.x >> 1);
    } else {
        cluster_arrive();
        cd_role_begin(&item_counter);
        mriq_role<false, VPT>(m, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
    }
}

template <int STAGES, int VPT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMaxMixThreadsSfu, 1)
mix_mrif2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmArgs g, const MrifArgs m) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int item_counter;
    const int warp = threadIdx.x >> 5;
    if (warp < kGemmWarps) {
        gemm_role2<STAGES>(&tmap_a, &tmap_b, g, align_smem_1024(smem_raw), warp, threadIdx.x & 31, blockIdx.x >> 1,
                           gridDim.x >> 1);
    } else {
        cluster_arrive();
        cd_role_begin(&item_counter);
        mrif_role<false, VPT>(m, &item_counter, threadIdx.x & 31, blockIdx.x, gridDim.x);
    }
}

// ---- input preparation ----
__global__ void cp_pack_kernel(const float4* __restrict__ atoms, int count, float zplane,
                               float4* __restrict__ packed) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) {
        float4 a = atoms[i];
        const float dz = __fsub_rn(zplane, a.z);
        a.z = __fmul_rn(dz, dz);
        packed[i] = a;
    }
}

__global__ void mriq_pack_kernel(const float* __restrict__ kx, const float* __restrict__ ky,
                                 const float* __restrict__ kz, const float* __restrict__ phiR,
                                 const float* __restrict__ phiI, int numK, float4* __restrict__ kvals) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k < numK) {
        const float re = phiR[k], im = phiI[k];
        // real*real + imag*imag with the contraction nvcc applies to the reference's expression
        kvals[k] = make_float4(kx[k], ky[k], kz[k], __fmaf_rn(re, re, __fmul_rn(im, im)));
    }
}

// ComputeRhoPhiGPU (src/ori_kernel/mrif_kernel.cu:63-76) and the packing of the sample table in one pass:
// RhoPhiR = phiR*dR + phiI*dI, RhoPhiI = phiR*dI - phiI*dR with the contractions nvcc applies
__global__ void mrif_pack_kernel(const float* __restrict__ kx, const float* __restrict__ ky,
                                 const float* __restrict__ kz, const float* __restrict__ phiR,
                                 const float* __restrict__ phiI, const float* __restrict__ dR,
                                 const float* __restrict__ dI, int numK, float4* __restrict__ kvals) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k < numK) {
        const float pr = phiR[k], pi = phiI[k], rdr = dR[k], rdi = dI[k];
        kvals[k] = make_float4(kx[k], ky[k], kz[k], __fmaf_rn(pr, rdr, __fmul_rn(pi, rdi)));
        reinterpret_cast<float*>(kvals + numK)[k] = __fmaf_rn(pr, rdi, -__fmul_rn(pi, rdr));
    }
}

// ---- bordered NHWC fp16 activations (the operand format of the implicit-GEMM convolution) ----
// out[(h + 1)][(w + 1)][c] = act(x[h*W + w][c] + bias[c]) as fp16; x has leading dimension ldx; the border of `out`
// is not touched (it is zeroed once, when the buffer is created)
__global__ void bias_act_f16_bordered_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ bias,
                                             __half* __restrict__ out, int H, int W, int C, int act) {
    const long long total = static_cast<long long>(H) * W * C;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(e % C);
        const long long px = e / C;
        const int w = static_cast<int>(px % W), h = static_cast<int>(px / W);
        float v = x[px * ldx + c] + (bias ? __ldg(bias + c) : 0.0f);
        if (act == 1) v = fmaxf(v, 0.0f);
        out[(static_cast<size_t>(h + 1) * (W + 2) + (w + 1)) * C + c] = __float2half_rn(v);
    }
}

// 2 x 2 max pooling from a bordered image [(H + 2)][(W + 2)][C] into a bordered image [(H/2 + 2)][(W/2 + 2)][C];
// eight channels (16 bytes) per thread
__global__ void maxpool2x2_f16_bordered_kernel(const __half* __restrict__ x, int H, int W, int C,
                                               __half* __restrict__ out) {
    const int OH = H / 2, OW = W / 2, C8 = C / 8;
    const long long total = static_cast<long long>(OH) * OW * C8;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(e % C8) * 8;
        const int ow = static_cast<int>((e / C8) % OW), oh = static_cast<int>(e / (static_cast<long long>(C8) * OW));
        const __half* p = x + (static_cast<size_t>(2 * oh + 1) * (W + 2) + (2 * ow + 1)) * C + c;
        const size_t rowp = static_cast<size_t>(W + 2) * C;
        uint4 a = *reinterpret_cast<const uint4*>(p), b = *reinterpret_cast<const uint4*>(p + C);
        uint4 d = *reinterpret_cast<const uint4*>(p + rowp), f = *reinterpret_cast<const uint4*>(p + rowp + C);
        __half2* ha = reinterpret_cast<__half2*>(&a);
        const __half2* hb = reinterpret_cast<const __half2*>(&b);
        const __half2* hd = reinterpret_cast<const __half2*>(&d);
        const __half2* hf = reinterpret_cast<const __half2*>(&f);
#pragma unroll
        for (int u = 0; u < 4; ++u) ha[u] = __hmax2(__hmax2(ha[u], hb[u]), __hmax2(hd[u], hf[u]));
        *reinterpret_cast<uint4*>(out + (static_cast<size_t>(oh + 1) * (OW + 2) + (ow + 1)) * C + c) = a;
    }
}

// A[0][(h*W + w)*C + c] = x[(h + 1)][(w + 1)][c]: the bordered image as one GEMM row (the input of the first dense layer)
__global__ void unborder_f16_kernel(const __half* __restrict__ x, int H, int W, int C, __half* __restrict__ row) {
    const long long total = static_cast<long long>(H) * W * C;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(e % C);
        const long long px = e / C;
        const int w = static_cast<int>(px % W), h = static_cast<int>(px / W);
        row[e] = x[(static_cast<size_t>(h + 1) * (W + 2) + (w + 1)) * C + c];
    }
}

// ---- LC-layer helpers ----
// One thread per (channel, output row, output column) as in the reference; consecutive threads
// take consecutive output columns so every one of the kh*kw stores of a warp is coalesced.
__global__ void im2col_kernel(long long n, const float* __restrict__ im, int height, int width, int kh,
                              int kw, int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w,
                              int hcol, int wcol, float* __restrict__ col) {
    for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < n;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int w = static_cast<int>(idx % wcol);
        const long long hidx = idx / wcol;
        const int h = static_cast<int>(hidx % hcol);
        const int c = static_cast<int>(hidx / hcol);
        const int h0 = h * stride_h - pad_h, w0 = w * stride_w - pad_w;
        float* dst = col + (static_cast<size_t>(c) * kh * kw * hcol + h) * wcol + w;
        const float* src = im + static_cast<size_t>(c) * height * width;
        for (int i = 0; i < kh; ++i)
            for (int j = 0; j < kw; ++j) {
                const int hi = h0 + i * dil_h, wi = w0 + j * dil_w;
                *dst = (hi >= 0 && wi >= 0 && hi < height && wi < width)
                           ? __ldg(src + static_cast<size_t>(hi) * width + wi)
                           : 0.0f;
                dst += static_cast<size_t>(hcol) * wcol;
            }
    }
}

__global__ void cvt_f32_f16_kernel(__half* __restrict__ out, const float* __restrict__ in, long long n) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const long long n4 = n / 4;
    const bool vec = ((reinterpret_cast<uintptr_t>(in) & 15u) == 0) && ((reinterpret_cast<uintptr_t>(out) & 7u) == 0);
    if (vec) {
        for (long long i = i0; i < n4; i += stride) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(in) + i);
            __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
            uint2 o;
            o.x = *reinterpret_cast<uint32_t*>(&lo);
            o.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(out)[i] = o;
        }
        for (long long i = n4 * 4 + i0; i < n; i += stride) out[i] = __float2half_rn(in[i]);
    } else {
        for (long long i = i0; i < n; i += stride) out[i] = __float2half_rn(in[i]);
    }
}

}  // namespace tk
