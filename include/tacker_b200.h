/*
 * tacker_b200.h -- C ABI of libtacker_b200.so: hand-written sm_100a kernels for the
 * fused tensor-core / CUDA-core hot path of Tacker/Aker.
 *
 * The reference has no plugin ABI: its operator boundary is the table
 *     std::unordered_map<std::string, void*> fmap           (src/main.cu:108-159)
 * whose values are __global__ symbols that GPTBKernel::executeImpl / MixKernel::executeImpl
 * launch with cudaLaunchKernel(func, grid, block, void** params, smem, stream)
 * (src/GPTBKernel.h:99-119, src/MixKernel.h:86-104).  This library replaces every value of
 * that table that lies on the hot path by a *launcher* with the same calling shape:
 *
 *     int launcher(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
 *                  unsigned smem_bytes, void* stream);
 *
 * `params[i]` points at the i-th kernel argument exactly as for cudaLaunchKernel (values are
 * read during the call; they need not outlive it).  The argument lists are the reference
 * kernels' lists (cited per launcher below) with three documented changes:
 *   - tzgemm takes `float alpha` after K_GLOBAL (the reference hard-codes 1.1f,
 *     src/header/tzgemm_header.h:64, and has the parameter commented out);
 *   - cp takes the packed atom array as a device pointer after `energygrid` (the reference
 *     reads a 64-entry __constant__ symbol filled by copyatomstoconstbuf,
 *     src/ori_kernel/cp_kernel.cu:159-179);
 *   - mriq takes the packed k-space samples as a device pointer after `Qi` (the reference
 *     reads a 1024-entry __constant__ symbol, src/ori_kernel/mriq_kernel.cu:9).
 * grid/block: grid[0] persistent CTAs are launched; block[0] is honoured for the CUDA-core
 * kernels (rounded down to the role's thread granularity) and for the CUDA-core part of a
 * fused kernel (block[0] - 192 threads); the tensor role always uses 192 threads.  The
 * virtual-block range [ptb_start_block_pos, ptb_end_block_pos) is honoured exactly, in the
 * reference's units; ptb_iter_block_step is accepted and ignored (the stride is grid[0]).
 * A range that runs past the last virtual block is clamped to it: the reference kernels wrap
 * such indices around (block_pos % grid_dimension_x) and would then update the same outputs from
 * two CTAs at once; its scheduler never asks for that (src/TaskManager.cu:598 takes the min with
 * the block count).
 *
 * All pointers in `params` are device pointers owned by the caller.  Nothing here allocates
 * device memory on the launch path, nothing exits the process; every entry point returns a
 * tk_status.  Launches are asynchronous on `stream`.  The library is thread-compatible: calls
 * for one device must not race with tk_set_option.
 * There is no CPU fallback: without a CUDA device the launchers return TK_ERR_CUDA.
 */
#ifndef TACKER_B200_H
#define TACKER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum tk_status {
    TK_OK = 0,
    TK_ERR_ARGS = -1,        /* wrong parameter count, null pointer, negative size */
    TK_ERR_ALIGN = -2,       /* pointer or leading dimension not aligned as required */
    TK_ERR_SHAPE = -3,       /* shape outside the kernel's contract (see each launcher) */
    TK_ERR_UNKNOWN_KEY = -4, /* tk_lookup / tk_query: no such kernel */
    TK_ERR_CUDA = -5,        /* a CUDA runtime or driver call failed; see tk_last_error() */
    TK_ERR_LAUNCH_CONFIG = -6, /* grid/block not usable for this kernel */
    TK_ERR_DEVICE_WAIT = -7, /* a bounded device-side wait expired; see tk_device_status() */
    TK_ERR_CAPACITY = -8     /* request exceeds a fixed capacity of the entry point */
} tk_status;

typedef int (*tk_launch_fn)(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                            unsigned smem_bytes, void* stream);

/* ---- library ------------------------------------------------------------------------ */
int tk_version(void);
const char* tk_status_string(int status);
/* text of the most recent CUDA failure seen by this thread ("" if none) */
const char* tk_last_error(void);
/* number of SMs of the current device: replaces the compile-time SM_NUM
 * (src/header/pets_common.h:4-6) */
int tk_sm_count(int* sm_count);
/* tuning / numerics switches (name -> integer):
 *   "tzgemm_bn"      0 = choose per shape, 128 or 256 = force the super-tile width
 *   "tzgemm_m256"    solo tzgemm with 256 x 256 super-tiles (a third less operand traffic per flop, no second
 *                    accumulator buffer): 0 = for large dense problems, 1 = always, -1 = never
 *   "cp_exact"       1 = IEEE 1/sqrt as the reference computes it (default 0: hardware rsqrt)
 *   "tzgemm_pair"    solo tzgemm on clusters of two CTAs (tcgen05.mma.cta_group::2, 256 x 256 pair tiles): 0 = by
 *                    shape, 1 = whenever the shape allows (M, N >= 256), -1 = never; "mix_pair" the same for the
 *                    tensor role of the fused kernels, "mix_pair_stages" (3..5) its operand stages next to the stencil
 *   "cp_exact"       1 = IEEE 1/sqrt as the reference computes it (default 0: hardware rsqrt)
 *   "cp_ppt"         solo Coulomb kernel: points per thread and work item, 8 (default, the reference's granularity),
 *                    4 or 2; "mix_cp_ppt" the same for the fused kernel (default 8)
 *   "cp_split"       atoms per Coulomb work item in the fast mode: -1 (default) = chosen from the launch shape,
 *                    0 = whole list (deterministic summation order), n = n rounded up to 64.  Items that cover a
 *                    part of the list add their partial sums to the lattice with reductions in no fixed order.
 *   "mriq_accurate"  1 = cosf/sinf as the reference calls them (default 0: reduced argument +
 *                    hardware sin/cos); "mrif_accurate" the same for MRI-FHd (plus the binary64 product of its phase)
 *   "mriq_split"     samples per MRI-Q / MRI-FHd work item, as "cp_split"
 *   "sgemm_split"    k-steps per sgemm work item (a multiple of 8), "cutcp_split" neighbour bins per cutcp work item:
 *                    -1 (default) = chosen from the launch shape (launches with many blocks per warp are never split),
 *                    0 = never (the reference's order of additions, bit for bit), n = n.  Split items add partial
 *                    sums with reductions in no fixed order, after a short kernel on the same stream that doubles C
 *                    (sgemm: C = 2 C + 2 A B) or zeroes the regions (cutcp).
 *   "sgemm_coop"     1 (default) = a solo sgemm launch with at least one full group of column blocks per CTA lets the
 *                    warps of a CTA share the A slices through shared memory; 0 = every warp streams its own (the form
 *                    of the fused kernels and of short block ranges); 2 = the shared form for every range it can take
 *                    (tests).  Same results either way.
 *   "wait_budget_us" budget of every bounded device-side wait (default 1,000,000 = about a second); applies to the
 *                    current device.  "test_skip_loads" n: test hook, the next n single-CTA tzgemm launches issue
 *                    no operand loads, so that their waits run out.
 *   "mriq_vpt"       voxels per thread (2 or 4; a work item is 32 x that many voxels) of the solo MRI-Q / MRI-FHd
 *                    kernels, "mix_mriq_vpt" of the fused ones (default 4)
 */
int tk_set_option(const char* name, int value);
int tk_get_option(const char* name, int* value);
/* Reads and clears the device status word that bounded device-side waits write when they
 * give up (0 = no expiry; otherwise the code of the first wait that expired: 1 = a producer waited for a free
 * operand stage, 2 = the MMA issuer for operand bytes, 3 = the MMA issuer for a drained accumulator, 4 = the
 * epilogue for an accumulator).  Synchronises the device.  The launch that wrote the word has returned; its
 * outputs are incomplete. */
int tk_device_status(unsigned* code);
/* The same as a status: TK_OK, or TK_ERR_DEVICE_WAIT when the word was not zero (also cleared). */
int tk_device_check(void);

/* ---- the fmap replacement --------------------------------------------------------------
 * Keys (same strings as the reference table): "gptb_tzgemm", "gptb_tzgemm_acc", "gptb_stencil", "gptb_cp",
 * "gptb_mriq", "gptb_mrif", "tzgemm_stencil", "tzgemm_cp", "tzgemm_mriq", "tzgemm_mrif"; plus "ori_stencil",
 * "ori_cp", "ori_mriq", "ori_mrif" for the non-persistent launch shape of the solo kernels; and "gptb_tzconv",
 * "tzconv_stencil", "tzconv_cp", "tzconv_mriq", "tzconv_mrif" for the implicit-GEMM convolution (not in the
 * reference's table); and "gptb_<k>", "tzgemm_<k>", "tzconv_<k>", "ori_<k>" for k = sgemm, lbm, fft, cutcp. */
tk_launch_fn tk_lookup(const char* key);
int tk_num_keys(void);
const char* tk_key(int index);

typedef struct tk_kernel_info {
    int threads_tensor;   /* threads of the tensor role (0 for CUDA-core kernels) */
    int threads_cd_min;   /* thread granularity of the CUDA-core role */
    int threads_cd_default;
    int regs_per_thread;  /* from cudaFuncGetAttributes */
    int static_smem;      /* bytes */
    int dynamic_smem;     /* bytes requested at launch */
    int tmem_columns;     /* tensor-memory columns held by one CTA */
    int max_ctas_per_sm;  /* occupancy at the default block size */
    int nparams;          /* length of the params array the launcher expects */
} tk_kernel_info;
/* Resource figures the scheduler and the fused-kernel generator need; replaces the
 * register/shared_memory/blocksize fields of src/config/kinfo-*.json and the table in
 * fusion/code/data.py:25-35. */
int tk_query(const char* key, tk_kernel_info* info);

/* ---- persistent solo kernels -------------------------------------------------------------
 * gptb_tzgemm  replaces general_ptb_tzgemm (src/gptb_kernel/tzgemm_kernel.cu:430-449).
 *   params (17): half* A, half* B, float* C, int M_GLOBAL, int N_GLOBAL, int K_GLOBAL,
 *                float alpha,
 *                int grid_dimension_{x,y,z}, int block_dimension_{x,y,z},
 *                int ptb_start_block_pos, int ptb_iter_block_step, int ptb_end_block_pos,
 *                int thread_base
 *   C[M][N] = alpha * A[M][K] * B[N][K]^T, fp16 in, fp32 accumulate and out; one virtual block =
 *   one 64x64 tile of C, tiles numbered row-major (tzgemm_kernel.cu:247-249).
 *   Contract: M % 128 == 0, N % 64 == 0, K % 64 == 0, all >= 64 (the reference rounds every
 *   dimension down to a multiple of 128 before the call, src/tzgemm_kernel.h:30-34);
 *   A, B, C 16-byte aligned. */
int tk_launch_gptb_tzgemm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                          unsigned smem_bytes, void* stream);

/* gptb_tzgemm_acc  the same kernel and argument list for skinny problems (few 64x64 tiles, long K: the
 *   batch-1 dense layers).  No counterpart in the reference, whose tzgemm leaves most SMs idle on such shapes.
 *   K is cut into ranges handled by different CTAs and the partial products are added into C with
 *   reductions, so C MUST BE ZERO on entry; the order of the additions, and with it the last bits of the
 *   result, can differ from run to run. */
int tk_launch_gptb_tzgemm_acc(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                              unsigned smem_bytes, void* stream);

/* gptb_stencil  replaces general_ptb_stencil (src/gptb_kernel/stencil_kernel.cu:3-105).
 *   params (17): float c0, float c1, float* A0, float* Anext, int nx, int ny, int nz,
 *                6 geometry ints, start, step, end, thread_base
 *   geometry: grid_dimension_x/y = ceil(nx/64), ceil(ny/4); block_dimension_x/y = 32, 4
 *   (src/ori_kernel/stencil_kernel.cu:173-178).  One virtual block = 64 x 4 columns, all z. */
int tk_launch_gptb_stencil(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                           unsigned smem_bytes, void* stream);

/* gptb_cp  replaces g_general_ptb_cp (src/gptb_kernel/cp_kernel.cu:8-96).
 *   params (14): int numatoms, float gridspacing, float* energygrid, float4* atoms_packed,
 *                6 geometry ints, start, step, end, thread_base
 *   atoms_packed[i] = {x, y, (zplane - z)^2, q} (tk_cp_pack_atoms); any numatoms >= 0.
 *   geometry: grid_dimension_x/y = nx/128, ny/8; block_dimension_x/y = 16, 8; the lattice pitch is
 *   grid_dimension_x * 128 floats.  Adds to energygrid (+=) like the reference. */
int tk_launch_gptb_cp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                      unsigned smem_bytes, void* stream);

/* gptb_mriq  replaces g_general_ptb_mriq (src/gptb_kernel/mriq_kernel.cu:3-70).
 *   params (18): int numK, int kGlobalIndex (ignored), float* x, float* y, float* z, float* Qr,
 *                float* Qi, float4* kvals, 6 geometry ints, start, step, end, thread_base
 *   kvals[k] = {Kx, Ky, Kz, phiR^2 + phiI^2} (tk_mriq_pack_kvalues); all numK samples are summed in
 *   one launch.  geometry: grid_dimension_x = numX / 256, block_dimension_x = 256. */
int tk_launch_gptb_mriq(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                        unsigned smem_bytes, void* stream);

/* gptb_mrif  replaces g_general_ptb_mrif (src/gptb_kernel/mrif_kernel.cu:6-92).
 *   params (18): int numK, int kGlobalIndex (ignored), float* x, float* y, float* z, float* outR,
 *                float* outI, float* kvals, 6 geometry ints, start, step, end, thread_base
 *   kvals = the table tk_mrif_pack_kvalues writes (the reference reads a 256-entry __constant__ symbol,
 *   src/ori_kernel/mrif_kernel.cu:9): numK x {Kx, Ky, Kz, RhoPhiR}, then numK x RhoPhiI; all numK samples
 *   are summed in one launch.  geometry: grid_dimension_x = numX / 256, block_dimension_x = 256. */
int tk_launch_gptb_mrif(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                        unsigned smem_bytes, void* stream);

/* ---- fused kernels: tensor role + CUDA-core role in one persistent CTA ---------------------
 * Replace stencil_tzgemm_mix / cp_tzgemm_mix / mriq_tzgemm_mix / mrif_tzgemm_mix
 * (src/mix_kernel/tzgemm_stencil.cu:281-299, tzgemm_cp.cu:994-1017, tzgemm_mriq.cu:638-657, tzgemm_mrif.cu).
 * params = CUDA-core kernel's list without thread_base, then tzgemm's list without thread_base,
 * the order MixKernel::initParams builds (src/MixKernel.h:55-73):
 *   tzgemm_stencil (32) = stencil 7 + 6 + 3, tzgemm 7 + 6 + 3
 *   tzgemm_cp      (29) = cp 4 + 6 + 3,      tzgemm 7 + 6 + 3
 *   tzgemm_mriq    (33) = mriq 8 + 6 + 3,    tzgemm 7 + 6 + 3
 *   tzgemm_mrif    (33) = mrif 8 + 6 + 3,    tzgemm 7 + 6 + 3
 * block[0] = 192 + CUDA-core threads.  Either range may be empty. */
int tk_launch_mix_tzgemm_stencil(void** params, int nparams, const unsigned grid[3],
                                 const unsigned block[3], unsigned smem_bytes, void* stream);
int tk_launch_mix_tzgemm_cp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                            unsigned smem_bytes, void* stream);
int tk_launch_mix_tzgemm_mriq(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                              unsigned smem_bytes, void* stream);
int tk_launch_mix_tzgemm_mrif(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                              unsigned smem_bytes, void* stream);

/* ---- implicit-GEMM convolution ---------------------------------------------------------------
 * gptb_tzconv  replaces the im2col_gpu_kernel + convertFp32ToFp16 + tzgemm sequence of mycudnnConvolutionForward
 * (src/include/dnn.h:45-99, 554-803) for 3 x 3 convolutions with stride 1 and padding 1: the A operand is never
 * written to memory, bias and activation are applied in the epilogue.  Activations are zero-bordered NHWC fp16
 * images [(H + 2)][(W + 2)][C]; the border of the output image is never written (zero it once).
 *   params (22): half* X, half* Wt, half* Y, int M, int N, int K, float alpha, float* bias, int H, int W, int C,
 *                int act, 6 geometry ints (ignored), start, step, end, thread_base
 *   X = bordered input, C a multiple of 64; Wt = weights [N][K], K = 9 C, k = (3 i + j) C + c for tap (i, j);
 *   Y = bordered output [(H + 2)][(W + 2)][N], N a multiple of 64; bias [N] or null; act 0 = none, 1 = ReLU;
 *   M = H (W + 2) rounded up to a multiple of 128: GEMM row m is pixel (m / (W + 2), m % (W + 2)) of the bordered
 *   grid, rows with m % (W + 2) >= W are computed and dropped.  [start, end) counts 64 x 64 tiles of that
 *   M x N problem, row-major, like gptb_tzgemm.
 * tzconv_<cd> (stencil 37, cp 34, mriq / mrif 38 params): the fused kernels with this tensor role; params = the
 * CUDA-core list (n + 6 + 3), then tzconv's 12 + 6 + 3. */
int tk_launch_gptb_tzconv(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                          unsigned smem_bytes, void* stream);
int tk_launch_mix_tzconv_stencil(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                 unsigned smem_bytes, void* stream);
int tk_launch_mix_tzconv_cp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                            unsigned smem_bytes, void* stream);
int tk_launch_mix_tzconv_mriq(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                              unsigned smem_bytes, void* stream);
int tk_launch_mix_tzconv_mrif(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                              unsigned smem_bytes, void* stream);
/* helpers for the bordered fp16 activation format (no counterpart in the reference, whose activations are fp32 NCHW):
 *   tk_bias_act_f16_bordered   Y[(h+1)][(w+1)][c] = act(x[h W + w][c] + bias[c]), x fp32 with leading dimension ldx
 *   tk_maxpool2x2_f16_bordered 2 x 2 max pooling, bordered in, bordered out (C a multiple of 8)
 *   tk_unborder_f16            the interior of a bordered image as one dense row of H W C halves */
int tk_bias_act_f16_bordered(const float* x, int ldx, const float* bias, void* out_half, int H, int W, int C, int act,
                             void* stream);
int tk_maxpool2x2_f16_bordered(const void* x_half, int H, int W, int C, void* out_half, void* stream);
int tk_unborder_f16(const void* x_half, int H, int W, int C, void* row_half, void* stream);

/* ---- non-persistent launch shape of the solo kernels ------------------------------------------
 * ori_stencil (7 params, src/ori_kernel/stencil_kernel.cu:9), ori_cp (4 params with atoms_packed,
 * src/ori_kernel/cp_kernel.cu:26), ori_mriq (8 params with kvals, src/ori_kernel/mriq_kernel.cu:56):
 * grid/block are the reference launch geometry, every virtual block is computed. */
int tk_launch_ori_stencil(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                          unsigned smem_bytes, void* stream);
int tk_launch_ori_cp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                     unsigned smem_bytes, void* stream);
int tk_launch_ori_mriq(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                       unsigned smem_bytes, void* stream);
/* ori_mrif (8 params with kvals, src/ori_kernel/mrif_kernel.cu:78) */
int tk_launch_ori_mrif(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                       unsigned smem_bytes, void* stream);

/* ---- sgemm, lbm, fft, cutcp ------------------------------------------------------------------------
 * The other four Parboil kernels the reference pairs with tzgemm (src/Creator.cu:53-178, src/main.cu:108-159).
 * gptb_<k> (solo list + 6 geometry ints + start, step, end, thread_base), tzgemm_<k> (the list without
 * thread_base, then tzgemm's 7 + 6 + 3) and ori_<k> (the solo list; grid / block = the original launch).
 *   sgemm (6)  float* A, float* B, float* C, int M, int N, int K      C = 2 C + 2 A B; A [K][M], B [K][N], C [N][M];
 *              original grid (M / 128, N / 16), block (16, 8)           replaces general_ptb_sgemm
 *                                                                       (src/gptb_kernel/sgemm_kernel.cu:3-64)
 *   lbm (2)    float* srcGrid, float* dstGrid                           one D3Q19 step, scatter form; the pointers
 *              original grid (ny, nz), block (nx)                       address cell (0,0,0), two z-planes of margin
 *                                                                       on either side; nx % 32 == 0; replaces
 *                                                                       general_ptb_lbm (src/gptb_kernel/lbm_kernel.cu)
 *   fft (1)    float2* data                                             256-point transforms in place; replaces
 *              original grid (batch), block (128)                       g_general_ptb_fft (src/gptb_kernel/fft_kernel.cu)
 *   cutcp (10) int binDim_x, int binDim_y, float4* binZeroAddr,         replaces general_ptb_cutcp
 *              float h, float cutoff2, float inv_cutoff2,               (src/gptb_kernel/cutcp_kernel.cu:12-183);
 *              float* regionZeroAddr, int zRegionIndex_t,               nbr / nbrlen added: the table
 *              int4* nbr, int nbrlen                                    tk_cutcp_pack_neighbours writes, replacing
 *              original grid (gx, gy, gz) regions, block (8, 2, 8)      the __constant__ NbrList / NbrListLen
 *                                                                       (src/ori_kernel/cutcp_kernel.cu:12-13)
 * Results are the reference's bit for bit (each output has one fixed sequence of operations in all four). */
int tk_launch_gptb_sgemm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                         unsigned smem_bytes, void* stream);
int tk_launch_gptb_lbm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                       unsigned smem_bytes, void* stream);
int tk_launch_gptb_fft(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                       unsigned smem_bytes, void* stream);
int tk_launch_gptb_cutcp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                         unsigned smem_bytes, void* stream);
int tk_launch_mix_tzgemm_sgemm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                               unsigned smem_bytes, void* stream);
int tk_launch_mix_tzgemm_lbm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                             unsigned smem_bytes, void* stream);
int tk_launch_mix_tzgemm_fft(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                             unsigned smem_bytes, void* stream);
int tk_launch_mix_tzgemm_cutcp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                               unsigned smem_bytes, void* stream);
/* tzconv_<k>: the same pairs with the implicit-GEMM convolution as the tensor role (list, then tzconv's 12 + 6 + 3) */
int tk_launch_mix_tzconv_sgemm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                               unsigned smem_bytes, void* stream);
int tk_launch_mix_tzconv_lbm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                             unsigned smem_bytes, void* stream);
int tk_launch_mix_tzconv_fft(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                             unsigned smem_bytes, void* stream);
int tk_launch_mix_tzconv_cutcp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                               unsigned smem_bytes, void* stream);
int tk_launch_ori_sgemm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                        unsigned smem_bytes, void* stream);
int tk_launch_ori_lbm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                      unsigned smem_bytes, void* stream);
int tk_launch_ori_fft(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                      unsigned smem_bytes, void* stream);
int tk_launch_ori_cutcp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                        unsigned smem_bytes, void* stream);
/* neighbour offsets {dx, dy, dz} x n (device) -> the table of the cutcp kernels (device, 16-byte aligned, 16 n bytes) */
int tk_cutcp_pack_neighbours(const int* nbr_xyz, int n, void* table, void* stream);

/* ---- input preparation the reference does on the host -------------------------------------------
 * tk_cp_pack_atoms  replaces copyatomstoconstbuf (src/ori_kernel/cp_kernel.cu:159-179):
 *   atoms_xyzq[count][4] (device) -> packed[count] = {x, y, (zplane - z)^2, q} (device). */
int tk_cp_pack_atoms(const float* atoms_xyzq, int count, float zplane, float* packed, void* stream);
/* tk_mriq_pack_kvalues  replaces ori_ComputePhiMag plus the host loop that fills the kValues
 * structs (src/ori_kernel/mriq_kernel.cu:47-54, src/header/mriq_header.h:12-17). */
int tk_mriq_pack_kvalues(const float* kx, const float* ky, const float* kz, const float* phiR,
                         const float* phiI, int numK, float* kvals, void* stream);
/* tk_mrif_pack_kvalues  replaces ComputeRhoPhiGPU plus the host loop that fills the kValues structs
 * (src/ori_kernel/mrif_kernel.cu:63-76, src/header/mrif_header.h:27-33): RhoPhiR = phiR*dR + phiI*dI,
 * RhoPhiI = phiR*dI - phiI*dR.  kvals (device, 16-byte aligned) receives 5 * numK floats. */
int tk_mrif_pack_kvalues(const float* kx, const float* ky, const float* kz, const float* phiR,
                         const float* phiI, const float* dR, const float* dI, int numK, float* kvals,
                         void* stream);

/* ---- LC-layer helpers -----------------------------------------------------------------------------
 * tk_im2col_f32  replaces im2col_gpu_kernel (src/include/dnn.h:45-92): Caffe layout,
 *   data_col[(c*kh*kw + i*kw + j)][h_col][w_col], zero padding. */
int tk_im2col_f32(const float* data_im, int channels, int height, int width, int kernel_h, int kernel_w,
                  int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w,
                  float* data_col, void* stream);
/* tk_convert_fp32_to_fp16  replaces convertFp32ToFp16 (src/include/dnn.h:94-99); out is __half. */
int tk_convert_fp32_to_fp16(void* out_half, const float* in, long long n, void* stream);
/* tk_tzgemm_dims  replaces getTZGEMMGridDim (src/tzgemm_kernel.h:30-48): {M_GLOBAL, N_GLOBAL,
 *   K_GLOBAL, number of 64x64 tiles}. */
int tk_tzgemm_dims(int m, int n, int k, int out[4]);
/* tk_conv_mnk  replaces get_mnk_from_cudnn_args (src/TaskManager.cu:92-123). */
int tk_conv_mnk(const int cudnn_args[14], int mnk[3]);

/* ---- whole operators (device buffers; the caller supplies the scratch) ---------------------------
 * tk_mriq_compute = tk_mriq_pack_kvalues + every virtual block of gptb_mriq: the sequence
 *   OriMRIQKernel::initParams + executeImpl run (src/ori_kernel/mriq_kernel.cu:125-330).
 *   kvals_scratch: numK * 16 bytes of device memory, 16-byte aligned.  numX % 256 == 0. */
int tk_mriq_compute(const float* kx, const float* ky, const float* kz, const float* phiR, const float* phiI,
                    int numK, const float* x, const float* y, const float* z, float* Qr, float* Qi, int numX,
                    float* kvals_scratch, void* stream);
/* tk_coulomb_compute = tk_cp_pack_atoms + every virtual block of gptb_cp (OriCPKernel::initParams +
 *   executeImpl, src/ori_kernel/cp_kernel.cu:271-340, all atoms in one call).
 *   packed_scratch: numatoms * 16 bytes of device memory, 16-byte aligned.  nx % 128 == 0, ny % 8 == 0. */
int tk_coulomb_compute(const float* atoms_xyzq, int numatoms, float zplane, float gridspacing, float* energygrid,
                       int nx, int ny, float* packed_scratch, void* stream);

/* ---- host-buffer pair (what an end-to-end caller times) ---------------------------------------------
 * C = alpha * A * B^T together with `sweeps` ping-pong stencil sweeps of A0: the first two sweeps are fused
 * launches that each co-run with half of the GEMM's tiles, the remaining sweeps run alone.  All five buffers are HOST memory (pinned
 * for full copy speed).  Uploads, kernels and downloads run on three streams of the library and the workspace holds
 * two sets of device buffers used in turn, so the upload and the kernels of one call overlap the downloads of the
 * previous one (the downloads are the longer direction); `stream` joins at the end: the call returns once
 * everything is enqueued, and the results are in the host buffers once `stream` is synchronised.  The host input
 * buffers must be ready when the call is made (the uploads do not wait for `stream`), and host buffers must not be
 * reused for two calls in flight.  Mirrors what the reference's harness does around a
 * fused launch: cudaMemcpy of the inputs in initParams (src/ori_kernel/stencil_kernel.cu:143-160), the
 * launch (src/TaskManager.cu:285), and the copy-back its test mains do (fusion/code/cp_code.py:99-121).
 * workspace: device memory of at least tk_pair_tzgemm_stencil_workspace() bytes, 256-byte aligned. */
int tk_pair_tzgemm_stencil_workspace(int M, int N, int K, int nx, int ny, int nz, size_t* bytes);
int tk_pair_tzgemm_stencil_host(const void* A_host, const void* B_host, float* C_host, int M, int N, int K,
                                float alpha, float c0, float c1, const float* A0_host, float* Aout_host, int nx,
                                int ny, int nz, int sweeps, int cd_threads, void* workspace,
                                size_t workspace_bytes, void* stream);

/* ---- layer kernels of the LC / BE DNN tasks -------------------------------------------------------------
 * The reference's generated DNN classes call cuDNN / cuBLAS and NNFusion element-wise kernels for
 * everything that is not routed to tzgemm (the `<model>_kernel_class.h` files under src/dnn/); these are the hand-written
 * stand-ins.  Activations are fp32, NHWC for images, [rows][cols] for sequences.
 * tk_im2col_nhwc_f16: conv input -> tzgemm A operand in one pass (im2col_gpu_kernel + convertFp32ToFp16,
 *   src/include/dnn.h:45-99): A[m][k] fp16, m = oh*OW + ow, k = (i*kw + j)*C + c, zero padded to
 *   M_pad x K_pad (K_pad % 8 == 0). */
int tk_im2col_nhwc_f16(const float* x, int H, int W, int C, int kh, int kw, int pad, int stride, void* A_half,
                       int M_pad, int K_pad, void* stream);
/* fp32 [rows][ld_in] -> fp16 [rows_pad][cols_pad], zero padded (FC input -> tzgemm A operand) */
int tk_rows_f32_to_f16(const float* x, int rows, int cols, int ld_in, void* A_half, int rows_pad, int cols_pad,
                       void* stream);
/* out[r][c] = act(x[r][c] + bias[c]); act 0 none, 1 relu, 2 gelu; bias may be null */
int tk_bias_act_f32(const float* x, int ldx, const float* bias, float* out, int rows, int cols, int ld_out, int act,
                    void* stream);
int tk_maxpool2x2_nhwc_f32(const float* x, int H, int W, int C, float* out, void* stream);
int tk_add_f32(const float* a, const float* b, float* out, long long n, void* stream);
int tk_softmax_rows_f32(const float* x, float* out, long long rows, int cols, float scale, void* stream);
int tk_layernorm_rows_f32(const float* x, const float* gamma, const float* beta, float* out, long long rows, int cols,
                          float eps, void* stream);
/* out = layernorm((a + bias) + b) row by row (the bias of the product that made a, the residual addition and the
 * normalisation in one pass; bias [cols] and b may be null); rows of 128, 256, .., 1024 columns in 16-byte aligned arrays, else TK_ERR_SHAPE */
int tk_add_layernorm_rows_f32(const float* a, const float* bias, const float* b, const float* gamma, const float* beta,
                              float* out, void* out_half, long long rows, int cols, float eps, void* stream);
/* Producers that also (or only) write the fp16 operand of the product that follows, so that it needs no conversion
 * pass of its own: tk_add_layernorm_rows_f32 (b and out_half may be null; out_half is [rows][cols] fp16),
 * tk_bias_act_f32_f16 (out or out_half may be null; columns and leading dimensions multiples of 4),
 * tk_softmax_rows_f16, tk_merge_heads_f16, and tk_split_qkv_heads_f16: the heads of three projections that lie side by
 * side in one row (ld >= 3 * heads * dh; bias [3 * heads * dh] or null is added first), q and k as [B*heads][S][dh],
 * v transposed [B*heads][dh][S], in one launch (S and dh multiples of 32). */
int tk_bias_act_f32_f16(const float* x, int ldx, const float* bias, float* out, int ld_out, void* out_half, int ld_half,
                        int rows, int cols, int act, void* stream);
int tk_softmax_rows_f16(const float* x, void* out_half, long long rows, int cols, float scale, void* stream);
int tk_merge_heads_f16(const float* ctx, int B, int S, int heads, int dh, void* out_half, void* stream);
int tk_split_qkv_heads_f16(const float* x, const float* bias, int ld, int B, int S, int heads, int dh, void* q_half,
                           void* k_half, void* vt_half, void* stream);
/* x [B*S][ld] fp32, `heads` blocks of `dh` columns from col0 -> fp16 [B*heads][S][dh] (transpose 0) or
 * [B*heads][dh][S] (transpose 1); and the way back for the attention context */
int tk_split_heads_f16(const float* x, int ld, int col0, int B, int S, int heads, int dh, int transpose,
                       void* out_half, void* stream);
int tk_merge_heads_f32(const float* ctx, int B, int S, int heads, int dh, float* out, void* stream);
/* `batch` independent tzgemms of one shape in one launch (the attention GEMMs; the reference calls
 * cublasSgemmStridedBatched, src/dnn/bert/bert_kernel_class.h:2049).  Strides in elements, 0 = dense. */
int tk_tzgemm_batched(const void* A, const void* B, float* C, int M, int N, int K, int batch, long long stride_a,
                      long long stride_b, long long stride_c, float alpha, void* stream);

/* ---- work-distribution plans (host only, no device needed) -------------------------------------------------
 * The enumeration code of the persistent kernels, run on the host so that its invariants can be checked
 * exhaustively (the reference relies on compute-sanitizer-free trial runs of generated binaries,
 * fusion/code/gen_run.py:164-196).
 * tk_plan_tzgemm: cover[t] += 1 for every 64x64 tile t of the M x N result that a launch of `ctas` CTAs with
 *   super-tile width bn writes for [start, end); work[c] (optional) += super-tiles of CTA c.
 * tk_plan_stencil: planes[b*nz + k] += 1 for every plane k of bundle b some warp computes, loads[b*nz + k]
 *   (optional) += 1 for every plane streamed; split = {slabs per bundle, planes per slab} chosen for the launch. */
int tk_plan_tzgemm(int M, int N, int bn, int start, int end, int ctas, int* cover, int* work);
int tk_plan_tzgemm_m256(int M, int N, int start, int end, int ctas, int* cover); /* 256 x 256 super-tile kernel */
int tk_plan_stencil(int nz, int blocks_start, int blocks_end, int gx, int gy, int ctas, int warps_per_cta,
                    int* planes, int* loads, int split[2]);

/* ---- MRI-Q for callers that cannot allocate device memory ----------------------------------------------
 * (No counterpart in the reference: it always cudaMallocs its buffers up front.)
 * Same computation and same results as tk_mriq_compute, but the packed k-space table is a fixed array
 * inside the library instead of caller-supplied scratch, so the call needs no buffer beyond its inputs
 * and outputs.  Meant for code that runs where cudaMalloc is off limits: inside a real-time or
 * latency-critical loop that must not take the allocator's locks or implicit synchronisation, in a
 * process whose device memory has been handed out completely to a pool owned by someone else, or in
 * a plug-in that is only given the buffers of its host application.
 *   - Limit: numK <= TK_MRIQ_STATIC_MAX_K samples; more returns TK_ERR_CAPACITY (tk_last_error() says
 *     so) and nothing is launched.  The table costs 64 KiB of device memory on every GPU that loads the
 *     library, for the life of the process.
 *   - The first call on each device looks the table's device address up (cudaGetSymbolAddress, with
 *     that device current).  Make that first call before starting any stream capture.
 *   - It calls no cudaMalloc/cudaFree and no allocating library routine.
 *   - All calls on one device share the table.  Calls that overlap on the GPU (different streams, or
 *     different host threads without ordering) race on it; calls queued on one stream are safe.  The
 *     table keeps the last call's samples, which the next call overwrites before reading. */
#define TK_MRIQ_STATIC_MAX_K 4096
int tk_mriq_compute_static(const float* kx, const float* ky, const float* kz, const float* phiR,
                           const float* phiI, int numK, const float* x, const float* y, const float* z,
                           float* Qr, float* Qi, int numX, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TACKER_B200_H */
