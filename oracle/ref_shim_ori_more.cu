// ref_shim_ori_more.cu -- the REFERENCE's unfused, non-persistent kernels ori_sgemm, ori_lbm, ori_fft and ori_cutcp
// (unmodified, #included from the reference tree given with -I at build time); second translation unit of
// oracle/_ref/libtacker_ref_ori.so (see ref_shim_ori.cu: test infrastructure only).  Only the launch wrappers below
// are code of this repository.
#include "Logger.h"
#include "ModuleCenter.h"

#include "ori_kernel/cutcp_kernel.cu"
#include "ori_kernel/fft_kernel.cu"
#include "ori_kernel/sgemm_kernel.cu"
// lbm last: its header names cell entries C, N, S, E, W, T, B, ... at file scope
#include "ori_kernel/lbm_kernel.cu"

#define REF_API extern "C" __attribute__((visibility("default")))

static int last_error_more() { return static_cast<int>(cudaGetLastError()); }

// C = 2 C + 2 A B with the reference's layouts: A [K][M], B [K][N], C [N][M]; geometry of
// src/ori_kernel/sgemm_kernel.cu:116-121
REF_API int ref_ori_sgemm(float* A, float* B, float* C, int M, int N, int K, void* stream) {
    ori_sgemm<<<dim3(M / TILE_M, N / TILE_N), dim3(TILE_N, TILE_TB_HEIGHT), 0, static_cast<cudaStream_t>(stream)>>>(
        A, B, C, M, N, K);
    return last_error_more();
}

// src / dst point at cell (0, 0, 0) of element 0; geometry of src/ori_kernel/lbm_kernel.cu:222-226
REF_API int ref_ori_lbm(float* src, float* dst, void* stream) {
    ori_lbm<<<dim3(SIZE_Y, SIZE_Z), SIZE_X, 0, static_cast<cudaStream_t>(stream)>>>(src, dst);
    return last_error_more();
}

// `nfft` transforms of 256 points, in place (one block per transform, src/ori_kernel/fft_kernel.cu:48-60)
REF_API int ref_ori_fft(void* data, int nfft, void* stream) {
    ori_fft<<<nfft, FFT_T, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<float2*>(data));
    return last_error_more();
}

// bins_dev: device copy of the bins (base address); regions_dev: gx * gy * gz regions of 512 floats; one block per
// region (src/ori_kernel/cutcp_kernel.cu:19-43, block 8 x 2 x 8 as at :252-258)
REF_API int ref_ori_cutcp(const int* nbr_host, int nbrlen, int binDim_x, int binDim_y, int c, void* bins_dev, float h,
                          float cutoff2, float inv_cutoff2, float* regions_dev, int gx, int gy, int gz, void* stream) {
    if (nbrlen > NBRLIST_MAXLEN) return -2;
    cudaError_t e = cudaMemcpyToSymbol(NbrListLen, &nbrlen, sizeof(int));
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaMemcpyToSymbol(NbrList, nbr_host, nbrlen * sizeof(int3));
    if (e != cudaSuccess) return static_cast<int>(e);
    float4* zero = static_cast<float4*>(bins_dev) + ((c * binDim_y + c) * binDim_x + c) * BIN_DEPTH;
    ori_cutcp<<<dim3(gx, gy, gz), dim3(8, 2, 8), 0, static_cast<cudaStream_t>(stream)>>>(
        binDim_x, binDim_y, zero, h, cutoff2, inv_cutoff2, regions_dev, gz - 1);
    return last_error_more();
}
