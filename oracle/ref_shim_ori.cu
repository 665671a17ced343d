// ref_shim_ori.cu -- the REFERENCE's unfused, non-persistent kernels ori_stencil, ori_cp, ori_mriq and ori_mrif
// (unmodified, #included from the reference tree given with -I at build time), built into
// oracle/_ref/libtacker_ref_ori.so together with ref_shim_ori_more.cu and the reference's own Logger.cc and
// ModuleCenter.cu, which the host classes in those files refer to.
//
// TEST INFRASTRUCTURE ONLY, like ref_shim.cu: it pins the CPU restatement (tacker_oracle.c) through
// tests/golden/ref_ori.npz and is never linked or loaded by the product.  Only the launch wrappers below are code of
// this repository.  The header the reference's CMake step would generate is replaced by ref_stub/TackerConfig.h.
#include "Logger.h"
#include "ModuleCenter.h"

// the two globals the reference defines in src/main.cu:102-104 and every ori_kernel source declares extern
Logger logger(LOG_FILE_PATH, false, false);
ModuleCenter moduleCenter;

#include "ori_kernel/cp_kernel.cu"
#include "ori_kernel/mrif_kernel.cu"
#include "ori_kernel/mriq_kernel.cu"
#include "ori_kernel/stencil_kernel.cu"

#define REF_API extern "C" __attribute__((visibility("default")))

static int last_error() { return static_cast<int>(cudaGetLastError()); }

// launch geometry of src/ori_kernel/stencil_kernel.cu:173-178
REF_API int ref_ori_stencil(float c0, float c1, float* A0, float* Anext, int nx, int ny, int nz, void* stream) {
    const dim3 grid((nx + tile_x * 2 - 1) / (tile_x * 2), (ny + tile_y - 1) / tile_y), block(tile_x, tile_y);
    ori_stencil<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(c0, c1, A0, Anext, nx, ny, nz);
    return last_error();
}

// atoms: host array of packed {x, y, dz^2, q}, fed MAXATOMS at a time through the constant buffer with one launch
// per chunk (src/ori_kernel/cp_kernel.cu:159-179, 314); lattice of gx * 128 by gy * 8 points
REF_API int ref_ori_cp(const float* packed_host, int count, float spacing, float* lattice, int gx, int gy, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int a0 = 0; a0 < count; a0 += MAXATOMS) {
        const int n = count - a0 < MAXATOMS ? count - a0 : MAXATOMS;
        cudaError_t e = cudaMemcpyToSymbolAsync(atominfo, packed_host + 4 * a0, n * 4 * sizeof(float), 0,
                                                cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return static_cast<int>(e);
        ori_cp<<<dim3(gx, gy), dim3(BLOCKSIZEX, BLOCKSIZEY), 0, st>>>(n, spacing, lattice);
        if (last_error()) return -1;
        e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    return 0;
}

// kvals: host array of {Kx, Ky, Kz, PhiMag}, KERNEL_Q_K_ELEMS_PER_GRID per launch (src/ori_kernel/mriq_kernel.cu:244-257)
REF_API int ref_ori_mriq(const float* kvals_host, int numK, float* x, float* y, float* z, float* Qr, float* Qi, int numX,
                         void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (numK % 2) return -2;
    for (int k0 = 0; k0 < numK; k0 += KERNEL_Q_K_ELEMS_PER_GRID) {
        const int n = numK - k0 < KERNEL_Q_K_ELEMS_PER_GRID ? numK - k0 : KERNEL_Q_K_ELEMS_PER_GRID;
        cudaError_t e = cudaMemcpyToSymbolAsync(ck, kvals_host + 4 * k0, n * sizeof(mriq_kValues), 0,
                                                cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return static_cast<int>(e);
        ori_mriq<<<numX / KERNEL_Q_THREADS_PER_BLOCK, KERNEL_Q_THREADS_PER_BLOCK, 0, st>>>(n, 0, x, y, z, Qr, Qi);
        if (last_error()) return -1;
        e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    return 0;
}

// kvals: host array of the reference's structs {Kx, Ky, Kz, RhoPhiR, RhoPhiI}, KERNEL_FH_K_ELEMS_PER_GRID per launch
// (src/ori_kernel/mrif_kernel.cu:291-304)
REF_API int ref_ori_mrif(const float* kvals_host, int numK, float* x, float* y, float* z, float* outR, float* outI,
                         int numX, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int k0 = 0; k0 < numK; k0 += KERNEL_FH_K_ELEMS_PER_GRID) {
        const int n = numK - k0 < KERNEL_FH_K_ELEMS_PER_GRID ? numK - k0 : KERNEL_FH_K_ELEMS_PER_GRID;
        cudaError_t e = cudaMemcpyToSymbolAsync(c, kvals_host + 5 * k0, n * sizeof(mrif_kValues), 0,
                                                cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return static_cast<int>(e);
        ori_mrif<<<numX / KERNEL_FH_THREADS_PER_BLOCK, KERNEL_FH_THREADS_PER_BLOCK, 0, st>>>(n, 0, x, y, z, outR, outI);
        if (last_error()) return -1;
        e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    return 0;
}
