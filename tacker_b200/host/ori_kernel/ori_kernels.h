// The CUDA-core benchmark operators as host objects: allocate and seed their inputs, hold the
// argument list and the original launch geometry (reference: src/ori_kernel/stencil_kernel.cu:114-204,
// cp_kernel.cu:150-340, mriq_kernel.cu:107-330, mrif_kernel.cu:152-330, sgemm_kernel.cu:46-150, lbm_kernel.cu:158-225,
// fft_kernel.cu:63-125, cutcp_kernel.cu:167-330).  Inputs are seeded synthetically (the reference reads
// MRI-Q input from a file that is not distributed and seeds the others with cuRAND / rand()).
#pragma once
#include "../Kernel.h"

struct StencilProblem {
    int nx = 512, ny = 512, nz = 64;
    float c0 = 1.0f / 6.0f, c1 = 1.0f / 6.0f / 6.0f;  // src/ori_kernel/stencil_kernel.cu:132-133
};
struct CPProblem {
    int nx = 512, ny = 512, atoms = 8192;
    float spacing = 0.125f, zplane = 32.0f, box = 64.0f;
};
struct MRIQProblem {
    int numK = 2048, numX = 262144;
};
struct MRIFProblem {
    int numK = 2048, numX = 262144;
};
struct SGEMMProblem {
    int M = 4096, N = 4128, K = 4064;  // src/ori_kernel/sgemm_kernel.cu:85-87
};
struct LBMProblem {
    int nx = 128, ny = 128, nz = 128;  // src/header/lbm_header.h:17-19
};
struct FFTProblem {
    int batch = 10240;                 // FFT_B, src/header/fft_header.h:13
};
struct CUTCPProblem {
    // lattice points and spacing; the reference's input gives 208^3 points of which its launch covers two slabs of
    // regions in z (src/ori_kernel/cutcp_kernel.cu:243-275)
    int nx = 208, ny = 208, nz = 16;
    float h = 0.5f, cutoff = 12.0f, density = 0.1f;  // atoms per cubic Angstrom (src/header/cutcp_header.h:8-9)
};

class OriSTENCILKernel : public Kernel {
public:
    explicit OriSTENCILKernel(int id, StencilProblem p = StencilProblem());
    ~OriSTENCILKernel() override;
    void initParams() override;
    void loadKernel() override;
    std::vector<int> getArgs() override { return std::vector<int>(); }
    StencilProblem prob;
    float c0, c1;
    float* A0 = nullptr;
    float* Anext = nullptr;
    int nx, ny, nz;

protected:
    void executeImpl(stream_t stream) override { launch(kernelParams, stream); }
};

class OriCPKernel : public Kernel {
public:
    explicit OriCPKernel(int id, CPProblem p = CPProblem());
    ~OriCPKernel() override;
    void initParams() override;
    void loadKernel() override;
    std::vector<int> getArgs() override { return std::vector<int>(); }
    CPProblem prob;
    int numatoms;
    float gridspacing;
    float* energygrid = nullptr;
    float* atoms = nullptr;  // packed {x, y, dz^2, q}

protected:
    void executeImpl(stream_t stream) override { launch(kernelParams, stream); }
};

class OriMRIQKernel : public Kernel {
public:
    explicit OriMRIQKernel(int id, MRIQProblem p = MRIQProblem());
    ~OriMRIQKernel() override;
    void initParams() override;
    void loadKernel() override;
    std::vector<int> getArgs() override { return std::vector<int>(); }
    MRIQProblem prob;
    int numK, kGlobalIndex = 0;
    float *x = nullptr, *y = nullptr, *z = nullptr, *Qr = nullptr, *Qi = nullptr, *kvals = nullptr;

protected:
    void executeImpl(stream_t stream) override { launch(kernelParams, stream); }
};

class OriMRIFKernel : public Kernel {
public:
    explicit OriMRIFKernel(int id, MRIFProblem p = MRIFProblem());
    ~OriMRIFKernel() override;
    void initParams() override;
    void loadKernel() override;
    std::vector<int> getArgs() override { return std::vector<int>(); }
    MRIFProblem prob;
    int numK, kGlobalIndex = 0;
    float *x = nullptr, *y = nullptr, *z = nullptr, *outR = nullptr, *outI = nullptr, *kvals = nullptr;

protected:
    void executeImpl(stream_t stream) override { launch(kernelParams, stream); }
};

// C = 2 C + 2 A B on uniform random matrices: A [K][M], B [K][N], C [N][M]
class OriSGEMMKernel : public Kernel {
public:
    explicit OriSGEMMKernel(int id, SGEMMProblem p = SGEMMProblem());
    ~OriSGEMMKernel() override;
    void initParams() override;
    void loadKernel() override;
    std::vector<int> getArgs() override { return std::vector<int>(); }
    SGEMMProblem prob;
    float *A = nullptr, *B = nullptr, *C = nullptr;
    int M, N, K;

protected:
    void executeImpl(stream_t stream) override { launch(kernelParams, stream); }
};

// one lattice-Boltzmann step on a uniform random grid (flags included, as in the reference)
class OriLBMKernel : public Kernel {
public:
    explicit OriLBMKernel(int id, LBMProblem p = LBMProblem());
    ~OriLBMKernel() override;
    void initParams() override;
    void loadKernel() override;
    std::vector<int> getArgs() override { return std::vector<int>(); }
    LBMProblem prob;
    float *src = nullptr, *dst = nullptr;  // cell (0, 0, 0) of element 0; the allocations start two z-planes earlier

protected:
    void executeImpl(stream_t stream) override { launch(kernelParams, stream); }
};

// `batch` transforms of 256 complex points, in place
class OriFFTKernel : public Kernel {
public:
    explicit OriFFTKernel(int id, FFTProblem p = FFTProblem());
    ~OriFFTKernel() override;
    void initParams() override;
    void loadKernel() override;
    std::vector<int> getArgs() override { return std::vector<int>(); }
    FFTProblem prob;
    float* data = nullptr;

protected:
    void executeImpl(stream_t stream) override { launch(kernelParams, stream); }
};

// cutoff Coulomb potential: atoms hashed into bins on the host, neighbour table uploaded
class OriCUTCPKernel : public Kernel {
public:
    explicit OriCUTCPKernel(int id, CUTCPProblem p = CUTCPProblem());
    ~OriCUTCPKernel() override;
    void initParams() override;
    void loadKernel() override;
    std::vector<int> getArgs() override { return std::vector<int>(); }
    CUTCPProblem prob;
    int binDim_x, binDim_y, binDim_z, zRegionIndex_t, nbrlen;
    float h, cutoff2, inv_cutoff2;
    float* binZero = nullptr;  // bin at the lattice origin (inside the allocation `bins`)
    float* bins = nullptr;
    float* regions = nullptr;
    int* nbr = nullptr;        // {dx, dy, dz, 0} x nbrlen
    int extraAtoms = 0;        // atoms that found no room in their bin (the reference computes these on the CPU)

protected:
    void executeImpl(stream_t stream) override { launch(kernelParams, stream); }
};
