// The CUDA-core benchmark operators as host objects: allocate and seed their inputs, hold the
// argument list and the original launch geometry (reference: src/ori_kernel/stencil_kernel.cu:114-204,
// cp_kernel.cu:150-340, mriq_kernel.cu:107-330, mrif_kernel.cu:152-330).  Inputs are seeded synthetically (the reference reads
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
