#include "ori_kernels.h"

#include <vector>

#include "../Logger.h"

namespace {
float* upload_uniform(size_t n, uint64_t seed, float lo, float hi) {
    std::vector<float> h(n);
    for (size_t i = 0; i < n; ++i) h[i] = lo + tk_unit_draw(seed, i) * (hi - lo);
    float* d = static_cast<float*>(backend().deviceAlloc(n * sizeof(float)));
    backend().upload(d, h.data(), n * sizeof(float), nullptr);
    backend().streamSync(nullptr);
    return d;
}
}  // namespace

// ---------------------------------------------------------------- stencil ----
OriSTENCILKernel::OriSTENCILKernel(int id, StencilProblem p) : prob(p) {
    Id = id;
    kernelName = "stencil";
    funcKey = "ori_stencil";
    initParams();
    loadKernel();
}
OriSTENCILKernel::~OriSTENCILKernel() {
    for (auto& ptr : cudaFreeList) backend().deviceFree(ptr);
}
void OriSTENCILKernel::initParams() {
    if (initialized) return;
    nx = prob.nx;
    ny = prob.ny;
    nz = prob.nz;
    c0 = prob.c0;
    c1 = prob.c1;
    const size_t n = static_cast<size_t>(nx) * ny * nz;
    A0 = upload_uniform(n, 1337, 0.0f, 1.0f);  // the reference seeds cuRAND with 1337
    Anext = static_cast<float*>(backend().deviceAlloc(n * sizeof(float)));
    // Anext starts as a copy of A0, so boundary cells hold A0's values (stencil_kernel.cu:160)
    {
        std::vector<float> h(n);
        backend().download(h.data(), A0, n * sizeof(float), nullptr);
        backend().streamSync(nullptr);
        backend().upload(Anext, h.data(), n * sizeof(float), nullptr);
        backend().streamSync(nullptr);
    }
    cudaFreeList.push_back(A0);
    cudaFreeList.push_back(Anext);
    launchBlockDim = dim3h(32, 4, 1);  // tile_x, tile_y (src/header/stencil_header.h:2-3)
    launchGridDim = dim3h((nx + 63) / 64, (ny + 3) / 4, 1);
    kernelParams = {&c0, &c1, &A0, &Anext, &nx, &ny, &nz};
    smem = 0;
    initialized = true;
}
void OriSTENCILKernel::loadKernel() {
    kernelFunc = reinterpret_cast<void*>(backend().lookup(funcKey));
    if (!kernelFunc) logger.ERROR("load kernel {" + funcKey + "} failed!");
}

// ---------------------------------------------------------------- coulomb ----
OriCPKernel::OriCPKernel(int id, CPProblem p) : prob(p) {
    Id = id;
    kernelName = "cp";
    funcKey = "ori_cp";
    initParams();
    loadKernel();
}
OriCPKernel::~OriCPKernel() {
    for (auto& ptr : cudaFreeList) backend().deviceFree(ptr);
}
void OriCPKernel::initParams() {
    const size_t cells = static_cast<size_t>(prob.nx) * prob.ny;
    if (initialized) {  // the reference re-zeroes the lattice on every initParams (cp_kernel.cu:288)
        backend().fillZero(energygrid, cells * sizeof(float), initStream);
        return;
    }
    numatoms = prob.atoms;
    gridspacing = prob.spacing;
    std::vector<float> h(4 * static_cast<size_t>(numatoms));
    for (int i = 0; i < numatoms; ++i) {  // positions in the box, charge in [-1, 1] (initatoms, cp_kernel.cu:185-209)
        h[4 * i + 0] = tk_unit_draw(54321, 4ull * i + 0) * prob.box;
        h[4 * i + 1] = tk_unit_draw(54321, 4ull * i + 1) * prob.box;
        h[4 * i + 2] = tk_unit_draw(54321, 4ull * i + 2) * prob.box;
        h[4 * i + 3] = tk_unit_draw(54321, 4ull * i + 3) * 2.0f - 1.0f;
    }
    float* raw = static_cast<float*>(backend().deviceAlloc(h.size() * sizeof(float)));
    atoms = static_cast<float*>(backend().deviceAlloc(h.size() * sizeof(float)));
    backend().upload(raw, h.data(), h.size() * sizeof(float), nullptr);
    TK_HOST_CHECK(backend().cpPackAtoms(raw, numatoms, prob.zplane, atoms, nullptr));  // copyatomstoconstbuf
    backend().streamSync(nullptr);
    backend().deviceFree(raw);
    energygrid = static_cast<float*>(backend().deviceAlloc(cells * sizeof(float)));
    backend().fillZero(energygrid, cells * sizeof(float), nullptr);
    backend().streamSync(nullptr);
    cudaFreeList.push_back(atoms);
    cudaFreeList.push_back(energygrid);
    launchBlockDim = dim3h(16, 8, 1);  // BLOCKSIZEX, BLOCKSIZEY (src/header/cp_header.h:2-3)
    launchGridDim = dim3h(prob.nx / 128, prob.ny / 8, 1);
    kernelParams = {&numatoms, &gridspacing, &energygrid, &atoms};
    smem = 0;
    initialized = true;
}
void OriCPKernel::loadKernel() {
    kernelFunc = reinterpret_cast<void*>(backend().lookup(funcKey));
    if (!kernelFunc) logger.ERROR("load kernel {" + funcKey + "} failed!");
}

// ------------------------------------------------------------------ mri-q ----
OriMRIQKernel::OriMRIQKernel(int id, MRIQProblem p) : prob(p) {
    Id = id;
    kernelName = "mriq";
    funcKey = "ori_mriq";
    initParams();
    loadKernel();
}
OriMRIQKernel::~OriMRIQKernel() {
    for (auto& ptr : cudaFreeList) backend().deviceFree(ptr);
}
void OriMRIQKernel::initParams() {
    const size_t nX = static_cast<size_t>(prob.numX);
    if (initialized) {
        backend().fillZero(Qr, nX * sizeof(float), initStream);
        backend().fillZero(Qi, nX * sizeof(float), initStream);
        return;
    }
    numK = prob.numK;
    float* kx = upload_uniform(numK, 401, -0.5f, 0.5f);
    float* ky = upload_uniform(numK, 402, -0.5f, 0.5f);
    float* kz = upload_uniform(numK, 403, -0.5f, 0.5f);
    float* phiR = upload_uniform(numK, 404, 0.0f, 1.0f);
    float* phiI = upload_uniform(numK, 405, 0.0f, 1.0f);
    kvals = static_cast<float*>(backend().deviceAlloc(4ull * numK * sizeof(float)));
    TK_HOST_CHECK(backend().mriqPackKvalues(kx, ky, kz, phiR, phiI, numK, kvals, nullptr));  // ComputePhiMag + pack
    backend().streamSync(nullptr);
    for (float* p : {kx, ky, kz, phiR, phiI}) backend().deviceFree(p);
    x = upload_uniform(nX, 601, -32.0f, 32.0f);
    y = upload_uniform(nX, 602, -32.0f, 32.0f);
    z = upload_uniform(nX, 603, -32.0f, 32.0f);
    Qr = static_cast<float*>(backend().deviceAlloc(nX * sizeof(float)));
    Qi = static_cast<float*>(backend().deviceAlloc(nX * sizeof(float)));
    backend().fillZero(Qr, nX * sizeof(float), nullptr);
    backend().fillZero(Qi, nX * sizeof(float), nullptr);
    backend().streamSync(nullptr);
    for (float* p : {kvals, x, y, z, Qr, Qi}) cudaFreeList.push_back(p);
    launchBlockDim = dim3h(256, 1, 1);  // KERNEL_Q_THREADS_PER_BLOCK (src/header/mriq_header.h:9)
    launchGridDim = dim3h(prob.numX / 256, 1, 1);
    kernelParams = {&numK, &kGlobalIndex, &x, &y, &z, &Qr, &Qi, &kvals};
    smem = 0;
    initialized = true;
}
void OriMRIQKernel::loadKernel() {
    kernelFunc = reinterpret_cast<void*>(backend().lookup(funcKey));
    if (!kernelFunc) logger.ERROR("load kernel {" + funcKey + "} failed!");
}

// ---------------------------------------------------------------- mri-fhd ----
OriMRIFKernel::OriMRIFKernel(int id, MRIFProblem p) : prob(p) {
    Id = id;
    kernelName = "mrif";
    funcKey = "ori_mrif";
    initParams();
    loadKernel();
}
OriMRIFKernel::~OriMRIFKernel() {
    for (auto& ptr : cudaFreeList) backend().deviceFree(ptr);
}
void OriMRIFKernel::initParams() {
    const size_t nX = static_cast<size_t>(prob.numX);
    if (initialized) {  // the outputs accumulate (+=): a new run starts from zero
        backend().fillZero(outR, nX * sizeof(float), initStream);
        backend().fillZero(outI, nX * sizeof(float), initStream);
        return;
    }
    numK = prob.numK;
    float* kx = upload_uniform(numK, 701, -0.5f, 0.5f);
    float* ky = upload_uniform(numK, 702, -0.5f, 0.5f);
    float* kz = upload_uniform(numK, 703, -0.5f, 0.5f);
    float* phiR = upload_uniform(numK, 704, -1.0f, 1.0f);
    float* phiI = upload_uniform(numK, 705, -1.0f, 1.0f);
    float* dR = upload_uniform(numK, 706, -1.0f, 1.0f);
    float* dI = upload_uniform(numK, 707, -1.0f, 1.0f);
    kvals = static_cast<float*>(backend().deviceAlloc(5ull * numK * sizeof(float)));
    TK_HOST_CHECK(backend().mrifPackKvalues(kx, ky, kz, phiR, phiI, dR, dI, numK, kvals, nullptr));  // ComputeRhoPhiGPU + pack
    backend().streamSync(nullptr);
    for (float* p : {kx, ky, kz, phiR, phiI, dR, dI}) backend().deviceFree(p);
    x = upload_uniform(nX, 801, -32.0f, 32.0f);
    y = upload_uniform(nX, 802, -32.0f, 32.0f);
    z = upload_uniform(nX, 803, -32.0f, 32.0f);
    outR = static_cast<float*>(backend().deviceAlloc(nX * sizeof(float)));
    outI = static_cast<float*>(backend().deviceAlloc(nX * sizeof(float)));
    backend().fillZero(outR, nX * sizeof(float), nullptr);
    backend().fillZero(outI, nX * sizeof(float), nullptr);
    backend().streamSync(nullptr);
    for (float* p : {kvals, x, y, z, outR, outI}) cudaFreeList.push_back(p);
    launchBlockDim = dim3h(256, 1, 1);  // KERNEL_FH_THREADS_PER_BLOCK (src/header/mrif_header.h:11)
    launchGridDim = dim3h(prob.numX / 256, 1, 1);
    kernelParams = {&numK, &kGlobalIndex, &x, &y, &z, &outR, &outI, &kvals};
    smem = 0;
    initialized = true;
}
void OriMRIFKernel::loadKernel() {
    kernelFunc = reinterpret_cast<void*>(backend().lookup(funcKey));
    if (!kernelFunc) logger.ERROR("load kernel {" + funcKey + "} failed!");
}
