#include "ori_kernels.h"

#include <cmath>
#include <cstring>
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

// ------------------------------------------------------------------ sgemm ----
OriSGEMMKernel::OriSGEMMKernel(int id, SGEMMProblem p) : prob(p) {
    Id = id;
    kernelName = "sgemm";
    funcKey = "ori_sgemm";
    initParams();
    loadKernel();
}
OriSGEMMKernel::~OriSGEMMKernel() {
    for (auto& ptr : cudaFreeList) backend().deviceFree(ptr);
}
void OriSGEMMKernel::initParams() {
    if (initialized) {  // C is updated in place (C = 2 C + ..): a new run starts from zero
        backend().fillZero(C, static_cast<size_t>(M) * N * sizeof(float), initStream);
        return;
    }
    M = prob.M;
    N = prob.N;
    K = prob.K;
    A = upload_uniform(static_cast<size_t>(M) * K, 1337, 0.0f, 1.0f);  // curandGenerateUniform, seed 1337
    B = upload_uniform(static_cast<size_t>(K) * N, 1338, 0.0f, 1.0f);
    C = static_cast<float*>(backend().deviceAlloc(static_cast<size_t>(M) * N * sizeof(float)));
    backend().fillZero(C, static_cast<size_t>(M) * N * sizeof(float), nullptr);
    backend().streamSync(nullptr);
    for (float* q : {A, B, C}) cudaFreeList.push_back(q);
    launchBlockDim = dim3h(16, 8, 1);              // TILE_N x TILE_TB_HEIGHT (src/header/sgemm_header.h:1-3)
    launchGridDim = dim3h(M / 128, N / 16, 1);
    kernelParams = {&A, &B, &C, &M, &N, &K};
    smem = 0;
    initialized = true;
}
void OriSGEMMKernel::loadKernel() {
    kernelFunc = reinterpret_cast<void*>(backend().lookup(funcKey));
    if (!kernelFunc) logger.ERROR("load kernel {" + funcKey + "} failed!");
}

// -------------------------------------------------------------------- lbm ----
OriLBMKernel::OriLBMKernel(int id, LBMProblem p) : prob(p) {
    Id = id;
    kernelName = "lbm";
    funcKey = "ori_lbm";
    initParams();
    loadKernel();
}
OriLBMKernel::~OriLBMKernel() {
    for (auto& ptr : cudaFreeList) backend().deviceFree(ptr);
}
void OriLBMKernel::initParams() {
    if (initialized) return;
    const size_t cells = static_cast<size_t>(prob.nx) * prob.ny * prob.nz;
    const size_t margin = 2ull * prob.nx * prob.ny;  // REAL_MARGIN: two z-planes (src/header/lbm_header.h:246)
    const size_t total = 20 * cells + 2 * margin;
    float* s0 = upload_uniform(total, 1337, 0.0f, 1.0f);
    float* d0 = upload_uniform(total, 1338, 0.0f, 1.0f);
    cudaFreeList.push_back(s0);
    cudaFreeList.push_back(d0);
    src = s0 + margin;
    dst = d0 + margin;
    launchBlockDim = dim3h(prob.nx, 1, 1);
    launchGridDim = dim3h(prob.ny, prob.nz, 1);
    kernelParams = {&src, &dst};
    smem = 0;
    initialized = true;
}
void OriLBMKernel::loadKernel() {
    kernelFunc = reinterpret_cast<void*>(backend().lookup(funcKey));
    if (!kernelFunc) logger.ERROR("load kernel {" + funcKey + "} failed!");
}

// -------------------------------------------------------------------- fft ----
OriFFTKernel::OriFFTKernel(int id, FFTProblem p) : prob(p) {
    Id = id;
    kernelName = "fft";
    funcKey = "ori_fft";
    initParams();
    loadKernel();
}
OriFFTKernel::~OriFFTKernel() {
    for (auto& ptr : cudaFreeList) backend().deviceFree(ptr);
}
void OriFFTKernel::initParams() {
    if (initialized) return;
    data = upload_uniform(static_cast<size_t>(prob.batch) * 512, 54321, -1.0f, 1.0f);  // srand(54321), values in [-1, 1)
    cudaFreeList.push_back(data);
    launchBlockDim = dim3h(128, 1, 1);  // FFT_T
    launchGridDim = dim3h(prob.batch, 1, 1);
    kernelParams = {&data};
    smem = 0;
    initialized = true;
}
void OriFFTKernel::loadKernel() {
    kernelFunc = reinterpret_cast<void*>(backend().lookup(funcKey));
    if (!kernelFunc) logger.ERROR("load kernel {" + funcKey + "} failed!");
}

// ------------------------------------------------------------------ cutcp ----
OriCUTCPKernel::OriCUTCPKernel(int id, CUTCPProblem p) : prob(p) {
    Id = id;
    kernelName = "cutcp";
    funcKey = "ori_cutcp";
    initParams();
    loadKernel();
}
OriCUTCPKernel::~OriCUTCPKernel() {
    for (auto& ptr : cudaFreeList) backend().deviceFree(ptr);
}
void OriCUTCPKernel::initParams() {
    constexpr float kBinLen = 4.0f, kBinInv = 1.0f / kBinLen;  // BIN_LENGTH (src/header/cutcp_header.h:7-8)
    constexpr int kBinDepth = 8;
    const int gx = (prob.nx + 7) / 8, gy = (prob.ny + 7) / 8, gz = (prob.nz + 7) / 8;
    if (initialized) {
        backend().fillZero(regions, 512ull * gx * gy * gz * sizeof(float), initStream);
        return;
    }
    h = prob.h;
    cutoff2 = prob.cutoff * prob.cutoff;
    inv_cutoff2 = 1.0f / cutoff2;
    // bins: the lattice's box plus c bins of margin on every side (src/header/cutcp_header.h:163-170)
    const int c = static_cast<int>(std::ceil(prob.cutoff * kBinInv));
    binDim_x = static_cast<int>(std::ceil(8 * gx * h * kBinInv)) + 2 * c;
    binDim_y = static_cast<int>(std::ceil(8 * gy * h * kBinInv)) + 2 * c;
    binDim_z = static_cast<int>(std::ceil(8 * gz * h * kBinInv)) + 2 * c;
    const size_t nbins = static_cast<size_t>(binDim_x) * binDim_y * binDim_z;
    // neighbour offsets: every bin that can hold an atom within the cutoff of a point of the region around the centre
    // bin (src/header/cutcp_header.h:176-218; the two cases differ in how far a region reaches beyond its bin)
    std::vector<int> table;
    {
        const float ratio = kBinLen / (8 * h);
        float s = 0.0f;
        if (std::ceil(ratio) == std::floor(ratio)) s = std::sqrt(3.0f);
        else if (8 * h <= 2 * kBinLen) s = 2.0f * std::sqrt(3.0f);
        else logger.ERROR("cutcp: lattice spacing above a quarter of the bin length");
        const float r2 = (prob.cutoff + s * kBinLen) * (prob.cutoff + s * kBinLen);
        for (int k = -c; k <= c; ++k)
            for (int j = -c; j <= c; ++j)
                for (int i = -c; i <= c; ++i) {
                    if ((i * i + j * j + k * k) * kBinLen * kBinLen >= r2) continue;
                    table.insert(table.end(), {i, j, k, 0});
                }
    }
    nbrlen = static_cast<int>(table.size() / 4);
    // atoms at `density` per cubic Angstrom in the box of the bins, hashed into them; a full bin drops the atom
    std::vector<float> hb(nbins * kBinDepth * 4, 0.0f);
    std::vector<int> count(nbins, 0);
    const float ext[3] = {binDim_x * kBinLen, binDim_y * kBinLen, binDim_z * kBinLen};
    const size_t natoms = static_cast<size_t>(prob.density * ext[0] * ext[1] * ext[2]);
    extraAtoms = 0;
    for (size_t n = 0; n < natoms; ++n) {
        float p[4];
        for (int d = 0; d < 3; ++d) p[d] = tk_unit_draw(1700 + d, n) * ext[d] - c * kBinLen;
        p[3] = 2.0f * tk_unit_draw(1703, n) - 1.0f;
        if (p[3] == 0.0f) p[3] = 0.5f;  // a zero charge marks the end of a bin
        const int i = static_cast<int>(std::floor(p[0] * kBinInv)), j = static_cast<int>(std::floor(p[1] * kBinInv)),
                  k = static_cast<int>(std::floor(p[2] * kBinInv));
        if (i < -c || i >= binDim_x - c || j < -c || j >= binDim_y - c || k < -c || k >= binDim_z - c) continue;
        const size_t index = (static_cast<size_t>(k + c) * binDim_y + (j + c)) * binDim_x + (i + c);
        if (count[index] >= kBinDepth) {
            ++extraAtoms;
            continue;
        }
        std::memcpy(&hb[(index * kBinDepth + count[index]) * 4], p, sizeof(p));
        ++count[index];
    }
    bins = static_cast<float*>(backend().deviceAlloc(hb.size() * sizeof(float)));
    backend().upload(bins, hb.data(), hb.size() * sizeof(float), nullptr);
    nbr = static_cast<int*>(backend().deviceAlloc(table.size() * sizeof(int)));
    backend().upload(nbr, table.data(), table.size() * sizeof(int), nullptr);
    regions = static_cast<float*>(backend().deviceAlloc(512ull * gx * gy * gz * sizeof(float)));
    backend().fillZero(regions, 512ull * gx * gy * gz * sizeof(float), nullptr);
    backend().streamSync(nullptr);
    cudaFreeList.push_back(bins);
    cudaFreeList.push_back(nbr);
    cudaFreeList.push_back(regions);
    binZero = bins + ((static_cast<size_t>(c) * binDim_y + c) * binDim_x + c) * kBinDepth * 4;
    zRegionIndex_t = gz - 1;
    launchBlockDim = dim3h(8, 2, 8);
    launchGridDim = dim3h(gx, gy, gz);
    kernelParams = {&binDim_x, &binDim_y, &binZero, &h, &cutoff2, &inv_cutoff2, &regions, &zRegionIndex_t, &nbr, &nbrlen};
    smem = 0;
    initialized = true;
}
void OriCUTCPKernel::loadKernel() {
    kernelFunc = reinterpret_cast<void*>(backend().lookup(funcKey));
    if (!kernelFunc) logger.ERROR("load kernel {" + funcKey + "} failed!");
}
