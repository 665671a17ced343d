#include "Creator.h"

#include <map>
#include <memory>

#include "json.h"

StencilProblem creatorStencilProblem;
CPProblem creatorCPProblem;
MRIQProblem creatorMRIQProblem;
MRIFProblem creatorMRIFProblem;
SGEMMProblem creatorSGEMMProblem;
LBMProblem creatorLBMProblem;
FFTProblem creatorFFTProblem;
CUTCPProblem creatorCUTCPProblem;

namespace {
std::map<std::string, GPTBKernel*> kernelMap;
std::map<std::string, MixKernel*> mixKernelMap;
std::vector<Kernel*> owned;

// persistent grid: SM count x CTAs per SM, CUDA-core threads per CTA; JSON overrides
// ("<name>": {"gridsize": .., "blocksize": ..}) where the model file carries them
void geometry(const std::string& name, int dflt_per_sm, int dflt_block, dim3h* grid, dim3h* block) {
    int per_sm = get_kernel_info(name, "gridsize");
    int threads = get_kernel_info(name, "blocksize");
    if (per_sm == JSON_NOT_FOUND || per_sm <= 0) per_sm = dflt_per_sm;
    if (threads == JSON_NOT_FOUND || threads <= 0) threads = dflt_block;
    *grid = dim3h(static_cast<unsigned>(backend().smCount() * per_sm), 1, 1);
    *block = dim3h(static_cast<unsigned>(threads), 1, 1);
}
}  // namespace

GPTBKernel* createKernel(const std::string& name) {
    auto it = kernelMap.find(name);
    if (it != kernelMap.end()) return it->second;
    Kernel* ori = nullptr;
    int id = 0;
    dim3h grid, block;
    if (name == "cp") {
        ori = new OriCPKernel(id = 10, creatorCPProblem);
        geometry(name, 2, 512, &grid, &block);
    } else if (name == "mriq") {
        ori = new OriMRIQKernel(id = 18, creatorMRIQProblem);
        geometry(name, 2, 512, &grid, &block);
    } else if (name == "mrif") {  // id as in src/Creator.cu:109-121
        ori = new OriMRIFKernel(id = 17, creatorMRIFProblem);
        geometry(name, 2, 512, &grid, &block);
    } else if (name == "stencil") {
        ori = new OriSTENCILKernel(id = 20, creatorStencilProblem);
        geometry(name, 2, 256, &grid, &block);
    } else if (name == "cutcp") {  // ids as in src/Creator.cu:53-178
        ori = new OriCUTCPKernel(id = 11, creatorCUTCPProblem);
        geometry(name, 2, 512, &grid, &block);
    } else if (name == "fft") {
        ori = new OriFFTKernel(id = 12, creatorFFTProblem);
        geometry(name, 2, 512, &grid, &block);
    } else if (name == "lbm") {
        ori = new OriLBMKernel(id = 16, creatorLBMProblem);
        geometry(name, 2, 512, &grid, &block);
    } else if (name == "sgemm") {
        ori = new OriSGEMMKernel(id = 19, creatorSGEMMProblem);
        geometry(name, 2, 256, &grid, &block);
    } else {
        logger.ERROR("createKernel: unknown kernel {" + name + "}");
    }
    owned.push_back(ori);
    const int blocks = static_cast<int>(ori->launchGridDim.x * ori->launchGridDim.y * ori->launchGridDim.z);
    GPTBKernel* k = new GPTBKernel(id, name, "gptb_" + name, ori, grid, block, 0, blocks);
    kernelMap[name] = k;
    return k;
}

MixKernel* createMixKernel(const std::string& name, int m, int n, int k) {
    const std::string prefix = "tzgemm_";
    if (name.compare(0, prefix.size(), prefix) != 0) logger.ERROR("createMixKernel: unknown pair {" + name + "}");
    const std::string cd = name.substr(prefix.size());
    if (m <= 0 || n <= 0 || k <= 0) {  // headline GEMM of each pair
        if (cd == "stencil") m = 4096, n = 4096, k = 1024;
        else if (cd == "cp") m = 2048, n = 2048, k = 2048;
        else if (cd == "mriq" || cd == "mrif" || cd == "sgemm" || cd == "lbm" || cd == "fft" || cd == "cutcp")
            m = 4096, n = 4096, k = 2048;
        else logger.ERROR("createMixKernel: unknown pair {" + name + "}");
    }
    const std::string key = name + ":" + std::to_string(m) + "x" + std::to_string(n) + "x" + std::to_string(k);
    auto it = mixKernelMap.find(key);
    if (it != mixKernelMap.end()) return it->second;
    GPTBKernel* cdk = createKernel(cd);
    OriTZGEMMKernel* ori = new OriTZGEMMKernel(0, m, n, k);
    owned.push_back(ori);
    const unsigned sms = static_cast<unsigned>(backend().smCount());
    GPTBKernel* tz = new GPTBKernel(1, "tzgemm", "gptb_tzgemm", ori, dim3h(sms, 1, 1), dim3h(192, 1, 1), 0, ori->ori_blks);
    owned.push_back(tz);
    dim3h grid, block;
    geometry(name, 1, 192 + 384, &grid, &block);
    MixKernel* mk = new MixKernel(static_cast<int>(mixKernelMap.size()), name, cdk, tz, grid, block,
                                  cdk->gptbParams.ptb_start_block_pos, cdk->gptbParams.ptb_end_block_pos, 0,
                                  ori->ori_blks);
    mixKernelMap[key] = mk;
    return mk;
}

void destroyCreatedKernels() {
    for (auto& m : mixKernelMap) delete m.second;
    for (auto& k : kernelMap) delete k.second;
    for (auto* o : owned) delete o;
    mixKernelMap.clear();
    kernelMap.clear();
    owned.clear();
}
