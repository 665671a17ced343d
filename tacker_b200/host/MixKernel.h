// MixKernel.h -- one launch that runs two persistent kernels in disjoint thread ranges of the same CTAs
// (reference: src/MixKernel.h:9-115).  Arguments = kernel1's list + {start, step, end} followed by
// kernel2's list + {start, step, end}; for the tzgemm_<cd> kernels kernel1 is the CUDA-core kernel and
// kernel2 the tzgemm (src/TaskManager.cu:253-264).
#pragma once
#include "GPTBKernel.h"

class MixKernel : public Kernel {
public:
    MixKernel(int id, const std::string& funcKey, GPTBKernel* kernel1, GPTBKernel* kernel2, dim3h gridDim,
              dim3h blockDim, int ptb_start_block_pos1, int ptb_end_block_pos1, int ptb_start_block_pos2,
              int ptb_end_block_pos2)
        : kernel1(kernel1), kernel2(kernel2) {
        this->Id = id;
        this->funcKey = funcKey;
        this->kernelName = funcKey;
        this->launchGridDim = gridDim;
        this->launchBlockDim = blockDim;
        this->smem = 0;
        kernel1_iter_block_step = gridDim.x * gridDim.y * gridDim.z;
        kernel2_iter_block_step = kernel1_iter_block_step;
        kernel1_start_block_pos = ptb_start_block_pos1;
        kernel1_end_block_pos = ptb_end_block_pos1;
        kernel2_start_block_pos = ptb_start_block_pos2;
        kernel2_end_block_pos = ptb_end_block_pos2;
        initParams();
        loadKernel();
    }
    ~MixKernel() override {}

    int kernel1_start_block_pos, kernel1_iter_block_step, kernel1_end_block_pos;
    int kernel2_start_block_pos, kernel2_iter_block_step, kernel2_end_block_pos;

    // move the two ranges without rebuilding the object (the scheduler reuses one MixKernel per layer)
    void setRanges(int s1, int e1, int s2, int e2) {
        kernel1_start_block_pos = s1;
        kernel1_end_block_pos = e1;
        kernel2_start_block_pos = s2;
        kernel2_end_block_pos = e2;
    }

    void initParams() override {
        kernelParams.clear();
        for (auto& param : kernel1->kernelParams) kernelParams.push_back(param);
        kernelParams.push_back(&kernel1_start_block_pos);
        kernelParams.push_back(&kernel1_iter_block_step);
        kernelParams.push_back(&kernel1_end_block_pos);
        for (auto& param : kernel2->kernelParams) kernelParams.push_back(param);
        kernelParams.push_back(&kernel2_start_block_pos);
        kernelParams.push_back(&kernel2_iter_block_step);
        kernelParams.push_back(&kernel2_end_block_pos);
    }
    void loadKernel() override {
        kernelFunc = reinterpret_cast<void*>(backend().lookup(funcKey));
        if (!kernelFunc) logger.ERROR("load kernel {" + funcKey + "} failed!");
    }
    std::vector<int> getArgs() override { return std::vector<int>(); }
    // Launch through a launcher of another module (a fused kernel emitted by the generator and registered with the
    // ModuleCenter) instead of the library's own kernel of this key; same argument list.
    void useFunction(tk_launch_fn fn, const std::string& module) {
        kernelFunc = reinterpret_cast<void*>(fn);
        moduleName = module;
    }

protected:
    void executeImpl(stream_t stream) override { launch(kernelParams, stream); }

private:
    GPTBKernel* kernel1;
    GPTBKernel* kernel2;
};
