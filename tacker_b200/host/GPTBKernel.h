// GPTBKernel.h -- a solo kernel run as persistent thread blocks (reference: src/GPTBKernel.h:12-124):
// the solo argument list, six ints with the original launch geometry, and at launch time
// start, step, end, thread_base.
#pragma once
#include "Kernel.h"
#include "Logger.h"

class GPTBKernel : public Kernel {
public:
    GPTBKernel(int id, const std::string kernelName, const std::string funcKey, Kernel* kernel, dim3h gridDim,
               dim3h blockDim, int ptb_start_block_pos, int ptb_end_block_pos)
        : kernel_(kernel) {
        Id = id;
        this->kernelName = kernelName;
        this->funcKey = funcKey;
        launchGridDim = gridDim;     // persistent CTAs
        launchBlockDim = blockDim;
        smem = kernel->smem;
        const dim3h& og = kernel->launchGridDim;   // geometry of the launch being emulated
        const dim3h& ob = kernel->launchBlockDim;
        gptbParams = GPTBParams{static_cast<int>(og.x), static_cast<int>(og.y), static_cast<int>(og.z),
                                static_cast<int>(ob.x), static_cast<int>(ob.y), static_cast<int>(ob.z),
                                ptb_start_block_pos, static_cast<int>(gridDim.x * gridDim.y * gridDim.z),
                                ptb_end_block_pos};
        kernelParams = kernel->kernelParams;       // the solo argument list comes first
        loadKernel();
        initParams();
    }
    ~GPTBKernel() override {}

    GPTBParams gptbParams;
    Kernel* kernel_;

    void initParams() override {
        kernelParams.push_back(&gptbParams.grid_dimension_x);
        kernelParams.push_back(&gptbParams.grid_dimension_y);
        kernelParams.push_back(&gptbParams.grid_dimension_z);
        kernelParams.push_back(&gptbParams.block_dimension_x);
        kernelParams.push_back(&gptbParams.block_dimension_y);
        kernelParams.push_back(&gptbParams.block_dimension_z);
        // start/step/end are pushed at launch so that MixKernel can reuse the list up to here
    }
    void loadKernel() override {
        kernelFunc = reinterpret_cast<void*>(backend().lookup(funcKey));
        if (!kernelFunc) logger.ERROR("load kernel {" + funcKey + "} failed!");
    }
    std::vector<int> getArgs() override { return std::vector<int>(); }

protected:
    void executeImpl(stream_t stream) override {
        gptbParams.ptb_iter_block_step = launchGridDim.x * launchGridDim.y * launchGridDim.z;
        int thread_base = 0;  // a solo persistent kernel owns the whole CTA
        std::vector<void*> p(kernelParams);
        p.push_back(&gptbParams.ptb_start_block_pos);
        p.push_back(&gptbParams.ptb_iter_block_step);
        p.push_back(&gptbParams.ptb_end_block_pos);
        p.push_back(&thread_base);
        launch(p, stream);
    }
};
