// Kernel.h -- abstract operator (reference: src/Kernel.h:12-59): launch geometry, argument list as a
// vector of pointers to host scalars, the function to launch, `mixable` and getArgs() for the scheduler.
// kernelFunc holds a launcher of the C ABI (tk_launch_fn) where the reference holds a __global__ symbol.
#pragma once
#include <string>
#include <utility>
#include <vector>

#include "Backend.h"
#include "util.h"

enum lmode { DRIVER_LAUNCH = 0, RUNTIME_LAUNCH };

class Kernel {
public:
    template <typename... Args>
    void execute(Args&&... args) {
        executeImpl(std::forward<Args>(args)...);
    }
    virtual void initParams() = 0;
    virtual void loadKernel() = 0;
    virtual ~Kernel() = default;

    int getKernelId() { return Id; }
    std::string& getKernelName() { return kernelName; }
    virtual std::vector<int> getArgs() = 0;

    int Id = 0;
    std::string kernelName;
    std::string moduleName;
    std::string funcKey;
    unsigned int smem = 0;
    std::vector<void*> kernelParams;
    std::vector<void*> cudaFreeList;
    dim3h launchGridDim;
    dim3h launchBlockDim;
    lmode launchMode = RUNTIME_LAUNCH;
    void* kernelFunc = nullptr;  // tk_launch_fn
    unsigned mixable = 0;        // 0 = never fused, 1 = GEMM (getArgs: m, n, k), 2 = convolution (14 ints)
    bool initialized = false;
    // Stream on which a repeated initParams() queues its device work (re-zeroing of accumulated outputs): set it to
    // the stream the kernel is launched on, so that the reset is ordered against those launches.  The reference's
    // blocking streams gave that ordering implicitly; the streams of this runtime do not synchronise with the
    // null stream.
    stream_t initStream = nullptr;

protected:
    virtual void executeImpl(stream_t stream) = 0;
    // cudaLaunchKernel(kernelFunc, grid, block, params, smem, stream) through the C ABI
    void launch(std::vector<void*>& params, stream_t stream) {
        const unsigned g[3] = {launchGridDim.x, launchGridDim.y, launchGridDim.z};
        const unsigned b[3] = {launchBlockDim.x, launchBlockDim.y, launchBlockDim.z};
        const int rc = reinterpret_cast<tk_launch_fn>(kernelFunc)(params.data(), static_cast<int>(params.size()), g, b,
                                                                 smem, stream);
        if (rc != 0)
            throw std::runtime_error("launch of {" + funcKey + "} failed: " + tk_status_string(rc) + " " +
                                     tk_last_error());
    }
};

struct GPTBParams {
    int grid_dimension_x, grid_dimension_y, grid_dimension_z;
    int block_dimension_x, block_dimension_y, block_dimension_z;
    int ptb_start_block_pos, ptb_iter_block_step, ptb_end_block_pos;
};
