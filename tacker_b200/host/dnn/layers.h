// dnn/layers.h -- the layer kernels the model tasks are made of.
// The reference generates one Kernel subclass per graph node (src/dnn/<model>/*_kernel_class.h) and routes
// convolutions and dense layers to tzgemm through mycudnnConvolutionForward / mycublasSgemm
// (src/include/dnn.h:554-880): convolutions carry mixable = 2 and their 14 cuDNN ints, dense layers
// mixable = 1 and (m, n, k); everything else is mixable = 0.  The same contract holds here, with the nodes
// written by hand and kept on real buffers: activations flow through the task's arena (fp32, NHWC).
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "../GPTBKernel.h"
#include "../tzgemm_kernel.h"

// Device memory of one model instance: activations, fp16 GEMM operands, weights.
struct DnnArena {
    ~DnnArena();
    float* act(size_t floats);              // a new fp32 activation buffer
    void* half(size_t halves);              // a new fp16 buffer
    void* weightsHalf(size_t halves, uint64_t seed, float scale);  // seeded fp16 weights, uniform * scale
    float* weightsF32(size_t n, uint64_t seed, float lo, float hi);
    size_t bytes = 0;
    std::vector<void*> owned;
};

inline int roundUp(int v, int m) { return ((v + m - 1) / m) * m; }
uint16_t dnn_half_bits(float f);  // binary32 -> binary16 bits, round to nearest even

// Common part of the two tzgemm-backed layers: operands, the persistent GEMM kernel over all tiles and
// what the scheduler needs to fuse it with a best-effort kernel.
class TzLayer : public Kernel {
public:
    // GEMM over the padded operands: M_pad x N_pad x K_pad, alpha = 1
    void buildGemm(int id);
    virtual void prepare(stream_t stream) = 0;  // fill the fp16 A operand from the layer input
    GPTBKernel* gemm() { return gptb.get(); }
    int tiles() const { return tiles_; }
    // key prefix of the fused kernels this layer's tensor role belongs to: "tzgemm_" or "tzconv_"
    const char* fusedPrefix() const { return implicit ? "tzconv_" : "tzgemm_"; }
    bool implicit = false;
    int M = 0, N = 0, K = 0, M_pad = 0, N_pad = 0, K_pad = 0;
    void* A = nullptr;   // fp16 [M_pad][K_pad]
    void* B = nullptr;   // fp16 [N_pad][K_pad] weights
    float* C = nullptr;  // fp32 [M_pad][N_pad]
    void initParams() override {}
    void loadKernel() override {}

protected:
    void executeImpl(stream_t stream) override {  // solo LC path: operand preparation + tzgemm alone
        prepare(stream);
        if (skinny) {
            backend().fillZero(C, static_cast<size_t>(M_pad) * N_pad * sizeof(float), stream);
            gptb_acc->execute(stream);
        } else {
            gptb->execute(stream);
        }
    }
    bool skinny = false;
    int tiles_ = 0;
    std::unique_ptr<OriTZGEMMKernel> ori;
    std::unique_ptr<OriTZCONVKernel> ori_conv;
    std::unique_ptr<GPTBKernel> gptb, gptb_acc;
};

// 2-D convolution, NHWC, square kernel (mixable = 2; getArgs = the 14 ints of cudnnConvolutionForward in
// the order get_mnk_from_cudnn_args reads them, src/TaskManager.cu:92-123)
class ConvKernel : public TzLayer {
public:
    ConvKernel(int id, const std::string& name, DnnArena& arena, const float* input, int H, int W, int Cin, int Cout,
               int ksize, int pad, int stride, uint64_t seed);
    std::vector<int> getArgs() override;
    void prepare(stream_t stream) override;
    const float* input;
    int H, W, Cin, Cout, ksize, pad, stride, OH, OW;
};

// 3 x 3 convolution, stride 1, padding 1, as one implicit-GEMM kernel with bias and activation in its epilogue:
// zero-bordered NHWC fp16 image in, zero-bordered NHWC fp16 image out, no operand preparation (same mixable /
// getArgs contract as ConvKernel)
class ConvImplicitKernel : public TzLayer {
public:
    ConvImplicitKernel(int id, const std::string& name, DnnArena& arena, void* x_bordered, int H, int W, int Cin,
                       int Cout, int act, uint64_t seed, const float* bias, void* y_bordered);
    std::vector<int> getArgs() override;
    void prepare(stream_t) override {}
    int H, W, Cin, Cout;
};

// dense layer y = x W^T on `rows` rows (mixable = 1; getArgs = m, n, k)
class GemmKernel : public TzLayer {
public:
    GemmKernel(int id, const std::string& name, DnnArena& arena, const float* input, int rows, int in_features,
               int out_features, uint64_t seed);
    std::vector<int> getArgs() override { return std::vector<int>{M, N, K}; }
    void prepare(stream_t stream) override;
    const float* input;
    bool a_ready = false;  // the producer of `input` writes the fp16 operand A itself: prepare() has nothing to do
    // alternative input: a bordered fp16 image [(bH + 2)][(bW + 2)][bC] whose interior, flattened, is the single row
    const void* bordered = nullptr;
    int bH = 0, bW = 0, bC = 0;
};

// everything that is not a GEMM (mixable = 0): one call into the library
class OpKernel : public Kernel {
public:
    enum Op { BiasAct, MaxPool, Add, SoftmaxRows, LayerNorm, SplitHeads, MergeHeads, BatchedGemm, RowsToHalf,
              BiasActHalfBordered, MaxPoolHalfBordered, SplitQkv };
    OpKernel(int id, const std::string& name, Op op) : op(op) {
        Id = id;
        kernelName = name;
        mixable = 0;
    }
    void initParams() override {}
    void loadKernel() override {}
    std::vector<int> getArgs() override { return std::vector<int>(); }
    Op op;
    // operands (meaning depends on op; see layers.cc)
    const float* a = nullptr;
    const float* b = nullptr;
    const float* c = nullptr;
    const float* res = nullptr;  // LayerNorm: second operand added to `a` before the normalisation (or null)
    const float* bias = nullptr; // LayerNorm, SplitQkv: bias of the product whose raw output `a` is (added first), or null
    bool absorbed = false;       // the node's work is done by its consumer: executing it launches nothing
    float* out = nullptr;
    void* hout = nullptr;   // fp16 output; for BiasAct, SoftmaxRows, LayerNorm, MergeHeads: the operand of the next product
    void* hout2 = nullptr;  // SplitQkv: key heads
    void* hout3 = nullptr;  // SplitQkv: value heads, transposed
    const void* ha = nullptr;
    const void* hb = nullptr;
    int i0 = 0, i1 = 0, i2 = 0, i3 = 0, i4 = 0, i5 = 0, i6 = 0;
    float f0 = 0.0f;

protected:
    void executeImpl(stream_t stream) override;
};
