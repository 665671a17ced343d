// dnn/models.h -- the model tasks: ordered kernel lists built from layer tables.
// The reference generates these from NNFusion output (src/dnn/vgg16/vgg16.h:5-25, vgg16.cu:11-32,
// src/dnn/bert/bert.cu:11-52, src/dnn/resnet50/resnet50.cu); weights are random (He / uniform), inputs
// synthetic, so that only shapes and timing matter -- as in the reference, whose layers run on scratch data.
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "../Task.h"
#include "layers.h"

class DnnTask : public Task {
public:
    DnnTask(int id, const std::string& name) : Task(id, name) {}
    ~DnnTask() override;
    void initExecution() override;  // upload the input of one query
    // the task's result on the device after a pass: `resultCount` floats (VGG16: the class scores before the
    // softmax, then the probabilities; ResNet-50: the class scores; BERT: the last layer's hidden states)
    const float* result = nullptr;
    size_t resultCount = 0;
    std::vector<float> downloadResult(stream_t stream);
    size_t numMixable() const;
    double gemmFlops() const;       // 2*M*N*K summed over the tzgemm-backed layers (unpadded shapes)
    DnnArena arena;

protected:
    Kernel* keep(Kernel* k) {
        owned.emplace_back(k);
        addKernel(k);
        return k;
    }
    float* input = nullptr;         // device
    std::vector<float> hostInput;
    std::vector<std::unique_ptr<Kernel>> owned;
    int nextId = 0;
    // helpers used by the builders; each returns the output activation
    float* conv(const float* x, int H, int W, int Cin, int Cout, int k, int pad, int stride, int act, int* OH,
                int* OW);
    float* dense(const float* x, int rows, int in, int out, int act, float* y = nullptr);  // y: where the output goes
    float* pool(const float* x, int H, int W, int C);
    // the bordered fp16 activation path (3 x 3 / stride 1 / padding 1 convolutions as implicit GEMMs):
    void* borderedImage(int H, int W, int C);  // zeroed [(H + 2)][(W + 2)][C] fp16
    // first layer (few input channels): explicit im2col + tzgemm, then bias + activation into a bordered image
    void* convToBordered(const float* x, int H, int W, int Cin, int Cout, int act);
    void* convBordered(void* x, int H, int W, int Cin, int Cout, int act);  // implicit GEMM, one kernel
    void* poolBordered(void* x, int H, int W, int C);
    // dense layer on the flattened interior of a bordered image (one row)
    float* denseFromBordered(void* x, int H, int W, int C, int out, int act);
    // what the last conv / dense helper created, for builders that replace the seeded constants by loaded ones
    TzLayer* lastLayer = nullptr;
    float* lastBias = nullptr;
    // the last bias + activation or normalisation node created (dense(), denseParts(), layernorm(), addLayernorm())
    OpKernel* lastOp = nullptr;
    // Lets `producer` write the fp16 operand of `consumer` directly (no conversion pass in between).  Possible when the
    // operand needs no padding: rows a multiple of 128, cols a multiple of 64.  Returns whether it was done.
    bool feedHalf(OpKernel* producer, GemmKernel* consumer, int rows, int cols);
    float* addTo(const float* a, const float* b, int rows, int cols, int act);
    float* layernorm(const float* x, int rows, int cols);
    // layernorm(a + b) as one kernel; numbered and seeded like addTo(a, b, ..., 0) followed by layernorm()
    float* addLayernorm(const float* a, const float* b, int rows, int cols);
    // `parts` dense layers of the same shape on the same input as ONE GEMM of parts * out columns (weights and biases
    // of the parts side by side); numbered and seeded like `parts` consecutive dense() calls.  Returns the
    // [rows][parts * out] output; part i is its columns i * out ...
    float* denseParts(const float* x, int rows, int in, int out, int parts, int act);
};

// VGG16, batch 1, 224 x 224 x 3: 13 conv3x3 + 3 FC
class VGG16 : public DnnTask {
public:
    explicit VGG16(int numClasses = 1000);
};

// ResNet-50, batch 1, 224 x 224 x 3: bottleneck stages [3, 4, 6, 3]
class Resnet50 : public DnnTask {
public:
    explicit Resnet50(int numClasses = 1000);
};

// BERT-base encoder: 12 layers, hidden 768, 12 heads, FFN 3072, batch 8, sequence 128
class Bert : public DnnTask {
public:
    explicit Bert(int layers = 12, int batch = 8, int seq = 128);
    int batch, seq;
};

// A model read from a description file instead of being compiled in -- the role the reference gives to the classes
// src/nnf/gen_code.py generates from NNFusion output (src/nnf/gen_code.py:69-246) and to the Constant_<n>_0.bin files
// those classes read (src/dnn/vgg16/vgg16_kernel_class.h:378-391).  JSON:
//   {"name": "..", "config": "vgg16",                       model file whose kernel tables the scheduler uses
//    "input": {"h": 32, "w": 32, "c": 3, "seed": 42, "file": "input.bin"},
//    "constants": "Constant",                               directory of the .bin files, relative to the description
//    "layers": [{"op": "conv3x3", "out": 64, "act": "relu", "weight": "Constant_1_0.bin", "bias": "Constant_2_0.bin"},
//               {"op": "maxpool"}, {"op": "dense", "out": 10, "act": "none", ...}, {"op": "softmax"}]}
// Constants are raw little-endian fp32 in NNFusion's layouts: convolution filters [3][3][Cin][Cout], dense weights
// [in][out], biases [out]; a layer without files keeps its seeded constants.  Convolutions are 3 x 3 / stride 1 /
// padding 1; after the first one the channel counts must be multiples of 64 (the implicit-GEMM form).
class GraphTask : public DnnTask {
public:
    explicit GraphTask(const std::string& descriptionFile);
    std::string config = "vgg16";
    int loadedConstants = 0;  // files read

private:
    std::vector<float> readConstant(const std::string& file, size_t count);
    void loadConv(const std::string& wfile, const std::string& bfile, int Cin, int Cout);
    void loadDense(const std::string& wfile, const std::string& bfile, int in, int out);
    std::string constantDir;
};

// "vgg16", "resnet50", "bert" (src/main.cu:227-244), or the path of a model description (*.json)
Task* createTask(const std::string& taskName);
