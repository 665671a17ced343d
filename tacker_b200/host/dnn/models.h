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
    // the task's result on the device after a pass: `resultCount` floats (VGG16 / ResNet-50: the class scores
    // before the softmax, then the probabilities; BERT: the last hidden state)
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
    float* addTo(const float* a, const float* b, int rows, int cols, int act);
    float* layernorm(const float* x, int rows, int cols);
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

Task* createTask(const std::string& taskName);  // "vgg16", "resnet50", "bert" (src/main.cu:227-244)
