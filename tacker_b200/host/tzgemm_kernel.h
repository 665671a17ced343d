// tzgemm_kernel.h -- the GEMM operator the LC layers are mapped to
// (reference: src/tzgemm_kernel.h:30-48 getTZGEMMGridDim, :56-147 OriTZGEMMKernel).
// C[M][N] = alpha * A[M][K] * B[N][K]^T, fp16 inputs, fp32 output; one virtual block = one 64x64 tile.
#pragma once
#include <vector>

#include "Kernel.h"
#include "Logger.h"

// {M_GLOBAL, N_GLOBAL, K_GLOBAL, number of 64x64 tiles}: every dimension rounded down to a multiple of
// 128, never below 128
inline std::vector<int> getTZGEMMGridDim(int m, int n, int k) {
    int out[4];
    tk_tzgemm_dims(m, n, k, out);
    return std::vector<int>(out, out + 4);
}

// Scratch operands shared by every LC GEMM, as in the reference (global ori_wmma_A/B/C,
// src/TaskManager.cu:21-46): sized for the largest layer seen, seeded once, reused by all layers.
struct TZGEMMScratch {
    void* A = nullptr;  // __half [maxA]
    void* B = nullptr;  // __half [maxB]
    float* C = nullptr;
    long long bytesA = 0, bytesB = 0, bytesC = 0;
    // grows the three buffers when a layer needs more; contents are reseeded (uniform [-1, 1))
    void reserve(long long a_bytes, long long b_bytes, long long c_bytes);
    void release();
};
extern TZGEMMScratch tzgemmScratch;

class OriTZGEMMKernel : public Kernel {
public:
    static constexpr float alpha_g = 1.1f;  // src/header/tzgemm_header.h:64
    OriTZGEMMKernel(int id, int m, int n, int k, void* A = nullptr, void* B = nullptr, float* C = nullptr,
                    float alpha = alpha_g)
        : m(m), n(n), k(k), alpha(alpha), A(A), B(B), C(C) {
        this->Id = id;
        this->kernelName = "tzgemm";
        initParams();
    }
    void initParams() override {
        std::vector<int> d = getTZGEMMGridDim(m, n, k);
        M_GLOBAL = d[0];
        N_GLOBAL = d[1];
        K_GLOBAL = d[2];
        ori_blks = d[3];
        launchGridDim = dim3h(ori_blks, 1, 1);
        launchBlockDim = dim3h(192, 1, 1);  // tensor role: TMA, MMA and four epilogue warps
        kernelParams.clear();
        if (!A || !B || !C) {
            // reference behaviour: operate on the shared scratch operands; the list holds the address of
            // the global pointers (as the reference pushes &ori_wmma_A), so a later growth is picked up
            tzgemmScratch.reserve(2ll * M_GLOBAL * K_GLOBAL, 2ll * N_GLOBAL * K_GLOBAL, 4ll * M_GLOBAL * N_GLOBAL);
            kernelParams.push_back(&tzgemmScratch.A);
            kernelParams.push_back(&tzgemmScratch.B);
            kernelParams.push_back(&tzgemmScratch.C);
        } else {
            kernelParams.push_back(&A);
            kernelParams.push_back(&B);
            kernelParams.push_back(&C);
        }
        kernelParams.push_back(&M_GLOBAL);
        kernelParams.push_back(&N_GLOBAL);
        kernelParams.push_back(&K_GLOBAL);
        kernelParams.push_back(&alpha);
        smem = 0;
    }
    std::vector<int> getArgs() override { return std::vector<int>{m, n, k}; }
    int m, n, k;
    int M_GLOBAL, N_GLOBAL, K_GLOBAL;
    int ori_blks;
    float alpha;
    void* A;
    void* B;
    float* C;

protected:
    void executeImpl(stream_t) override { logger.ERROR("should not execute ori tzgemm!"); }  // as the reference
    void loadKernel() override {}
};

// The implicit-GEMM convolution as a host object (no counterpart in the reference, whose convolutions are im2col +
// tzgemm on scratch data, src/include/dnn.h:554-803): 3 x 3, stride 1, padding 1 on zero-bordered NHWC fp16 images.
// Solo argument list of "gptb_tzconv": X, Wt, Y, M, N, K, alpha, bias, H, W, C, act.
class OriTZCONVKernel : public Kernel {
public:
    OriTZCONVKernel(int id, void* X, void* Wt, void* Y, const float* bias, int H, int W, int Cin, int Cout, int act)
        : X(X), Wt(Wt), Y(Y), bias(bias), H(H), W(W), Cin(Cin), act(act) {
        this->Id = id;
        this->kernelName = "tzconv";
        M_GLOBAL = ((H * (W + 2) + 127) / 128) * 128;
        N_GLOBAL = Cout;
        K_GLOBAL = 9 * Cin;
        ori_blks = (M_GLOBAL / 64) * (N_GLOBAL / 64);
        initParams();
    }
    void initParams() override {
        launchGridDim = dim3h(static_cast<unsigned>(ori_blks), 1, 1);
        launchBlockDim = dim3h(192, 1, 1);
        kernelParams = {&X, &Wt, &Y, &M_GLOBAL, &N_GLOBAL, &K_GLOBAL, &alpha, &bias, &H, &W, &Cin, &act};
        smem = 0;
    }
    std::vector<int> getArgs() override { return std::vector<int>{M_GLOBAL, N_GLOBAL, K_GLOBAL}; }
    void* X;
    void* Wt;
    void* Y;
    const float* bias;
    int H, W, Cin, act;
    int M_GLOBAL, N_GLOBAL, K_GLOBAL, ori_blks;
    float alpha = 1.0f;

protected:
    void executeImpl(stream_t) override { logger.ERROR("should not execute ori tzconv!"); }
    void loadKernel() override {}
};
