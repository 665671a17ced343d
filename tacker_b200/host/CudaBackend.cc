// CudaBackend.cc -- Backend over the CUDA runtime and the C ABI of libtacker_b200.so.
#include <cuda_runtime.h>

#include "Backend.h"
#include "Logger.h"

namespace {

#define CU(call)                                                                                       \
    do {                                                                                               \
        cudaError_t _e = (call);                                                                       \
        if (_e != cudaSuccess)                                                                         \
            throw std::runtime_error(std::string("error: " #call " failed: ") + cudaGetErrorString(_e)); \
    } while (0)

class CudaBackend : public Backend {
public:
    const char* name() const override { return "cuda"; }
    void setDevice(int device) override { CU(cudaSetDevice(device)); }
    int smCount() override {
        int n = 0;
        TK_HOST_CHECK(tk_sm_count(&n));
        return n;
    }
    tk_launch_fn lookup(const std::string& key) override { return tk_lookup(key.c_str()); }
    int query(const std::string& key, tk_kernel_info* info) override { return tk_query(key.c_str(), info); }
    void* deviceAlloc(size_t bytes) override {
        void* p = nullptr;
        CU(cudaMalloc(&p, bytes ? bytes : 16));
        return p;
    }
    void deviceFree(void* p) override {
        if (p) cudaFree(p);
    }
    void* hostAllocPinned(size_t bytes) override {
        void* p = nullptr;
        CU(cudaMallocHost(&p, bytes ? bytes : 16));
        return p;
    }
    void hostFreePinned(void* p) override {
        if (p) cudaFreeHost(p);
    }
    void upload(void* dst, const void* src, size_t bytes, stream_t s) override {
        CU(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(s)));
    }
    void download(void* dst, const void* src, size_t bytes, stream_t s) override {
        CU(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(s)));
    }
    void fillZero(void* dst, size_t bytes, stream_t s) override {
        CU(cudaMemsetAsync(dst, 0, bytes, static_cast<cudaStream_t>(s)));
    }
    stream_t streamCreate() override {
        cudaStream_t s;
        CU(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
        return s;
    }
    void streamSync(stream_t s) override { CU(cudaStreamSynchronize(static_cast<cudaStream_t>(s))); }
    void deviceSync() override { CU(cudaDeviceSynchronize()); }
    void* eventCreate() override {
        cudaEvent_t e;
        CU(cudaEventCreate(&e));
        return e;
    }
    void eventDestroy(void* e) override { cudaEventDestroy(static_cast<cudaEvent_t>(e)); }
    void eventRecord(void* e, stream_t s) override {
        CU(cudaEventRecord(static_cast<cudaEvent_t>(e), static_cast<cudaStream_t>(s)));
    }
    float eventElapsedMs(void* a, void* b) override {
        CU(cudaEventSynchronize(static_cast<cudaEvent_t>(b)));
        float ms = 0.0f;
        CU(cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(a), static_cast<cudaEvent_t>(b)));
        return ms;
    }
    void* graphCapture(stream_t s, const std::function<void()>& body) override {
        cudaStream_t st = static_cast<cudaStream_t>(s);
        if (st == nullptr) return nullptr;  // the legacy default stream cannot be captured
        cudaGraph_t graph = nullptr;
        CU(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        try {
            body();
        } catch (...) {
            cudaStreamEndCapture(st, &graph);
            if (graph) cudaGraphDestroy(graph);
            throw;
        }
        CU(cudaStreamEndCapture(st, &graph));
        cudaGraphExec_t exec = nullptr;
        cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) throw std::runtime_error(std::string("cudaGraphInstantiate failed: ") + cudaGetErrorString(e));
        return exec;
    }
    void graphLaunch(void* graph, stream_t s) override {
        CU(cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph), static_cast<cudaStream_t>(s)));
    }
    void graphDestroy(void* graph) override {
        if (graph) cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph));
    }
    int cpPackAtoms(const float* atoms, int count, float zplane, float* packed, stream_t s) override {
        return tk_cp_pack_atoms(atoms, count, zplane, packed, s);
    }
    int mriqPackKvalues(const float* kx, const float* ky, const float* kz, const float* phiR, const float* phiI,
                        int numK, float* kvals, stream_t s) override {
        return tk_mriq_pack_kvalues(kx, ky, kz, phiR, phiI, numK, kvals, s);
    }
    int mrifPackKvalues(const float* kx, const float* ky, const float* kz, const float* phiR, const float* phiI,
                        const float* dR, const float* dI, int numK, float* kvals, stream_t s) override {
        return tk_mrif_pack_kvalues(kx, ky, kz, phiR, phiI, dR, dI, numK, kvals, s);
    }
    int im2colNhwcHalf(const float* x, int H, int W, int C, int kh, int kw, int pad, int stride, void* A, int M_pad,
                       int K_pad, stream_t s) override {
        return tk_im2col_nhwc_f16(x, H, W, C, kh, kw, pad, stride, A, M_pad, K_pad, s);
    }
    int biasActHalfBordered(const float* x, int ldx, const float* bias, void* out, int H, int W, int C, int act,
                            stream_t s) override {
        return tk_bias_act_f16_bordered(x, ldx, bias, out, H, W, C, act, s);
    }
    int maxpoolHalfBordered(const void* x, int H, int W, int C, void* out, stream_t s) override {
        return tk_maxpool2x2_f16_bordered(x, H, W, C, out, s);
    }
    int unborderHalf(const void* x, int H, int W, int C, void* row, stream_t s) override {
        return tk_unborder_f16(x, H, W, C, row, s);
    }
    int rowsToHalf(const float* x, int rows, int cols, int ld, void* A, int rows_pad, int cols_pad,
                   stream_t s) override {
        return tk_rows_f32_to_f16(x, rows, cols, ld, A, rows_pad, cols_pad, s);
    }
    int biasAct(const float* x, int ldx, const float* bias, float* out, int rows, int cols, int ldo, int act,
                stream_t s) override {
        return tk_bias_act_f32(x, ldx, bias, out, rows, cols, ldo, act, s);
    }
    int maxpool2x2(const float* x, int H, int W, int C, float* out, stream_t s) override {
        return tk_maxpool2x2_nhwc_f32(x, H, W, C, out, s);
    }
    int add(const float* a, const float* b, float* out, long long n, stream_t s) override {
        return tk_add_f32(a, b, out, n, s);
    }
    int softmaxRows(const float* x, float* out, long long rows, int cols, float scale, stream_t s) override {
        return tk_softmax_rows_f32(x, out, rows, cols, scale, s);
    }
    int layernormRows(const float* x, const float* g, const float* b, float* out, long long rows, int cols, float eps,
                      stream_t s) override {
        return tk_layernorm_rows_f32(x, g, b, out, rows, cols, eps, s);
    }
    int addLayernormRows(const float* a, const float* bias, const float* res, const float* g, const float* b, float* out,
                         void* out_half, long long rows, int cols, float eps, stream_t s) override {
        return tk_add_layernorm_rows_f32(a, bias, res, g, b, out, out_half, rows, cols, eps, s);
    }
    int biasActHalf(const float* x, int ldx, const float* bias, float* out, int ldo, void* out_half, int ldh, int rows, int cols,
                    int act, stream_t s) override {
        return tk_bias_act_f32_f16(x, ldx, bias, out, ldo, out_half, ldh, rows, cols, act, s);
    }
    int softmaxRowsHalf(const float* x, void* out_half, long long rows, int cols, float scale, stream_t s) override {
        return tk_softmax_rows_f16(x, out_half, rows, cols, scale, s);
    }
    int mergeHeadsHalf(const float* ctx, int B, int S, int heads, int dh, void* out_half, stream_t s) override {
        return tk_merge_heads_f16(ctx, B, S, heads, dh, out_half, s);
    }
    int splitQkv(const float* x, const float* bias, int ld, int B, int S, int heads, int dh, void* q, void* k, void* vt,
                 stream_t s) override {
        return tk_split_qkv_heads_f16(x, bias, ld, B, S, heads, dh, q, k, vt, s);
    }
    int splitHeads(const float* x, int ld, int col0, int B, int S, int heads, int dh, int transpose, void* out,
                   stream_t s) override {
        return tk_split_heads_f16(x, ld, col0, B, S, heads, dh, transpose, out, s);
    }
    int mergeHeads(const float* ctx, int B, int S, int heads, int dh, float* out, stream_t s) override {
        return tk_merge_heads_f32(ctx, B, S, heads, dh, out, s);
    }
    int tzgemmBatched(const void* A, const void* B, float* C, int M, int N, int K, int batch, float alpha,
                      stream_t s) override {
        return tk_tzgemm_batched(A, B, C, M, N, K, batch, 0, 0, 0, alpha, s);
    }
    unsigned deviceStatus() override {
        unsigned code = 0;
        TK_HOST_CHECK(tk_device_status(&code));
        return code;
    }
};

}  // namespace

Backend* makeCudaBackend() { return new CudaBackend(); }
