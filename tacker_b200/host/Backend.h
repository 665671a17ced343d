// Backend.h -- the only door between the host runtime and the GPU.
// The runtime (Kernel classes, Creator, Task, TaskManager, DNN tasks) is plain C++ and talks to the
// device through this interface: CudaBackend (CudaBackend.cc) forwards to the CUDA runtime and to the
// C ABI of libtacker_b200.so; the host self-test links a recording double instead, so the marshalling
// and the scheduling rules can be checked on a machine without a GPU.  There is no CPU compute path.
#pragma once
#include <cstddef>
#include <functional>
#include <string>

#include "tacker_b200.h"
#include "util.h"

class Backend {
public:
    virtual ~Backend() {}
    virtual const char* name() const = 0;
    virtual void setDevice(int device) = 0;
    virtual int smCount() = 0;
    virtual tk_launch_fn lookup(const std::string& key) = 0;  // fmap[key]
    virtual int query(const std::string& key, tk_kernel_info* info) = 0;
    // memory
    virtual void* deviceAlloc(size_t bytes) = 0;
    virtual void deviceFree(void* p) = 0;
    virtual void* hostAllocPinned(size_t bytes) = 0;
    virtual void hostFreePinned(void* p) = 0;
    virtual void upload(void* dst, const void* src, size_t bytes, stream_t s) = 0;
    virtual void download(void* dst, const void* src, size_t bytes, stream_t s) = 0;
    virtual void fillZero(void* dst, size_t bytes, stream_t s) = 0;
    // streams, events, time
    virtual stream_t streamCreate() = 0;
    virtual void streamSync(stream_t s) = 0;
    virtual void deviceSync() = 0;
    virtual void* eventCreate() = 0;
    virtual void eventDestroy(void* e) = 0;
    virtual void eventRecord(void* e, stream_t s) = 0;
    virtual float eventElapsedMs(void* start, void* stop) = 0;  // waits for `stop`
    // Records everything `body` enqueues on `s` into a CUDA graph and returns an executable handle (nullptr when
    // the backend cannot capture: the caller then just runs `body`).  Launch-bound kernel sequences -- a whole
    // inference of the LC task, a chunk of the BE task -- are replayed with one call instead of dozens.
    virtual void* graphCapture(stream_t s, const std::function<void()>& body) = 0;
    virtual void graphLaunch(void* graph, stream_t s) = 0;
    virtual void graphDestroy(void* graph) = 0;
    // input preparation and LC-layer helpers of the library
    virtual int cpPackAtoms(const float* atoms, int count, float zplane, float* packed, stream_t s) = 0;
    virtual int mriqPackKvalues(const float* kx, const float* ky, const float* kz, const float* phiR,
                                const float* phiI, int numK, float* kvals, stream_t s) = 0;
    virtual int mrifPackKvalues(const float* kx, const float* ky, const float* kz, const float* phiR,
                                const float* phiI, const float* dR, const float* dI, int numK, float* kvals,
                                stream_t s) = 0;
    virtual int im2colNhwcHalf(const float* x, int H, int W, int C, int kh, int kw, int pad, int stride, void* A,
                               int M_pad, int K_pad, stream_t s) = 0;
    virtual int biasActHalfBordered(const float* x, int ldx, const float* bias, void* out, int H, int W, int C, int act,
                                    stream_t s) = 0;
    virtual int maxpoolHalfBordered(const void* x, int H, int W, int C, void* out, stream_t s) = 0;
    virtual int unborderHalf(const void* x, int H, int W, int C, void* row, stream_t s) = 0;
    virtual int rowsToHalf(const float* x, int rows, int cols, int ld, void* A, int rows_pad, int cols_pad,
                           stream_t s) = 0;
    virtual int biasAct(const float* x, int ldx, const float* bias, float* out, int rows, int cols, int ldo, int act,
                        stream_t s) = 0;
    virtual int maxpool2x2(const float* x, int H, int W, int C, float* out, stream_t s) = 0;
    virtual int add(const float* a, const float* b, float* out, long long n, stream_t s) = 0;
    virtual int softmaxRows(const float* x, float* out, long long rows, int cols, float scale, stream_t s) = 0;
    virtual int layernormRows(const float* x, const float* g, const float* b, float* out, long long rows, int cols,
                              float eps, stream_t s) = 0;
    // out = layernorm(a + res): rows of 128 .. 1024 columns (a multiple of 128)
    // (res may be null; out_half, if given, also receives the result as fp16 [rows][cols])
    // bias [cols], if given, is added to a first (the bias of the product that made a)
    virtual int addLayernormRows(const float* a, const float* bias, const float* res, const float* g, const float* b, float* out,
                                 void* out_half, long long rows, int cols, float eps, stream_t s) = 0;
    // producers that write the fp16 operand of the product that follows (see the library header)
    virtual int biasActHalf(const float* x, int ldx, const float* bias, float* out, int ldo, void* out_half, int ldh, int rows,
                            int cols, int act, stream_t s) = 0;
    virtual int softmaxRowsHalf(const float* x, void* out_half, long long rows, int cols, float scale, stream_t s) = 0;
    virtual int mergeHeadsHalf(const float* ctx, int B, int S, int heads, int dh, void* out_half, stream_t s) = 0;
    virtual int splitQkv(const float* x, const float* bias, int ld, int B, int S, int heads, int dh, void* q, void* k, void* vt,
                         stream_t s) = 0;
    virtual int splitHeads(const float* x, int ld, int col0, int B, int S, int heads, int dh, int transpose, void* out,
                           stream_t s) = 0;
    virtual int mergeHeads(const float* ctx, int B, int S, int heads, int dh, float* out, stream_t s) = 0;
    virtual int tzgemmBatched(const void* A, const void* B, float* C, int M, int N, int K, int batch, float alpha,
                              stream_t s) = 0;
    virtual unsigned deviceStatus() = 0;
};

Backend& backend();
void setBackend(Backend* b);  // not owned
Backend* makeCudaBackend();   // defined in CudaBackend.cc (needs the CUDA runtime and the library)
