#include "layers.h"

#include <cmath>
#include <cstdint>

namespace {
uint16_t half_bits(float f) {  // round to nearest even; inputs are small normal numbers or zero
    uint32_t x;
    __builtin_memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u, absx = x & 0x7fffffffu;
    if (absx < 0x38800000u) {
        if (absx < 0x33000000u) return static_cast<uint16_t>(sign);
        const uint32_t e = absx >> 23, m = (absx & 0x7fffffu) | 0x800000u, shift = 126u - e;
        uint32_t h = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1u), mid = 1u << (shift - 1u);
        if (rem > mid || (rem == mid && (h & 1u))) ++h;
        return static_cast<uint16_t>(sign | h);
    }
    uint32_t h = (((absx >> 23) - 112u) << 10) | ((absx & 0x7fffffu) >> 13);
    const uint32_t rem = absx & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
    return static_cast<uint16_t>(sign | h);
}
}  // namespace

uint16_t dnn_half_bits(float f) { return half_bits(f); }

DnnArena::~DnnArena() {
    for (void* p : owned) backend().deviceFree(p);
}

float* DnnArena::act(size_t floats) {
    void* p = backend().deviceAlloc(floats * sizeof(float));
    backend().fillZero(p, floats * sizeof(float), nullptr);
    backend().streamSync(nullptr);  // set-up time: landed before any launch on another stream can read it
    owned.push_back(p);
    bytes += floats * sizeof(float);
    return static_cast<float*>(p);
}

void* DnnArena::half(size_t halves) {
    void* p = backend().deviceAlloc(halves * 2);
    backend().fillZero(p, halves * 2, nullptr);
    backend().streamSync(nullptr);
    owned.push_back(p);
    bytes += halves * 2;
    return p;
}

void* DnnArena::weightsHalf(size_t halves, uint64_t seed, float scale) {
    std::vector<uint16_t> h(halves);
    for (size_t i = 0; i < halves; ++i) h[i] = half_bits((tk_unit_draw(seed, i) * 2.0f - 1.0f) * scale);
    void* p = backend().deviceAlloc(halves * 2);
    backend().upload(p, h.data(), halves * 2, nullptr);
    backend().streamSync(nullptr);
    owned.push_back(p);
    bytes += halves * 2;
    return p;
}

float* DnnArena::weightsF32(size_t n, uint64_t seed, float lo, float hi) {
    std::vector<float> h(n);
    for (size_t i = 0; i < n; ++i) h[i] = lo + tk_unit_draw(seed, i) * (hi - lo);
    void* p = backend().deviceAlloc(n * sizeof(float));
    backend().upload(p, h.data(), n * sizeof(float), nullptr);
    backend().streamSync(nullptr);
    owned.push_back(p);
    bytes += n * sizeof(float);
    return static_cast<float*>(p);
}

void TzLayer::buildGemm(int id) {
    ori.reset(new OriTZGEMMKernel(id, M_pad, N_pad, K_pad, A, B, C, 1.0f));
    // OriTZGEMMKernel rounds down to multiples of 128; the operands here are padded to 128 / 64 / 64, so N and
    // K are re-stated exactly (the kernel itself takes N % 64 == 0 and K % 64 == 0)
    ori->N_GLOBAL = N_pad;
    ori->K_GLOBAL = K_pad;
    ori->M_GLOBAL = M_pad;
    ori->ori_blks = (M_pad / 64) * (N_pad / 64);
    ori->launchGridDim = dim3h(static_cast<unsigned>(ori->ori_blks), 1, 1);
    tiles_ = ori->ori_blks;
    const unsigned sms = static_cast<unsigned>(backend().smCount());
    gptb.reset(new GPTBKernel(id, "tzgemm", "gptb_tzgemm", ori.get(), dim3h(sms, 1, 1), dim3h(192, 1, 1), 0, ori->ori_blks));
    // a layer with fewer 128 x 256 super-tiles than half the SMs and a long K (the batch-1 dense layers) runs
    // alone through the K-split form, which needs C zeroed first; fused launches keep the plain kernel
    const long long nsuper = static_cast<long long>(M_pad / 128) * ((N_pad + 255) / 256);
    skinny = nsuper * 2 <= sms && K_pad >= 1024;
    if (skinny)
        gptb_acc.reset(new GPTBKernel(id, "tzgemm", "gptb_tzgemm_acc", ori.get(), dim3h(sms, 1, 1), dim3h(192, 1, 1), 0,
                                      ori->ori_blks));
}

ConvKernel::ConvKernel(int id, const std::string& name, DnnArena& arena, const float* input, int H, int W, int Cin,
                       int Cout, int ksize, int pad, int stride, uint64_t seed)
    : input(input), H(H), W(W), Cin(Cin), Cout(Cout), ksize(ksize), pad(pad), stride(stride) {
    Id = id;
    kernelName = name;
    mixable = 2;
    OH = (H + 2 * pad - ksize) / stride + 1;
    OW = (W + 2 * pad - ksize) / stride + 1;
    M = OH * OW;
    N = Cout;
    K = ksize * ksize * Cin;
    M_pad = roundUp(M, 128);
    N_pad = roundUp(N, 64);
    K_pad = roundUp(K, 64);
    A = arena.half(static_cast<size_t>(M_pad) * K_pad);
    // He initialisation: uniform with variance 2 / fan_in
    B = arena.weightsHalf(static_cast<size_t>(N_pad) * K_pad, seed, std::sqrt(6.0f / static_cast<float>(K)));
    C = arena.act(static_cast<size_t>(M_pad) * N_pad);
    buildGemm(id);
}

std::vector<int> ConvKernel::getArgs() {
    // n, c, h, w, k, c, kh, kw, pad_h, pad_w, stride_h, stride_w, dilation_h, dilation_w
    return std::vector<int>{1, Cin, H, W, Cout, Cin, ksize, ksize, pad, pad, stride, stride, 1, 1};
}

void ConvKernel::prepare(stream_t stream) {
    TK_HOST_CHECK(backend().im2colNhwcHalf(input, H, W, Cin, ksize, ksize, pad, stride, A, M_pad, K_pad, stream));
}

ConvImplicitKernel::ConvImplicitKernel(int id, const std::string& name, DnnArena& arena, void* x_bordered, int H, int W,
                                       int Cin, int Cout, int act, uint64_t seed, const float* bias, void* y_bordered)
    : H(H), W(W), Cin(Cin), Cout(Cout) {
    Id = id;
    kernelName = name;
    mixable = 2;
    implicit = true;
    M = H * W;
    N = Cout;
    K = 9 * Cin;
    N_pad = N;
    K_pad = K;
    A = x_bordered;
    // He initialisation as in ConvKernel: same seed, same layout [N][K], k = (3 i + j) Cin + c
    B = arena.weightsHalf(static_cast<size_t>(N_pad) * K_pad, seed, std::sqrt(6.0f / static_cast<float>(K)));
    C = nullptr;
    ori_conv.reset(new OriTZCONVKernel(id, x_bordered, B, y_bordered, bias, H, W, Cin, Cout, act));
    M_pad = ori_conv->M_GLOBAL;
    tiles_ = ori_conv->ori_blks;
    const unsigned sms = static_cast<unsigned>(backend().smCount());
    gptb.reset(new GPTBKernel(id, "tzconv", "gptb_tzconv", ori_conv.get(), dim3h(sms, 1, 1), dim3h(192, 1, 1), 0, tiles_));
}

std::vector<int> ConvImplicitKernel::getArgs() {
    return std::vector<int>{1, Cin, H, W, Cout, Cin, 3, 3, 1, 1, 1, 1, 1, 1};
}

GemmKernel::GemmKernel(int id, const std::string& name, DnnArena& arena, const float* input, int rows, int in_features,
                       int out_features, uint64_t seed)
    : input(input) {
    Id = id;
    kernelName = name;
    mixable = 1;
    M = rows;
    N = out_features;
    K = in_features;
    M_pad = roundUp(M, 128);
    N_pad = roundUp(N, 64);
    K_pad = roundUp(K, 64);
    A = arena.half(static_cast<size_t>(M_pad) * K_pad);
    B = arena.weightsHalf(static_cast<size_t>(N_pad) * K_pad, seed, std::sqrt(6.0f / static_cast<float>(K)));
    C = arena.act(static_cast<size_t>(M_pad) * N_pad);
    buildGemm(id);
}

void GemmKernel::prepare(stream_t stream) {
    if (a_ready) return;
    if (bordered) TK_HOST_CHECK(backend().unborderHalf(bordered, bH, bW, bC, A, stream));  // rows 1.. of A stay zero
    else TK_HOST_CHECK(backend().rowsToHalf(input, M, K, K, A, M_pad, K_pad, stream));
}

void OpKernel::executeImpl(stream_t s) {
    if (absorbed) return;
    Backend& be = backend();
    switch (op) {
        case BiasAct:  // a = x [i0 rows][ld i2], b = bias, out [i0][i1 cols] ld i3, act i4
            if (hout) TK_HOST_CHECK(be.biasActHalf(a, i2, b, out, i3, hout, i5, i0, i1, i4, s));  // hout: ld i5; out may be null
            else TK_HOST_CHECK(be.biasAct(a, i2, b, out, i0, i1, i3, i4, s));
            break;
        case MaxPool:  // a = x [H i0][W i1][C i2]
            TK_HOST_CHECK(be.maxpool2x2(a, i0, i1, i2, out, s));
            break;
        case Add:
            TK_HOST_CHECK(be.add(a, b, out, static_cast<long long>(i0) * i1, s));
            break;
        case SoftmaxRows:  // rows i0 * i1, cols i2, scale f0
            if (hout) TK_HOST_CHECK(be.softmaxRowsHalf(a, hout, static_cast<long long>(i0) * i1, i2, f0, s));
            else TK_HOST_CHECK(be.softmaxRows(a, out, static_cast<long long>(i0) * i1, i2, f0, s));
            break;
        case LayerNorm:  // rows i0, cols i1, gamma b, beta c; res: added to a first
            if (res || hout || bias) TK_HOST_CHECK(be.addLayernormRows(a, bias, res, b, c, out, hout, i0, i1, 1e-12f, s));
            else TK_HOST_CHECK(be.layernormRows(a, b, c, out, i0, i1, 1e-12f, s));
            break;
        case SplitHeads:  // a [B i0 * S i1][ld i2] from col i3, heads i4, dh i5, transpose i6
            TK_HOST_CHECK(be.splitHeads(a, i2, i3, i0, i1, i4, i5, i6, hout, s));
            break;
        case MergeHeads:  // a [B*heads][S][dh] -> out [B*S][heads*dh]
            if (hout) TK_HOST_CHECK(be.mergeHeadsHalf(a, i0, i1, i4, i5, hout, s));
            else TK_HOST_CHECK(be.mergeHeads(a, i0, i1, i4, i5, out, s));
            break;
        case SplitQkv:  // a [B i0 * S i1][ld i2] = three projections side by side; heads i4, dh i5 -> hout, hout2, hout3
            TK_HOST_CHECK(be.splitQkv(a, bias, i2, i0, i1, i4, i5, hout, hout2, hout3, s));
            break;
        case BatchedGemm:  // out[batch i3] = f0 * ha [M i0][K i2] * hb [N i1][K i2]^T
            TK_HOST_CHECK(be.tzgemmBatched(ha, hb, out, i0, i1, i2, i3, f0, s));
            break;
        case BiasActHalfBordered:  // a = x [H i0 * W i1][ld i3], b = bias, hout = bordered fp16 [H+2][W+2][C i2], act i4
            TK_HOST_CHECK(be.biasActHalfBordered(a, i3, b, hout, i0, i1, i2, i4, s));
            break;
        case MaxPoolHalfBordered:  // ha = bordered fp16 [H i0 + 2][W i1 + 2][C i2] -> hout bordered [H/2 + 2][W/2 + 2][C]
            TK_HOST_CHECK(be.maxpoolHalfBordered(ha, i0, i1, i2, hout, s));
            break;
        case RowsToHalf:  // a [rows i0][cols i1] -> hout (same shape, fp16)
            TK_HOST_CHECK(be.rowsToHalf(a, i0, i1, i1, hout, i0, i1, s));
            break;
    }
}
