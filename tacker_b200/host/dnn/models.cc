#include "models.h"

#include <cmath>

#include "../Logger.h"

DnnTask::~DnnTask() {}

void DnnTask::initExecution() {
    if (input && !hostInput.empty())
        backend().upload(input, hostInput.data(), hostInput.size() * sizeof(float), execStream);
}

std::vector<float> DnnTask::downloadResult(stream_t stream) {
    std::vector<float> h(resultCount);
    if (result && resultCount) {
        backend().download(h.data(), result, resultCount * sizeof(float), stream);
        backend().streamSync(stream);
    }
    return h;
}

size_t DnnTask::numMixable() const {
    size_t n = 0;
    for (auto* k : kernels) n += (k->mixable != 0);
    return n;
}

double DnnTask::gemmFlops() const {
    double f = 0.0;
    for (auto* k : kernels)
        if (k->mixable != 0) {
            auto* t = static_cast<TzLayer*>(k);
            f += 2.0 * t->M * t->N * t->K;
        }
    return f;
}

float* DnnTask::conv(const float* x, int H, int W, int Cin, int Cout, int k, int pad, int stride, int act, int* OH,
                     int* OW) {
    const int id1 = nextId++;
    auto* c = new ConvKernel(id1, "Convolution_" + std::to_string(id1), arena, x, H, W, Cin, Cout, k, pad, stride,
                             1000 + id1);
    keep(c);
    *OH = c->OH;
    *OW = c->OW;
    float* y = arena.act(static_cast<size_t>(c->M) * Cout);
    float* bias = arena.weightsF32(Cout, 5000 + nextId, -0.05f, 0.05f);
    lastLayer = c;
    lastBias = bias;
    const int id2 = nextId++;
    auto* b = new OpKernel(id2, "BiasAct_" + std::to_string(id2), OpKernel::BiasAct);
    b->a = c->C;
    b->b = bias;
    b->out = y;
    b->i0 = c->M;
    b->i1 = Cout;
    b->i2 = c->N_pad;
    b->i3 = Cout;
    b->i4 = act;
    keep(b);
    return y;
}

float* DnnTask::dense(const float* x, int rows, int in, int out, int act, float* y) {
    const int id3 = nextId++;
    auto* g = new GemmKernel(id3, "Dot_" + std::to_string(id3), arena, x, rows, in, out, 2000 + id3);
    keep(g);
    if (!y) y = arena.act(static_cast<size_t>(rows) * out);
    float* bias = arena.weightsF32(out, 6000 + nextId, -0.05f, 0.05f);
    lastLayer = g;
    lastBias = bias;
    const int id4 = nextId++;
    auto* b = new OpKernel(id4, "BiasAct_" + std::to_string(id4), OpKernel::BiasAct);
    b->a = g->C;
    b->b = bias;
    b->out = y;
    b->i0 = rows;
    b->i1 = out;
    b->i2 = g->N_pad;
    b->i3 = out;
    b->i4 = act;
    keep(b);
    lastOp = b;
    return y;
}

float* DnnTask::pool(const float* x, int H, int W, int C) {
    float* y = arena.act(static_cast<size_t>(H / 2) * (W / 2) * C);
    const int id5 = nextId++;
    auto* p = new OpKernel(id5, "MaxPool_" + std::to_string(id5), OpKernel::MaxPool);
    p->a = x;
    p->out = y;
    p->i0 = H;
    p->i1 = W;
    p->i2 = C;
    keep(p);
    return y;
}

void* DnnTask::borderedImage(int H, int W, int C) {
    return arena.half(static_cast<size_t>(H + 2) * (W + 2) * C);  // zeroed: the border stays zero for good
}

void* DnnTask::convToBordered(const float* x, int H, int W, int Cin, int Cout, int act) {
    const int id1 = nextId++;
    auto* c = new ConvKernel(id1, "Convolution_" + std::to_string(id1), arena, x, H, W, Cin, Cout, 3, 1, 1, 1000 + id1);
    keep(c);
    void* y = borderedImage(H, W, Cout);
    float* bias = arena.weightsF32(Cout, 5000 + nextId, -0.05f, 0.05f);
    lastLayer = c;
    lastBias = bias;
    const int id2 = nextId++;
    auto* b = new OpKernel(id2, "BiasAct_" + std::to_string(id2), OpKernel::BiasActHalfBordered);
    b->a = c->C;
    b->b = bias;
    b->hout = y;
    b->i0 = H;
    b->i1 = W;
    b->i2 = Cout;
    b->i3 = c->N_pad;
    b->i4 = act;
    keep(b);
    return y;
}

void* DnnTask::convBordered(void* x, int H, int W, int Cin, int Cout, int act) {
    // numbered like conv(): one id for the convolution, one for the bias + activation node it has absorbed, so
    // that the seeds of weights and biases do not depend on which form a layer takes
    const int id1 = nextId++;
    void* y = borderedImage(H, W, Cout);
    float* bias = arena.weightsF32(Cout, 5000 + nextId, -0.05f, 0.05f);
    nextId++;
    auto* c = new ConvImplicitKernel(id1, "Convolution_" + std::to_string(id1), arena, x, H, W, Cin, Cout, act, 1000 + id1, bias, y);
    keep(c);
    lastLayer = c;
    lastBias = bias;
    return y;
}

void* DnnTask::poolBordered(void* x, int H, int W, int C) {
    void* y = borderedImage(H / 2, W / 2, C);
    const int id5 = nextId++;
    auto* p = new OpKernel(id5, "MaxPool_" + std::to_string(id5), OpKernel::MaxPoolHalfBordered);
    p->ha = x;
    p->hout = y;
    p->i0 = H;
    p->i1 = W;
    p->i2 = C;
    keep(p);
    return y;
}

float* DnnTask::denseFromBordered(void* x, int H, int W, int C, int out, int act) {
    const int id3 = nextId++;
    auto* g = new GemmKernel(id3, "Dot_" + std::to_string(id3), arena, nullptr, 1, H * W * C, out, 2000 + id3);
    g->bordered = x;
    g->bH = H, g->bW = W, g->bC = C;
    keep(g);
    float* y = arena.act(static_cast<size_t>(out));
    float* bias = arena.weightsF32(out, 6000 + nextId, -0.05f, 0.05f);
    lastLayer = g;
    lastBias = bias;
    const int id4 = nextId++;
    auto* b = new OpKernel(id4, "BiasAct_" + std::to_string(id4), OpKernel::BiasAct);
    b->a = g->C;
    b->b = bias;
    b->out = y;
    b->i0 = 1;
    b->i1 = out;
    b->i2 = g->N_pad;
    b->i3 = out;
    b->i4 = act;
    keep(b);
    return y;
}

float* DnnTask::addTo(const float* a, const float* b, int rows, int cols, int act) {
    float* y = arena.act(static_cast<size_t>(rows) * cols);
    const int id6 = nextId++;
    auto* k = new OpKernel(id6, "Add_" + std::to_string(id6), OpKernel::Add);
    k->a = a;
    k->b = b;
    k->out = y;
    k->i0 = rows;
    k->i1 = cols;
    keep(k);
    if (act) {
        const int id7 = nextId++;
        auto* r = new OpKernel(id7, "Relu_" + std::to_string(id7), OpKernel::BiasAct);
        r->a = y;
        r->b = nullptr;
        r->out = y;
        r->i0 = rows;
        r->i1 = cols;
        r->i2 = cols;
        r->i3 = cols;
        r->i4 = act;
        keep(r);
    }
    return y;
}

float* DnnTask::layernorm(const float* x, int rows, int cols) {
    float* y = arena.act(static_cast<size_t>(rows) * cols);
    const int id8 = nextId++;
    auto* k = new OpKernel(id8, "LayerNorm_" + std::to_string(id8), OpKernel::LayerNorm);
    k->a = x;
    k->b = arena.weightsF32(cols, 7000 + nextId, 0.9f, 1.1f);
    k->c = arena.weightsF32(cols, 7500 + nextId, -0.05f, 0.05f);
    k->out = y;
    k->i0 = rows;
    k->i1 = cols;
    keep(k);
    lastOp = k;
    return y;
}

float* DnnTask::addLayernorm(const float* a, const float* b, int rows, int cols) {
    if (cols % 128 != 0 || cols > 1024) return layernorm(addTo(a, b, rows, cols, 0), rows, cols);
    nextId++;  // the addition's node: absorbed
    float* y = arena.act(static_cast<size_t>(rows) * cols);
    const int id8 = nextId++;
    auto* k = new OpKernel(id8, "AddLayerNorm_" + std::to_string(id8), OpKernel::LayerNorm);
    k->a = a;
    k->res = b;
    k->b = arena.weightsF32(cols, 7000 + nextId, 0.9f, 1.1f);
    k->c = arena.weightsF32(cols, 7500 + nextId, -0.05f, 0.05f);
    k->out = y;
    k->i0 = rows;
    k->i1 = cols;
    keep(k);
    lastOp = k;
    return y;
}

float* DnnTask::denseParts(const float* x, int rows, int in, int out, int parts, int act) {
    const int total = parts * out;
    if (out % 64 != 0) throw std::runtime_error("denseParts: the parts must be multiples of 64 columns wide");
    const int id3 = nextId;  // ids of part i: id3 + 2 i (product), id3 + 2 i + 1 (bias + activation)
    auto* g = new GemmKernel(id3, "Dot_" + std::to_string(id3), arena, x, rows, in, total, 2000 + id3);
    keep(g);
    float* y = arena.act(static_cast<size_t>(rows) * total);
    float* bias = arena.act(static_cast<size_t>(total));
    const float scale = std::sqrt(6.0f / static_cast<float>(in));
    std::vector<uint16_t> w(static_cast<size_t>(out) * g->K_pad);
    std::vector<float> bv(out);
    for (int p = 0; p < parts; ++p) {
        // what dense() p would have drawn: weights [N_pad = out][K_pad] with seed 2000 + its id, bias with 6000 + the next id
        for (size_t i = 0; i < w.size(); ++i) w[i] = dnn_half_bits((tk_unit_draw(2000 + id3 + 2 * p, i) * 2.0f - 1.0f) * scale);
        backend().upload(static_cast<char*>(g->B) + static_cast<size_t>(p) * w.size() * 2, w.data(), w.size() * 2, nullptr);
        for (int i = 0; i < out; ++i) bv[i] = -0.05f + tk_unit_draw(6000 + id3 + 2 * p + 1, i) * 0.1f;
        backend().upload(bias + static_cast<size_t>(p) * out, bv.data(), bv.size() * sizeof(float), nullptr);
    }
    backend().streamSync(nullptr);
    nextId += 2 * parts;
    lastLayer = g;
    lastBias = bias;
    auto* b = new OpKernel(id3 + 1, "BiasAct_" + std::to_string(id3 + 1), OpKernel::BiasAct);
    b->a = g->C;
    b->b = bias;
    b->out = y;
    b->i0 = rows;
    b->i1 = total;
    b->i2 = g->N_pad;
    b->i3 = total;
    b->i4 = act;
    keep(b);
    lastOp = b;
    return y;
}

bool DnnTask::feedHalf(OpKernel* producer, GemmKernel* consumer, int rows, int cols) {
    if (!producer || !consumer || rows % 128 != 0 || cols % 64 != 0 || consumer->M_pad != rows || consumer->K_pad != cols)
        return false;
    if (producer->op == OpKernel::LayerNorm && (cols % 128 != 0 || cols > 1024)) return false;
    if (producer->op == OpKernel::BiasAct) producer->i5 = consumer->K_pad;
    producer->hout = consumer->A;
    consumer->a_ready = true;
    return true;
}

static void normal_input(std::vector<float>& h, uint64_t seed) {  // ~N(0,1) by Box-Muller on counter draws
    for (size_t i = 0; i < h.size(); ++i) {
        const float u1 = tk_unit_draw(seed, 2 * i) + 2.98e-8f, u2 = tk_unit_draw(seed, 2 * i + 1);
        h[i] = std::sqrt(-2.0f * std::log(u1)) * std::cos(6.2831853f * u2);
    }
}

// ------------------------------------------------------------------ VGG16 ----
VGG16::VGG16(int numClasses) : DnnTask(0, "vgg16") {
    taskType = LC;
    int H = 224, W = 224, C = 3;
    hostInput.resize(static_cast<size_t>(H) * W * C);
    normal_input(hostInput, 42);
    input = arena.act(hostInput.size());
    // The first convolution (3 input channels) goes through im2col + tzgemm; from there on the activations are
    // zero-bordered NHWC fp16 images and every convolution is one implicit-GEMM kernel with bias and ReLU in its
    // epilogue.  Layer numbering (and with it every seed) is that of the explicit form.
    const int cfg[] = {64, 64, -1, 128, 128, -1, 256, 256, 256, -1, 512, 512, 512, -1, 512, 512, 512, -1};
    void* img = nullptr;
    for (int c : cfg) {
        if (c < 0) {
            img = poolBordered(img, H, W, C);
            H /= 2;
            W /= 2;
        } else {
            img = img ? convBordered(img, H, W, C, c, 1) : convToBordered(input, H, W, C, c, 1);
            C = c;
        }
    }
    const float* x = denseFromBordered(img, H, W, C, 4096, 1);  // 7*7*512 = 25088
    x = dense(x, 1, 4096, 4096, 1);
    // scores and probabilities share one buffer so that both can be read back in one piece
    float* scores = arena.act(2 * static_cast<size_t>(numClasses));
    x = dense(x, 1, 4096, numClasses, 0, scores);
    float* probs = scores + numClasses;
    result = scores;
    resultCount = 2 * static_cast<size_t>(numClasses);
    const int id9 = nextId++;
    auto* sm = new OpKernel(id9, "Softmax", OpKernel::SoftmaxRows);
    sm->a = x;
    sm->out = probs;
    sm->i0 = 1;
    sm->i1 = 1;
    sm->i2 = numClasses;
    sm->f0 = 1.0f;
    keep(sm);
}

// --------------------------------------------------------------- ResNet-50 ----
Resnet50::Resnet50(int numClasses) : DnnTask(1, "resnet50") {
    taskType = LC;
    int H = 224, W = 224, C = 3, oh, ow;
    hostInput.resize(static_cast<size_t>(H) * W * C);
    normal_input(hostInput, 43);
    input = arena.act(hostInput.size());
    const float* x = conv(input, H, W, C, 64, 7, 3, 2, 1, &oh, &ow);  // 112 x 112 x 64
    H = oh, W = ow, C = 64;
    x = pool(x, H, W, C);  // 56 x 56 (2x2 window; the original uses 3x3 stride 2, same output size)
    H /= 2, W /= 2;
    const int blocks[4] = {3, 4, 6, 3}, width[4] = {64, 128, 256, 512};
    for (int s = 0; s < 4; ++s)
        for (int b = 0; b < blocks[s]; ++b) {
            const int stride = (b == 0 && s > 0) ? 2 : 1, mid = width[s], out = 4 * width[s];
            const float* shortcut = x;
            int sh = H, sw = W;
            if (b == 0) shortcut = conv(x, H, W, C, out, 1, 0, stride, 0, &sh, &sw);
            const float* y = conv(x, H, W, C, mid, 1, 0, 1, 1, &oh, &ow);
            y = conv(y, H, W, mid, mid, 3, 1, stride, 1, &oh, &ow);
            y = conv(y, oh, ow, mid, out, 1, 0, 1, 0, &oh, &ow);
            H = oh, W = ow, C = out;
            x = addTo(y, shortcut, H * W, C, 1);
        }
    while (H > 1) {  // global pooling stand-in: 7 -> 3 -> 1
        x = pool(x, H, W, C);
        H /= 2, W /= 2;
    }
    x = dense(x, 1, C, numClasses, 0);
    result = x;
    resultCount = static_cast<size_t>(numClasses);
}

// ------------------------------------------------------------------- BERT ----
Bert::Bert(int layers, int batch_, int seq_) : DnnTask(2, "bert"), batch(batch_), seq(seq_) {
    taskType = BE;
    const int hidden = 768, heads = 12, dh = 64, ffn = 3072, rows = batch * seq, bh = batch * heads;
    // token ids uniform over the vocabulary; the embedding lookup is done on the host, the encoder input is
    // the gathered rows (word + position), layer-normalised on the device
    const int vocab = 30522;
    hostInput.resize(static_cast<size_t>(rows) * hidden);
    for (int r = 0; r < rows; ++r) {
        const uint64_t token = static_cast<uint64_t>(tk_unit_draw(77, r) * vocab);
        for (int c = 0; c < hidden; ++c)
            hostInput[static_cast<size_t>(r) * hidden + c] =
                (tk_unit_draw(1000 + token, c) - 0.5f) * 0.1f + (tk_unit_draw(900000 + (r % seq), c) - 0.5f) * 0.02f;
    }
    input = arena.act(hostInput.size());
    // Every producer of a product's input writes that product's fp16 operand itself (normalisation, GELU, softmax and
    // head merge have an fp16 output next to or instead of the fp32 one), the three attention projections are one
    // product and their heads are cut out in one launch, and a product's bias is added by the node that reads it where
    // no activation sits between: 12 launches per layer instead of 30.  The node numbers, which
    // fix the seeds, advance as if every absorbed node were still there.
    const float* x = layernorm(input, rows, hidden);
    OpKernel* norm = lastOp;
    for (int l = 0; l < layers; ++l) {
        // query, key and value projections as one product of 3 x 768 columns
        denseParts(x, rows, hidden, hidden, 3, 0);
        GemmKernel* gq = static_cast<GemmKernel*>(lastLayer);
        feedHalf(norm, gq, rows, hidden);
        lastOp->absorbed = true;  // the projections' bias is added by the head split, which reads the raw product
        const float* qkv_bias = lastBias;
        void* qh = arena.half(static_cast<size_t>(rows) * hidden);
        void* kh = arena.half(static_cast<size_t>(rows) * hidden);
        void* vt = arena.half(static_cast<size_t>(rows) * hidden);
        const int id10 = nextId;
        nextId += 3;  // the three head splits
        auto* sp = new OpKernel(id10, "SplitHeads_" + std::to_string(id10), OpKernel::SplitQkv);
        sp->a = gq->C, sp->bias = qkv_bias, sp->hout = qh, sp->hout2 = kh, sp->hout3 = vt;
        sp->i0 = batch, sp->i1 = seq, sp->i2 = gq->N_pad, sp->i4 = heads, sp->i5 = dh;
        keep(sp);
        float* scores = arena.act(static_cast<size_t>(bh) * seq * seq);
        const int id11 = nextId++;
        auto* g1 = new OpKernel(id11, "BatchMatMul_" + std::to_string(id11), OpKernel::BatchedGemm);
        g1->ha = qh, g1->hb = kh, g1->out = scores;
        g1->i0 = seq, g1->i1 = seq, g1->i2 = dh, g1->i3 = bh, g1->f0 = 1.0f / std::sqrt(static_cast<float>(dh));
        keep(g1);
        void* ph = arena.half(static_cast<size_t>(bh) * seq * seq);
        const int id12 = nextId++;
        auto* sm = new OpKernel(id12, "Softmax_" + std::to_string(id12), OpKernel::SoftmaxRows);
        sm->a = scores, sm->hout = ph, sm->i0 = bh, sm->i1 = seq, sm->i2 = seq, sm->f0 = 1.0f;  // probabilities as fp16
        keep(sm);
        nextId++;  // the conversion node: absorbed by the softmax
        float* ctx = arena.act(static_cast<size_t>(rows) * hidden);
        const int id14 = nextId++;
        auto* g2 = new OpKernel(id14, "BatchMatMul_" + std::to_string(id14), OpKernel::BatchedGemm);
        g2->ha = ph, g2->hb = vt, g2->out = ctx;
        g2->i0 = seq, g2->i1 = dh, g2->i2 = seq, g2->i3 = bh, g2->f0 = 1.0f;
        keep(g2);
        float* merged = arena.act(static_cast<size_t>(rows) * hidden);
        const int id15 = nextId++;
        auto* mh = new OpKernel(id15, "MergeHeads_" + std::to_string(id15), OpKernel::MergeHeads);
        mh->a = ctx, mh->out = merged, mh->i0 = batch, mh->i1 = seq, mh->i4 = heads, mh->i5 = dh;
        keep(mh);
        const float* proj = dense(merged, rows, hidden, hidden, 0);
        GemmKernel* gp = static_cast<GemmKernel*>(lastLayer);
        feedHalf(mh, gp, rows, hidden);  // the merge then writes fp16 only
        OpKernel* proj_bias_node = lastOp;
        const float* proj_bias = lastBias;
        x = addLayernorm(proj, x, rows, hidden);
        norm = lastOp;
        if (norm->res && gp->N_pad == hidden) {  // the normalisation reads the raw product and adds its bias itself
            norm->a = gp->C, norm->bias = proj_bias;
            proj_bias_node->absorbed = true;
        }
        const float* h1 = dense(x, rows, hidden, ffn, 2);
        feedHalf(norm, static_cast<GemmKernel*>(lastLayer), rows, hidden);
        OpKernel* gelu = lastOp;
        const float* h2 = dense(h1, rows, ffn, hidden, 0);
        GemmKernel* g2f = static_cast<GemmKernel*>(lastLayer);
        if (feedHalf(gelu, g2f, rows, ffn)) gelu->out = nullptr;  // nobody reads the fp32 copy
        OpKernel* ffn_bias_node = lastOp;
        const float* ffn_bias = lastBias;
        x = addLayernorm(h2, x, rows, hidden);
        norm = lastOp;
        if (norm->res && g2f->N_pad == hidden) {
            norm->a = g2f->C, norm->bias = ffn_bias;
            ffn_bias_node->absorbed = true;
        }
    }
    result = x;  // the last layer's hidden states [batch * seq][hidden]
    resultCount = static_cast<size_t>(rows) * hidden;
}

Task* createTask(const std::string& taskName) {
    if (taskName == "vgg16") return new VGG16(1000);
    if (taskName == "resnet50") return new Resnet50(1000);
    if (taskName == "bert") return new Bert(12, 8, 128);
    if (taskName.size() > 5 && taskName.compare(taskName.size() - 5, 5, ".json") == 0) return new GraphTask(taskName);
    logger.ERROR("Task name not found: " + taskName);
}
