// GraphTask: a model task built from a description file, with constants read from NNFusion-style .bin files
// (see models.h).  Reference counterparts: the generated per-model classes (src/nnf/gen_code.py:69-246 turns
// NNFusion's nnfusion_rt.cu into them) and their Constant nodes (src/dnn/vgg16/vgg16_kernel_class.h:378-391: a raw
// read of `Constant/Constant_<n>_0.bin` into the node's buffer).
#include <cmath>
#include <fstream>
#include <sstream>
#include <stdexcept>

#include "../Logger.h"
#include "../json.h"
#include "models.h"

namespace {
std::string slurp(const std::string& path) {
    std::ifstream f(path, std::ios::in | std::ios::binary);
    if (f.fail()) throw std::runtime_error("cannot open " + path);
    std::ostringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

std::string dirOf(const std::string& path) {
    const size_t slash = path.find_last_of('/');
    return slash == std::string::npos ? std::string(".") : path.substr(0, slash);
}

double numberOr(const JsonValue* obj, const std::string& key, double dflt) {
    const JsonValue* v = obj ? obj->get(key) : nullptr;
    return v && v->kind == JsonValue::Number ? v->num : dflt;
}

std::string stringOr(const JsonValue* obj, const std::string& key, const std::string& dflt) {
    const JsonValue* v = obj ? obj->get(key) : nullptr;
    return v && v->kind == JsonValue::String ? v->str : dflt;
}

int actOf(const std::string& name) {  // the codes of tk_bias_act: 0 none, 1 ReLU, 2 GELU
    if (name == "relu") return 1;
    if (name == "gelu") return 2;
    if (name == "none" || name.empty()) return 0;
    throw std::runtime_error("unknown activation {" + name + "}");
}
}  // namespace

std::vector<float> GraphTask::readConstant(const std::string& file, size_t count) {
    const std::string path = constantDir + "/" + file;
    std::ifstream f(path, std::ios::in | std::ios::binary | std::ios::ate);
    if (f.fail()) throw std::runtime_error("Load " + path + " failed.");
    const std::streamsize bytes = f.tellg();
    if (bytes != static_cast<std::streamsize>(count * sizeof(float)))
        throw std::runtime_error(path + ": " + std::to_string(bytes) + " bytes, the layer needs " +
                                 std::to_string(count * sizeof(float)));
    f.seekg(0);
    std::vector<float> v(count);
    f.read(reinterpret_cast<char*>(v.data()), bytes);
    ++loadedConstants;
    return v;
}

// filter [3][3][Cin][Cout] -> the layer's fp16 operand B[n][(3 i + j) Cin + c]; bias [Cout]
void GraphTask::loadConv(const std::string& wfile, const std::string& bfile, int Cin, int Cout) {
    TzLayer* l = lastLayer;
    if (!wfile.empty()) {
        const std::vector<float> w = readConstant(wfile, 9ull * Cin * Cout);
        std::vector<uint16_t> b(static_cast<size_t>(l->N_pad) * l->K_pad, 0);
        for (int t = 0; t < 9; ++t)
            for (int c = 0; c < Cin; ++c)
                for (int n = 0; n < Cout; ++n)
                    b[static_cast<size_t>(n) * l->K_pad + t * Cin + c] = dnn_half_bits(w[(static_cast<size_t>(t) * Cin + c) * Cout + n]);
        backend().upload(l->B, b.data(), b.size() * 2, nullptr);
    }
    if (!bfile.empty()) {
        const std::vector<float> bias = readConstant(bfile, Cout);
        backend().upload(lastBias, bias.data(), bias.size() * sizeof(float), nullptr);
    }
    backend().streamSync(nullptr);
}

// weights [in][out] -> B[n][k]; bias [out]
void GraphTask::loadDense(const std::string& wfile, const std::string& bfile, int in, int out) {
    TzLayer* l = lastLayer;
    if (!wfile.empty()) {
        const std::vector<float> w = readConstant(wfile, static_cast<size_t>(in) * out);
        std::vector<uint16_t> b(static_cast<size_t>(l->N_pad) * l->K_pad, 0);
        for (int k = 0; k < in; ++k)
            for (int n = 0; n < out; ++n) b[static_cast<size_t>(n) * l->K_pad + k] = dnn_half_bits(w[static_cast<size_t>(k) * out + n]);
        backend().upload(l->B, b.data(), b.size() * 2, nullptr);
    }
    if (!bfile.empty()) {
        const std::vector<float> bias = readConstant(bfile, out);
        backend().upload(lastBias, bias.data(), bias.size() * sizeof(float), nullptr);
    }
    backend().streamSync(nullptr);
}

GraphTask::GraphTask(const std::string& descriptionFile) : DnnTask(3, "graph") {
    taskType = LC;
    const std::shared_ptr<JsonValue> root = parse_json(slurp(descriptionFile));
    if (root->kind != JsonValue::Object) throw std::runtime_error(descriptionFile + ": not a JSON object");
    taskName = stringOr(root.get(), "name", "graph");
    config = stringOr(root.get(), "config", "vgg16");
    constantDir = dirOf(descriptionFile) + "/" + stringOr(root.get(), "constants", ".");
    const JsonValue* in = root->get("input");
    int H = static_cast<int>(numberOr(in, "h", 0)), W = static_cast<int>(numberOr(in, "w", 0)),
        C = static_cast<int>(numberOr(in, "c", 0));
    if (H <= 0 || W <= 0 || C <= 0) throw std::runtime_error(descriptionFile + ": input needs h, w, c");
    hostInput.resize(static_cast<size_t>(H) * W * C);
    const std::string inputFile = stringOr(in, "file", "");
    if (!inputFile.empty()) {
        hostInput = readConstant(inputFile, hostInput.size());
    } else {
        const uint64_t seed = static_cast<uint64_t>(numberOr(in, "seed", 42));
        for (size_t i = 0; i < hostInput.size(); ++i) hostInput[i] = 2.0f * tk_unit_draw(seed, i) - 1.0f;
    }
    input = arena.act(hostInput.size());

    const JsonValue* layers = root->get("layers");
    if (!layers || layers->kind != JsonValue::Array) throw std::runtime_error(descriptionFile + ": no layers");
    void* img = nullptr;        // bordered fp16 image once a convolution has run
    const float* x = nullptr;   // fp32 row once a dense layer has run
    int features = 0;
    for (const auto& lp : layers->items) {
        const JsonValue* l = lp.get();
        const std::string op = stringOr(l, "op", "");
        if (op == "conv3x3") {
            if (x) throw std::runtime_error("conv3x3 after a dense layer");
            const int out = static_cast<int>(numberOr(l, "out", 0)), act = actOf(stringOr(l, "act", "relu"));
            if (out <= 0) throw std::runtime_error("conv3x3 needs out");
            if (img && (C % 64 || out % 64)) throw std::runtime_error("conv3x3: channel counts must be multiples of 64 after the first layer");
            img = img ? convBordered(img, H, W, C, out, act) : convToBordered(input, H, W, C, out, act);
            loadConv(stringOr(l, "weight", ""), stringOr(l, "bias", ""), C, out);
            C = out;
        } else if (op == "maxpool") {
            if (!img || H % 2 || W % 2) throw std::runtime_error("maxpool needs a convolution output of even size");
            img = poolBordered(img, H, W, C);
            H /= 2;
            W /= 2;
        } else if (op == "dense") {
            const int out = static_cast<int>(numberOr(l, "out", 0)), act = actOf(stringOr(l, "act", "none"));
            if (out <= 0) throw std::runtime_error("dense needs out");
            if (!x) {
                if (!img) throw std::runtime_error("dense as the first layer: start with conv3x3");
                features = H * W * C;
                x = denseFromBordered(img, H, W, C, out, act);
            } else {
                x = dense(x, 1, features, out, act);
            }
            loadDense(stringOr(l, "weight", ""), stringOr(l, "bias", ""), features, out);
            features = out;
        } else if (op == "softmax") {
            if (!x) throw std::runtime_error("softmax needs a dense output");
            // scores and probabilities share one buffer so that both can be read back in one piece
            float* both = arena.act(2 * static_cast<size_t>(features));
            const int idc = nextId++;
            auto* cp = new OpKernel(idc, "Copy_" + std::to_string(idc), OpKernel::BiasAct);
            cp->a = x, cp->b = nullptr, cp->out = both, cp->i0 = 1, cp->i1 = features, cp->i2 = features, cp->i3 = features, cp->i4 = 0;
            keep(cp);
            const int ids = nextId++;
            auto* sm = new OpKernel(ids, "Softmax_" + std::to_string(ids), OpKernel::SoftmaxRows);
            sm->a = both, sm->out = both + features, sm->i0 = 1, sm->i1 = 1, sm->i2 = features, sm->f0 = 1.0f;
            keep(sm);
            result = both;
            resultCount = 2 * static_cast<size_t>(features);
            x = both;
        } else {
            throw std::runtime_error("unknown op {" + op + "}");
        }
    }
    if (!result) {
        if (!x) throw std::runtime_error(descriptionFile + ": the model must end in a dense layer or a softmax");
        result = x;
        resultCount = static_cast<size_t>(features);
    }
}
