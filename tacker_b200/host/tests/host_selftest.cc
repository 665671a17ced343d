// host_selftest.cc -- the host runtime against a recording double of the device library.
// TEST INFRASTRUCTURE: no CUDA, no GPU, no arithmetic.  The double records every launch (key, argument
// list, geometry) and keeps a virtual clock driven by a simple cost model, so that argument marshalling,
// the registry, the JSON reader and the scheduling rules can be checked on any machine.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <unistd.h>
#include <fstream>
#include <functional>
#include <iostream>
#include <map>
#include <sstream>

#include "../Backend.h"
#include "../Creator.h"
#include "../Logger.h"
#include "../ModuleCenter.h"
#include "../Recorder.h"
#include "../TaskManager.h"
#include "../dnn/models.h"
#include "../json.h"

// ---- the few pure-host entry points of the C ABI the runtime calls directly ----
extern "C" {
const char* tk_status_string(int s) { return s == 0 ? "ok" : "error"; }
const char* tk_last_error(void) { return ""; }
int tk_tzgemm_dims(int m, int n, int k, int out[4]) {
    const int M = (m < 128) ? 128 : (m / 128) * 128, N = (n < 128) ? 128 : (n / 128) * 128,
              K = (k < 128) ? 128 : (k / 128) * 128;
    out[0] = M, out[1] = N, out[2] = K, out[3] = (M / 64) * (N / 64);
    return 0;
}
int tk_conv_mnk(const int a[14], int mnk[3]) {
    const int hcol = (a[2] + 2 * a[8] - (a[12] * (a[6] - 1) + 1)) / a[10] + 1;
    const int wcol = (a[3] + 2 * a[9] - (a[13] * (a[7] - 1) + 1)) / a[11] + 1;
    mnk[0] = a[0] * hcol * wcol, mnk[1] = a[4], mnk[2] = a[6] * a[7] * a[1];
    return 0;
}
}

struct Launch {
    std::string key;
    int nparams;
    unsigned grid, block;
    std::vector<int> tail;  // the last ints of the list (ranges)
};
static std::vector<Launch> g_launches;
static double g_clock_ms = 0.0;
static std::string g_current_key;

template <typename T>
static T argv_(void** p, int i) {
    T v;
    std::memcpy(&v, p[i], sizeof(T));
    return v;
}

static int record(const char* key, void** params, int n, const unsigned grid[3], const unsigned block[3]) {
    Launch l{key, n, grid[0], block[0], {}};
    const std::string k(key);
    double cost = 0.01;
    auto range = [&](int i_start) { return std::max(0, argv_<int>(params, i_start + 2) - argv_<int>(params, i_start)); };
    if (k == "gptb_tzgemm") {
        l.tail = {argv_<int>(params, 13), argv_<int>(params, 14), argv_<int>(params, 15)};
        cost = 0.001 * range(13) * argv_<int>(params, 5) / 1024.0 + 0.005;
    } else if (k == "gptb_tzconv") {  // 12 solo arguments, then geometry and the range
        l.tail = {argv_<int>(params, 18), argv_<int>(params, 19), argv_<int>(params, 20)};
        cost = 0.001 * range(18) * argv_<int>(params, 5) / 1024.0 + 0.005;
    } else if (k.rfind("tzconv_", 0) == 0) {
        const int cd_len = n - 21;
        l.tail = {argv_<int>(params, cd_len - 3), argv_<int>(params, cd_len - 1), argv_<int>(params, n - 3),
                  argv_<int>(params, n - 1)};
        const double cd = 0.00003 * range(cd_len - 3), tz = 0.001 * range(n - 3) * argv_<int>(params, cd_len + 5) / 1024.0;
        cost = std::max(cd, tz) + 0.25 * std::min(cd, tz) + 0.005;
    } else if (k == "gptb_stencil" || k == "gptb_mriq" || k == "gptb_cp" || k == "gptb_mrif" || k == "gptb_sgemm" ||
               k == "gptb_lbm" || k == "gptb_fft" || k == "gptb_cutcp") {
        const int s = n - 4;
        l.tail = {argv_<int>(params, s), argv_<int>(params, s + 1), argv_<int>(params, s + 2)};
        cost = 0.00003 * range(s) + 0.003;
    } else if (k.rfind("tzgemm_", 0) == 0) {
        const int cd_len = n - 16;
        l.tail = {argv_<int>(params, cd_len - 3), argv_<int>(params, cd_len - 1), argv_<int>(params, n - 3),
                  argv_<int>(params, n - 1)};
        const double cd = 0.00003 * range(cd_len - 3), tz = 0.001 * range(n - 3) * argv_<int>(params, cd_len + 5) / 1024.0;
        cost = std::max(cd, tz) + 0.25 * std::min(cd, tz) + 0.005;  // the two roles overlap
    }
    g_clock_ms += cost;
    g_launches.push_back(l);
    return 0;
}

#define FAKE_LAUNCHER(NAME, KEY)                                                                        \
    static int NAME(void** p, int n, const unsigned g[3], const unsigned b[3], unsigned, void*) {      \
        return record(KEY, p, n, g, b);                                                                 \
    }
FAKE_LAUNCHER(l_tz, "gptb_tzgemm")
FAKE_LAUNCHER(l_st, "gptb_stencil")
FAKE_LAUNCHER(l_cp, "gptb_cp")
FAKE_LAUNCHER(l_mq, "gptb_mriq")
FAKE_LAUNCHER(l_mst, "tzgemm_stencil")
FAKE_LAUNCHER(l_mcp, "tzgemm_cp")
FAKE_LAUNCHER(l_mmq, "tzgemm_mriq")
FAKE_LAUNCHER(l_tc, "gptb_tzconv")
FAKE_LAUNCHER(l_cst, "tzconv_stencil")
FAKE_LAUNCHER(l_ccp, "tzconv_cp")
FAKE_LAUNCHER(l_cmq, "tzconv_mriq")
FAKE_LAUNCHER(l_cmf, "tzconv_mrif")
FAKE_LAUNCHER(l_mf, "gptb_mrif")
FAKE_LAUNCHER(l_mmf, "tzgemm_mrif")
FAKE_LAUNCHER(l_omf, "ori_mrif")
FAKE_LAUNCHER(l_ost, "ori_stencil")
FAKE_LAUNCHER(l_ocp, "ori_cp")
FAKE_LAUNCHER(l_omq, "ori_mriq")
FAKE_LAUNCHER(l_sg, "gptb_sgemm")
FAKE_LAUNCHER(l_lb, "gptb_lbm")
FAKE_LAUNCHER(l_ff, "gptb_fft")
FAKE_LAUNCHER(l_cc, "gptb_cutcp")
FAKE_LAUNCHER(l_msg, "tzgemm_sgemm")
FAKE_LAUNCHER(l_mlb, "tzgemm_lbm")
FAKE_LAUNCHER(l_mff, "tzgemm_fft")
FAKE_LAUNCHER(l_mcc, "tzgemm_cutcp")
FAKE_LAUNCHER(l_csg, "tzconv_sgemm")
FAKE_LAUNCHER(l_clb, "tzconv_lbm")
FAKE_LAUNCHER(l_cff, "tzconv_fft")
FAKE_LAUNCHER(l_ccc, "tzconv_cutcp")
FAKE_LAUNCHER(l_osg, "ori_sgemm")
FAKE_LAUNCHER(l_olb, "ori_lbm")
FAKE_LAUNCHER(l_off, "ori_fft")
FAKE_LAUNCHER(l_occ, "ori_cutcp")

class FakeBackend : public Backend {
public:
    std::map<std::string, tk_launch_fn> table = {
        {"gptb_tzgemm", l_tz}, {"gptb_tzgemm_acc", l_tz}, {"gptb_stencil", l_st}, {"gptb_cp", l_cp},       {"gptb_mriq", l_mq},
        {"tzgemm_stencil", l_mst}, {"tzgemm_cp", l_mcp}, {"tzgemm_mriq", l_mmq}, {"ori_stencil", l_ost},
        {"ori_cp", l_ocp},     {"ori_mriq", l_omq},    {"gptb_mrif", l_mf},   {"tzgemm_mrif", l_mmf}, {"ori_mrif", l_omf},
        {"gptb_tzconv", l_tc}, {"tzconv_stencil", l_cst}, {"tzconv_cp", l_ccp}, {"tzconv_mriq", l_cmq}, {"tzconv_mrif", l_cmf},
        {"gptb_sgemm", l_sg},  {"gptb_lbm", l_lb},     {"gptb_fft", l_ff},    {"gptb_cutcp", l_cc},
        {"tzgemm_sgemm", l_msg}, {"tzgemm_lbm", l_mlb}, {"tzgemm_fft", l_mff}, {"tzgemm_cutcp", l_mcc},
        {"ori_sgemm", l_osg},  {"ori_lbm", l_olb},     {"ori_fft", l_off},    {"ori_cutcp", l_occ},
        {"tzconv_sgemm", l_csg}, {"tzconv_lbm", l_clb}, {"tzconv_fft", l_cff}, {"tzconv_cutcp", l_ccc}};
    int ops = 0;
    const char* name() const override { return "recording double"; }
    void setDevice(int) override {}
    int smCount() override { return 148; }
    tk_launch_fn lookup(const std::string& key) override {
        auto it = table.find(key);
        return it == table.end() ? nullptr : it->second;
    }
    int query(const std::string&, tk_kernel_info* info) override {
        std::memset(info, 0, sizeof(*info));
        return 0;
    }
    void* deviceAlloc(size_t bytes) override { return std::malloc(bytes < 64 ? 64 : (bytes > (1u << 20) ? (1u << 20) : bytes)); }
    void deviceFree(void* p) override { std::free(p); }
    void* hostAllocPinned(size_t bytes) override { return std::malloc(bytes); }
    void hostFreePinned(void* p) override { std::free(p); }
    // kernels never run here; small uploads are copied so that loaded constants can be inspected, and the streams of
    // uploads and fills are recorded
    std::vector<stream_t> upload_streams, fill_streams;
    void upload(void* dst, const void* src, size_t bytes, stream_t s) override {
        upload_streams.push_back(s);
        if (bytes <= (1u << 20)) std::memcpy(dst, src, bytes);  // allocations are capped at 1 MB: larger copies are dropped
    }
    void download(void*, const void*, size_t, stream_t) override {}
    void fillZero(void*, size_t, stream_t s) override { fill_streams.push_back(s); }
    stream_t streamCreate() override { return nullptr; }
    void streamSync(stream_t) override {}
    void deviceSync() override {}
    void* eventCreate() override { return new double(0.0); }
    void eventDestroy(void* e) override { delete static_cast<double*>(e); }
    void eventRecord(void* e, stream_t) override { *static_cast<double*>(e) = g_clock_ms; }
    float eventElapsedMs(void* a, void* b) override {
        return static_cast<float>(*static_cast<double*>(b) - *static_cast<double*>(a));
    }
    int captures = 0, replays = 0;
    void* graphCapture(stream_t, const std::function<void()>& body) override {
        ++captures;
        return new std::function<void()>(body);
    }
    void graphLaunch(void* g, stream_t) override {
        ++replays;
        (*static_cast<std::function<void()>*>(g))();
    }
    void graphDestroy(void* g) override { delete static_cast<std::function<void()>*>(g); }
    int op() {
        ++ops;
        g_clock_ms += 0.004;
        return 0;
    }
    int cpPackAtoms(const float*, int, float, float*, stream_t) override { return op(); }
    int mriqPackKvalues(const float*, const float*, const float*, const float*, const float*, int, float*, stream_t) override { return op(); }
    int mrifPackKvalues(const float*, const float*, const float*, const float*, const float*, const float*, const float*, int,
                        float*, stream_t) override { return op(); }
    int im2colNhwcHalf(const float*, int, int, int, int, int, int, int, void*, int, int, stream_t) override { return op(); }
    int rowsToHalf(const float*, int, int, int, void*, int, int, stream_t) override { return op(); }
    int biasActHalfBordered(const float*, int, const float*, void*, int, int, int, int, stream_t) override { return op(); }
    int maxpoolHalfBordered(const void*, int, int, int, void*, stream_t) override { return op(); }
    int unborderHalf(const void*, int, int, int, void*, stream_t) override { return op(); }
    int biasAct(const float*, int, const float*, float*, int, int, int, int, stream_t) override { return op(); }
    int maxpool2x2(const float*, int, int, int, float*, stream_t) override { return op(); }
    int add(const float*, const float*, float*, long long, stream_t) override { return op(); }
    int softmaxRows(const float*, float*, long long, int, float, stream_t) override { return op(); }
    int layernormRows(const float*, const float*, const float*, float*, long long, int, float, stream_t) override { return op(); }
    int addLayernormRows(const float*, const float*, const float*, const float*, const float*, float*, void*, long long, int, float, stream_t) override { return op(); }
    int biasActHalf(const float*, int, const float*, float*, int, void*, int, int, int, int, stream_t) override { return op(); }
    int softmaxRowsHalf(const float*, void*, long long, int, float, stream_t) override { return op(); }
    int mergeHeadsHalf(const float*, int, int, int, int, void*, stream_t) override { return op(); }
    int splitQkv(const float*, const float*, int, int, int, int, int, void*, void*, void*, stream_t) override { return op(); }
    int splitHeads(const float*, int, int, int, int, int, int, int, void*, stream_t) override { return op(); }
    int mergeHeads(const float*, int, int, int, int, float*, stream_t) override { return op(); }
    int tzgemmBatched(const void*, const void*, float*, int, int, int, int, float, stream_t) override { return op(); }
    unsigned deviceStatus() override { return 0; }
};

static int g_checks = 0, g_failed = 0;
#define CHECK(cond)                                                                   \
    do {                                                                              \
        ++g_checks;                                                                   \
        if (!(cond)) {                                                                \
            ++g_failed;                                                               \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);             \
        }                                                                             \
    } while (0)

static bool throws(const std::function<void()>& f) {
    try {
        f();
    } catch (const std::exception&) {
        return true;
    }
    return false;
}

int main(int argc, char** argv) {
    const std::string config_dir = argc > 1 ? argv[1] : "config";
    logger.quiet = true;
    FakeBackend fake;
    setBackend(&fake);

    // ---- JSON ----
    {
        auto v = parse_json("{\"a\": {\"b\": 3, \"c\": \"x\\u0041\", \"d\": [1, 2.5, true, null]}, \"e\": -1.5e2}");
        CHECK(v->get("a")->get("b")->num == 3);
        CHECK(v->get("a")->get("c")->str == "xA");
        CHECK(v->get("a")->get("d")->items.size() == 4 && v->get("a")->get("d")->items[1]->num == 2.5);
        CHECK(v->get("e")->num == -150.0);
        CHECK(throws([] { parse_json("{\"a\": }"); }));
        CHECK(throws([] { parse_json("{\"a\": 1} x"); }));
        CHECK(throws([] { read_json("/nonexistent/kinfo.json"); }));
        read_json(config_dir + "/kinfo-vgg16.json");
        read_common_json(config_dir + "/kinfo-common.json");
        CHECK(get_kernel_info("stencil", "ori_blks") == 1024);
        CHECK(get_kernel_info("stencil", "nope") == JSON_NOT_FOUND && get_kernel_info("nope", "x") == JSON_NOT_FOUND);
        CHECK(std::abs(fget_kernel_info("tzgemm_stencil", "4096") - 1.2f) < 1e-6f);
        CHECK(sget_kernel_info("throughput_test", "a") == "stencil");
        CHECK(geti(2, "vgg16", "MY_WMMA_BLK_PER_SM") == 1);
        CHECK(throws([] { geti(2, "vgg16", "missing"); }));
        add_kernel_info("stencil", "probe", 7);
        CHECK(get_kernel_info("stencil", "probe") == 7);
    }
    // ---- shape rules ----
    {
        auto d = getTZGEMMGridDim(1024, 1024, 1024);
        CHECK(d[0] == 1024 && d[3] == 256);
        d = getTZGEMMGridDim(1, 1000, 4096);
        CHECK(d[0] == 128 && d[1] == 896 && d[2] == 4096 && d[3] == 28);
        std::vector<int> a = {1, 64, 224, 224, 64, 64, 3, 3, 1, 1, 1, 1, 1, 1};
        auto mnk = get_mnk_from_cudnn_args(a);
        CHECK(mnk[0] == 50176 && mnk[1] == 64 && mnk[2] == 576);
    }
    // ---- registry and factories ----
    {
        GPTBKernel* cp = createKernel("cp");
        CHECK(cp == createKernel("cp"));
        CHECK(cp->funcKey == "gptb_cp" && cp->kernelParams.size() == 4 + 6);
        CHECK(cp->gptbParams.grid_dimension_x == 4 && cp->gptbParams.grid_dimension_y == 64);
        CHECK(cp->gptbParams.block_dimension_x == 16 && cp->gptbParams.block_dimension_y == 8);
        CHECK(cp->gptbParams.ptb_end_block_pos == 256);
        CHECK(throws([] { createKernel("pc"); }));      // an anagram is not a hit
        CHECK(throws([] { createKernel("hot3d"); }));     // outside the path
        CHECK(throws([] { createMixKernel("cp_fft"); }));
        GPTBKernel* st = createKernel("stencil");
        CHECK(st->kernelParams.size() == 7 + 6 && st->gptbParams.ptb_end_block_pos == 1024);
        CHECK(st->launchGridDim.x == 148u * 2u);
        g_launches.clear();
        st->execute(nullptr);
        CHECK(g_launches.size() == 1 && g_launches[0].key == "gptb_stencil" && g_launches[0].nparams == 17);
        CHECK(g_launches[0].tail[0] == 0 && g_launches[0].tail[1] == 296 && g_launches[0].tail[2] == 1024);
        MixKernel* mk = createMixKernel("tzgemm_stencil");
        CHECK(mk == createMixKernel("tzgemm_stencil"));
        CHECK(mk->kernelParams.size() == 32);  // stencil 7+6+3, tzgemm 7+6+3: CUDA-core list first
        CHECK(*static_cast<int*>(mk->kernelParams[13]) == 0 && *static_cast<int*>(mk->kernelParams[15]) == 1024);
        CHECK(*static_cast<int*>(mk->kernelParams[31]) == 4096);
        CHECK(*static_cast<float*>(mk->kernelParams[16 + 6]) == OriTZGEMMKernel::alpha_g);
        g_launches.clear();
        mk->setRanges(10, 20, 30, 40);
        mk->execute(nullptr);
        CHECK(g_launches.size() == 1 && g_launches[0].key == "tzgemm_stencil" && g_launches[0].block == 576);
        CHECK(g_launches[0].tail == (std::vector<int>{10, 20, 30, 40}));
        CHECK(createMixKernel("tzgemm_cp")->kernelParams.size() == 29);
        CHECK(createMixKernel("tzgemm_mriq")->kernelParams.size() == 33);
        GPTBKernel* mf = createKernel("mrif");
        CHECK(mf->funcKey == "gptb_mrif" && mf->kernelParams.size() == 8 + 6 && mf->gptbParams.ptb_end_block_pos == 1024);
        CHECK(createMixKernel("tzgemm_mrif")->kernelParams.size() == 33);
        // the other four Parboil kernels: argument counts and original grids of the reference's defaults
        creatorSGEMMProblem = SGEMMProblem{256, 64, 16};
        creatorLBMProblem = LBMProblem{32, 4, 3};
        creatorFFTProblem = FFTProblem{40};
        creatorCUTCPProblem = CUTCPProblem{16, 16, 16, 0.5f, 12.0f, 0.1f};
        GPTBKernel* sg = createKernel("sgemm");
        CHECK(sg->funcKey == "gptb_sgemm" && sg->kernelParams.size() == 6 + 6 && sg->gptbParams.ptb_end_block_pos == 2 * 4);
        GPTBKernel* lb = createKernel("lbm");
        CHECK(lb->funcKey == "gptb_lbm" && lb->kernelParams.size() == 2 + 6 && lb->gptbParams.ptb_end_block_pos == 12);
        GPTBKernel* ff = createKernel("fft");
        CHECK(ff->funcKey == "gptb_fft" && ff->kernelParams.size() == 1 + 6 && ff->gptbParams.ptb_end_block_pos == 40);
        GPTBKernel* cc = createKernel("cutcp");
        CHECK(cc->funcKey == "gptb_cutcp" && cc->kernelParams.size() == 10 + 6 && cc->gptbParams.ptb_end_block_pos == 8);
        {
            OriCUTCPKernel* oc = static_cast<OriCUTCPKernel*>(cc->kernel_);
            CHECK(oc->nbrlen == 335 && oc->binDim_x == 8 && oc->binDim_y == 8 && oc->binDim_z == 8);   // 7^3 cube without corners
            CHECK(*static_cast<int*>(cc->kernelParams[10]) == 2 && *static_cast<int*>(cc->kernelParams[13]) == 8 &&
                  *static_cast<int*>(cc->kernelParams[14]) == 2);
        }
        CHECK(createMixKernel("tzgemm_sgemm")->kernelParams.size() == 31 && createMixKernel("tzgemm_lbm")->kernelParams.size() == 27);
        CHECK(createMixKernel("tzgemm_fft")->kernelParams.size() == 26 && createMixKernel("tzgemm_cutcp")->kernelParams.size() == 35);
        OriTZGEMMKernel ori(0, 300, 200, 130);
        CHECK(ori.M_GLOBAL == 256 && ori.N_GLOBAL == 128 && ori.K_GLOBAL == 128 && ori.ori_blks == 8);
        CHECK(throws([&] { ori.execute(nullptr); }));   // "should not execute ori tzgemm!"
        CHECK(!moduleCenter.registerModule("nope", "/nonexistent/libnope.so") && !moduleCenter.hasModule("nope"));
        CHECK(moduleCenter.getFunction("nope", "tk_launch_gptb_cp") == nullptr);
    }
    // ---- model tasks ----
    {
        VGG16 vgg;
        CHECK(vgg.numMixable() == 16);
        int convs = 0;
        for (auto* k : vgg.kernels) convs += (k->mixable == 2);
        CHECK(convs == 13);
        auto* c1 = static_cast<TzLayer*>(vgg.kernels[0]);  // conv1_1: 3 input channels, explicit im2col + tzgemm
        CHECK(!c1->implicit && std::string(c1->fusedPrefix()) == "tzgemm_" && c1->K_pad == 64);
        auto* c2 = static_cast<TzLayer*>(vgg.kernels[2]);  // conv1_2: implicit GEMM over the bordered 224 x 226 grid
        std::vector<int> args = c2->getArgs();
        CHECK(args.size() == 14 && get_mnk_from_cudnn_args(args) == (std::vector<int>{50176, 64, 576}));
        CHECK(c2->implicit && std::string(c2->fusedPrefix()) == "tzconv_" && c2->gemm()->funcKey == "gptb_tzconv");
        CHECK(c2->M_pad == 50688 && c2->N_pad == 64 && c2->K_pad == 576 && c2->tiles() == 792);
        CHECK(c2->gemm()->kernelParams.size() == 12 + 6);
        CHECK(std::abs(vgg.gemmFlops() / 1e9 - 30.95) < 0.3);  // ~15.5 GMAC
        Bert bert(12, 8, 128);
        CHECK(bert.numMixable() == 48 && bert.taskType == BE);  // per layer: the fused query-key-value product, the output projection, two feed-forward layers
        Resnet50 rn;
        CHECK(rn.numMixable() == 54);  // 53 convolutions + the classifier
        CHECK(throws([] { createTask("alexnet"); }));
        // a model from a description file with NNFusion-style constant files
        {
            char dir[] = "tk_graph_selftest_XXXXXX";
            CHECK(mkdtemp(dir) != nullptr);
            const std::string d(dir);
            auto write_bin = [&](const std::string& name, size_t floats, float value) {
                std::vector<float> v(floats, value);
                std::ofstream f(d + "/" + name, std::ios::binary);
                f.write(reinterpret_cast<const char*>(v.data()), static_cast<std::streamsize>(floats * sizeof(float)));
            };
            write_bin("Constant_1_0.bin", 9 * 3 * 64, 0.5f);   // filter [3][3][3][64]
            write_bin("Constant_2_0.bin", 64, 0.25f);
            write_bin("Constant_3_0.bin", 4 * 4 * 64 * 10, 0.125f);   // dense [1024][10]
            {
                std::ofstream f(d + "/model.json");
                f << R"({"name": "tiny", "config": "vgg16", "input": {"h": 8, "w": 8, "c": 3, "seed": 7}, "constants": ".",
                         "layers": [{"op": "conv3x3", "out": 64, "act": "relu", "weight": "Constant_1_0.bin", "bias": "Constant_2_0.bin"},
                                    {"op": "maxpool"}, {"op": "dense", "out": 10, "act": "none", "weight": "Constant_3_0.bin"},
                                    {"op": "softmax"}]})";
            }
            std::unique_ptr<Task> t(createTask(d + "/model.json"));
            GraphTask* g = static_cast<GraphTask*>(t.get());
            CHECK(g->taskName == "tiny" && g->config == "vgg16" && g->loadedConstants == 3 && g->numMixable() == 2);
            CHECK(g->resultCount == 20);
            auto* conv = static_cast<TzLayer*>(g->kernels[0]);
            // B[n][(3 i + j) Cin + c] of the loaded filter: 0.5 = 0x3800 in binary16, zero in the padding of K
            const uint16_t* b = static_cast<const uint16_t*>(conv->B);
            CHECK(conv->K == 27 && conv->K_pad == 64 && b[0] == 0x3800 && b[26] == 0x3800 && b[27] == 0 && b[64] == 0x3800);
            write_bin("Constant_3_0.bin", 7, 0.0f);
            CHECK(throws([&] { createTask(d + "/model.json"); }));   // wrong size: refused, the file is named
            for (const char* f : {"Constant_1_0.bin", "Constant_2_0.bin", "Constant_3_0.bin", "model.json"}) unlink((d + "/" + f).c_str());
            rmdir(dir);
        }
        g_launches.clear();
        vgg.initExecution();
        vgg.executeTask(ExecutionMode::Aker, nullptr);
        CHECK(g_launches.size() == 16);  // the tzgemm / tzconv launches; every other node went through the layer calls
        CHECK(recorder.taskTime(vgg.taskId) > 0.0f);
        char recorder_path[] = "tk_recorder_selftest_XXXXXX";
        const int fd = mkstemp(recorder_path);
        CHECK(fd >= 0);
        if (fd >= 0) close(fd);
        CHECK(recorder.text(recorder_path) == vgg.kernels.size());
        std::remove(recorder_path);
    }
    // ---- scheduler ----
    {
        VGG16 vgg;
        TaskManager tm(&vgg, "stencil", "mriq");
        tm.profile_passes = 2, tm.schedule_passes = 2, tm.warmup_passes = 1;
        g_launches.clear();
        ScheduleResult aker = tm.executeAllTasks(ExecutionMode::Aker, nullptr);
        int fused = 0, over = 0, last_end = -1, restarts = 0;
        for (auto& l : g_launches)
            if (l.key == "tzgemm_stencil" || l.key == "tzconv_stencil") {
                ++fused;
                over += (l.tail[1] > 1024 || l.tail[0] < 0 || l.tail[1] <= l.tail[0]);
                restarts += (l.tail[0] == 0 && last_end > 0 && last_end != 0);
                last_end = l.tail[1] >= 1024 ? 0 : l.tail[1];
            }
        CHECK(fused > 0 && over == 0);
        CHECK(aker.mixable_times == 16 && aker.mix_times > 0 && aker.mix_times <= 16);
        CHECK(aker.be_blocks > 0 && aker.stage1_be_ms > 0 && aker.lc_solo_ms > 0);
        // Aker: blocks = tiles x ratio[K]; conv1_2 has 792 tiles and K = 576 -> ratio 1.2 * 576 / 4096
        bool saw = false;
        for (auto& l : g_launches)
            if (l.key == "tzconv_stencil" && l.tail[3] == 792 && l.tail[1] - l.tail[0] == static_cast<int>(792 * (1.2f * 576 / 4096.0f)))
                saw = true;
        CHECK(saw);
        g_launches.clear();
        ScheduleResult tacker = tm.executeAllTasks(ExecutionMode::Tacker, nullptr);
        bool all_blocks = false;
        for (auto& l : g_launches)
            if ((l.key == "tzgemm_stencil" || l.key == "tzconv_stencil") && l.tail[0] == 0 && l.tail[1] == 1024) all_blocks = true;
        CHECK(all_blocks && tacker.be_blocks >= aker.be_blocks);
        // stage 2: the leftover budget is filled with solo launches of both best-effort kernels, and what is
        // reported is what ran
        CHECK(aker.stage2_launches > 0 && aker.stage2_blocks1 > 0 && aker.stage2_blocks2 > 0);
        CHECK(aker.stage2_blocks1 % 1024 == 0 && aker.stage2_blocks2 % 1024 == 0);
        CHECK(aker.stage2_be_ms > 0 && aker.stage2_be_ms <= aker.qos_headroom_left + 1e-3f);
        // uploads and re-initialisations are queued on the stream the kernels run on
        {
            stream_t s1 = reinterpret_cast<stream_t>(0x40);
            fake.upload_streams.clear();
            fake.fill_streams.clear();
            TaskManager tm3(&vgg, "mriq", "cp");
            tm3.profile_passes = 1, tm3.schedule_passes = 1, tm3.warmup_passes = 1;
            tm3.executeAllTasks(ExecutionMode::Aker, s1);
            bool all_on_s1 = !fake.upload_streams.empty() && !fake.fill_streams.empty();
            for (stream_t s : fake.upload_streams) all_on_s1 = all_on_s1 && s == s1;
            int fills_on_s1 = 0;
            for (stream_t s : fake.fill_streams) fills_on_s1 += (s == s1);
            CHECK(all_on_s1 && fills_on_s1 >= 2);  // the LC input of every pass; Qr and Qi of the best-effort kernel
        }
        // a ratio that rounds to zero blocks leaves the layer unfused and the cursor where it was
        {
            add_kernel_info("tzgemm_cp", "576", 0);  // conv1_2 (K = 576): nothing to co-run
            TaskManager tm4(&vgg, "cp", "");
            tm4.profile_passes = 1, tm4.schedule_passes = 1, tm4.warmup_passes = 1;
            g_launches.clear();
            tm4.executeAllTasks(ExecutionMode::Aker, nullptr);
            int prev_end = 0, broken = 0, fused_cp = 0;
            for (auto& l : g_launches)
                if (l.key == "tzgemm_cp" || l.key == "tzconv_cp") {
                    ++fused_cp;
                    broken += !(l.tail[0] == prev_end || (l.tail[0] == 0 && prev_end >= 256));
                    broken += (l.tail[3] == 792);  // conv1_2 must not have been fused
                    prev_end = l.tail[1];
                }
            CHECK(fused_cp > 0 && broken == 0);
        }
        // the variant with one best-effort kernel: whole rounds of the SM count, always from block 0
        {
            TaskManager tm5(&vgg, "stencil", "mriq");
            tm5.profile_passes = 1, tm5.schedule_passes = 1, tm5.warmup_passes = 1;
            g_launches.clear();
            ScheduleResult one = tm5.execute_with_one_cd_kernel(ExecutionMode::Aker, nullptr);
            int bad = 0, n1 = 0;
            for (auto& l : g_launches)
                if (l.key == "tzgemm_stencil" || l.key == "tzconv_stencil") {
                    ++n1;
                    const int nb = l.tail[1] - l.tail[0];
                    bad += (l.tail[0] != 0) || !(nb == 1024 || nb % 148 == 0) || nb < 148;
                }
                else if (l.key == "gptb_mriq") ++bad;  // no second kernel in this variant
            CHECK(n1 > 0 && bad == 0 && one.stage2_launches == 0);
        }
        // fused request-driven co-location on the double: layers ride, blocks are counted in both phases
        {
            TaskManager tm6(&vgg, "stencil", "");
            tm6.warmup_passes = 1;
            FusedColocationResult fc = tm6.runFusedColocation(0.05, 2000.0, 1.5, 7, nullptr);
            CHECK(fc.mixable_layers == 16 && fc.fused_layers > 0 && fc.blocks_per_fused_query > 0);
            CHECK(fc.ts_be_blocks > 0 && fc.fu_be_blocks > 0 && fc.fu_be_blocks_in_lc == fc.fu_fused_queries * fc.blocks_per_fused_query);
            CHECK(fc.lc_served > 10 && fc.fu_fused_queries + fc.fu_plain_queries == fc.lc_served);
        }
        // no headroom -> nothing is fused
        tm.qos_budget_ms = 0.001f;
        g_launches.clear();
        ScheduleResult none = tm.executeAllTasks(ExecutionMode::Aker, nullptr);
        fused = 0;
        for (auto& l : g_launches) fused += (l.key == "tzgemm_stencil" || l.key == "tzconv_stencil");
        CHECK(fused == 0 && none.mix_times == 0 && none.be_blocks == 0);
        // request-driven co-location on the double: every arrival is served, the best-effort task advances
        Bert be_task(1, 8, 128);
        TaskManager tm2(&vgg, "stencil", "");
        tm2.warmup_passes = 1;
        ColocationResult co = tm2.runColocation(&be_task, 8, 0.05, 2000.0, 1.5, 7, nullptr);
        CHECK(co.lc_served > 10 && co.be_queries > 0 && co.be_queries % 8 == 0 && co.lc_p99_ms >= co.lc_p50_ms);
        CHECK(fake.captures >= 2 && fake.replays > fake.captures);  // LC pass and BE chunks are replayed as graphs
    }
    CHECK(throws([] { logger.ERROR("boom"); }));
    releaseFusedKernels();
    destroyCreatedKernels();
    tzgemmScratch.release();
    std::printf("host selftest: %d checks, %d failed\n", g_checks, g_failed);
    return g_failed == 0 ? 0 : 1;
}
