// aker -- command line of the runtime (reference: src/main.cu:246-336).
//   aker -s <aker|tacker> -m <vgg16|resnet50|bert> [-d device] [-c config_dir]
//        [--colocate seconds] [--colocate-fused seconds] [--qps rate] [--qos factor] [--be model] [--be-chunk-ms ms]
//        [--one-cd] [--be-kernel name] [--be-kernel2 name] [--dump-output file]
//        [--mix-module name=path.so]... [--module-dir dir]
// Without --colocate it runs the reference's experiment (both modes unless -s picks one; --one-cd: its variant
// with one best-effort kernel); with --colocate, the request-driven co-location of `-m` (latency-critical) with the
// model `--be` (best-effort) on this GPU; with --colocate-fused, the co-location with the benchmark kernel of the
// configuration as the best-effort job, time-sliced and fused.
#include <fstream>
#include <sstream>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <memory>
#include <string>
#include <vector>

#include "Backend.h"
#include "Creator.h"
#include "Logger.h"
#include "ModuleCenter.h"
#include "Recorder.h"
#include "TaskManager.h"
#include "dnn/models.h"
#include "json.h"
#include "json.h"

static void usage(const char* argv0) {
    std::cout << "SYNOPSIS\n        " << argv0
              << " -s <system_name> -m <model_name> [-d <device_no>] [-c <config_dir>]\n"
                 "            [--colocate <seconds>] [--qps <rate>] [--qos <factor>] [--be <model_name>]\n\n"
                 "OPTIONS\n        -s, --system   system name, aker/tacker\n        -m, --model    model name\n"
                 "        -d, --device   device number\n";
}

int main(int argc, char* argv[]) {
    std::string system_name, model, config_dir = "config", be_model = "bert", be_kernel_a, be_kernel_b, dump_output;
    int device_no = 0;
    double colocate = 0.0, colocate_fused = 0.0, qps = 200.0, qos = 1.5, be_chunk = -1.0, ride_scale = -1.0;
    bool one_cd = false;
    std::vector<std::string> mix_modules;
    std::string module_dir;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto val = [&](const char* what) -> std::string {
            if (i + 1 >= argc) {
                std::cerr << "missing value for " << what << "\n";
                std::exit(2);
            }
            return argv[++i];
        };
        if (a == "-s" || a == "--system") system_name = val("-s");
        else if (a == "-m" || a == "--model") model = val("-m");
        else if (a == "-d" || a == "--device") device_no = std::atoi(val("-d").c_str());
        else if (a == "-c" || a == "--config") config_dir = val("-c");
        else if (a == "--colocate") colocate = std::atof(val("--colocate").c_str());
        else if (a == "--colocate-fused") colocate_fused = std::atof(val("--colocate-fused").c_str());
        else if (a == "--one-cd") one_cd = true;
        else if (a == "--mix-module") mix_modules.push_back(val("--mix-module"));  // <name>=<path to .so>
        else if (a == "--module-dir") module_dir = val("--module-dir");
        else if (a == "--dump-output") dump_output = val("--dump-output");  // raw binary32 result of one LC pass
        else if (a == "--be-kernel") be_kernel_a = val("--be-kernel");    // overrides "throughput_test"."a"
        else if (a == "--be-kernel2") be_kernel_b = val("--be-kernel2");  // overrides "throughput_test"."b"
        else if (a == "--qps") qps = std::atof(val("--qps").c_str());
        else if (a == "--qos") qos = std::atof(val("--qos").c_str());
        else if (a == "--be") be_model = val("--be");
        else if (a == "--be-chunk-ms") be_chunk = std::atof(val("--be-chunk-ms").c_str());
        else if (a == "--ride-scale") ride_scale = std::atof(val("--ride-scale").c_str());
        else {
            usage(argv[0]);
            return 0;
        }
    }
    if (system_name.empty() || model.empty()) {
        usage(argv[0]);
        return 0;
    }
    std::cout << "system: " << system_name << ", model: " << model << std::endl;
    int rc = 0;
    try {
        std::unique_ptr<Backend> be(makeCudaBackend());
        setBackend(be.get());
        // a model description file (GraphTask) names the model whose kernel tables it is scheduled with
        std::string table_model = model;
        if (model.size() > 5 && model.compare(model.size() - 5, 5, ".json") == 0) {
            std::ifstream mf(model);
            std::stringstream ms;
            ms << mf.rdbuf();
            const std::shared_ptr<JsonValue> root = parse_json(ms.str());
            const JsonValue* c = root->get("config");
            table_model = c && c->kind == JsonValue::String ? c->str : std::string("vgg16");
        }
        read_json(config_dir + "/kinfo-" + table_model + ".json");
        read_common_json(config_dir + "/kinfo-common.json");
        // Fused kernels emitted by the generator: registered under a name from the command line (the pair's key, e.g.
        // tzgemm_mriq=/path/tzgemm_mriq_1_16.so, replaces the library's kernel of that pair) or named by the model
        // file ("tzgemm_<cd>": {"module": "tzgemm_<cd>_1_<W>"}) and looked up in the module directory.
        for (const std::string& spec : mix_modules) {
            const size_t eq = spec.find('=');
            if (eq == std::string::npos || !moduleCenter.registerModule(spec.substr(0, eq), spec.substr(eq + 1)))
                throw std::runtime_error("cannot load the module " + spec);
        }
        for (const char* pair : {"tzgemm_stencil", "tzgemm_cp", "tzgemm_mriq", "tzgemm_mrif", "tzgemm_sgemm", "tzgemm_lbm",
                                 "tzgemm_fft", "tzgemm_cutcp"}) {
            const std::string module = sget_kernel_info(pair, "module");
            if (module.empty() || moduleCenter.hasModule(module)) continue;
            std::string dir = module_dir;
            if (dir.empty()) {
                dir = argv[0];
                const size_t slash = dir.find_last_of('/');
                dir = (slash == std::string::npos ? std::string(".") : dir.substr(0, slash)) + "/../fusion/mix_kernel";
            }
            if (!moduleCenter.registerModule(module, dir + "/" + module + ".so"))
                logger.WARNING("model file names the module {" + module + "}, which is not in " + dir +
                               " (python -m tacker_b200.fusion.gen_run builds it); the library kernel is used");
        }
        be->setDevice(device_no);  // no device reset: the GPU may be shared (the reference calls cudaDeviceReset)
        std::cout << "SM count: " << be->smCount() << std::endl;
        stream_t streams[2] = {be->streamCreate(), be->streamCreate()};

        std::unique_ptr<Task> lc_task(createTask(model));
        for (int i = 0; i < 5; ++i) {  // warm-up (src/main.cu:290-297)
            lc_task->initExecution();
            lc_task->enqueue(streams[0]);
            be->streamSync(streams[0]);
        }
        if (!dump_output.empty()) {
            auto* dnn = dynamic_cast<DnnTask*>(lc_task.get());
            lc_task->execStream = streams[0];
            lc_task->initExecution();
            lc_task->enqueue(streams[0]);
            const std::vector<float> out = dnn ? dnn->downloadResult(streams[0]) : std::vector<float>();
            FILE* f = std::fopen(dump_output.c_str(), "wb");
            if (!f || std::fwrite(out.data(), sizeof(float), out.size(), f) != out.size())
                throw std::runtime_error("cannot write " + dump_output);
            std::fclose(f);
            std::printf("[Result] wrote %zu floats of the %s result to %s\n", out.size(), model.c_str(), dump_output.c_str());
        }
        const std::string a = be_kernel_a.empty() ? sget_kernel_info("throughput_test", "a") : be_kernel_a;
        const std::string b = be_kernel_b.empty() ? sget_kernel_info("throughput_test", "b") : be_kernel_b;
        std::printf("[Result] cd1: %s, cd2: %s, dnn: %s\n", a.c_str(), b.c_str(), model.c_str());
        TaskManager taskManager(lc_task.get(), a, b);
        if (be_chunk >= 0.0) taskManager.be_chunk_ms = be_chunk;
        if (ride_scale > 0.0) taskManager.ride_scale = static_cast<float>(ride_scale);
        if (colocate > 0.0) {
            std::unique_ptr<Task> be_task(createTask(be_model));
            const int per_pass = be_model == "bert" ? static_cast<Bert*>(be_task.get())->batch : 1;
            ColocationResult r = taskManager.runColocation(be_task.get(), per_pass, colocate, qps, qos,
                                                           1000 + static_cast<uint64_t>(device_no), streams[0]);
            std::printf("{\"device\": %d, \"lc\": \"%s\", \"be\": \"%s\", \"seconds\": %.3f, \"qps_offered\": %.1f, "
                        "\"lc_served\": %lld, \"lc_solo_p50_ms\": %.4f, \"lc_solo_p99_ms\": %.4f, \"lc_p50_ms\": %.4f, "
                        "\"lc_p99_ms\": %.4f, \"qos_bound_ms\": %.4f, \"qos_met\": %s, \"be_queries\": %lld, "
                        "\"be_qps\": %.2f}\n",
                        device_no, model.c_str(), be_model.c_str(), r.seconds, qps, r.lc_served, r.lc_solo_p50_ms,
                        r.lc_solo_p99_ms, r.lc_p50_ms, r.lc_p99_ms, r.qos_bound_ms, r.qos_met ? "true" : "false",
                        r.be_queries, r.be_qps);
        } else if (colocate_fused > 0.0) {
            FusedColocationResult r = taskManager.runFusedColocation(colocate_fused, qps, qos, 1000 + static_cast<uint64_t>(device_no),
                                                                     streams[0]);
            std::printf("{\"device\": %d, \"lc\": \"%s\", \"be_kernel\": \"%s\", \"be_blocks_per_job\": %d, \"seconds\": %.3f, "
                        "\"qps_offered\": %.1f, \"lc_served\": %lld, \"lc_solo_p50_ms\": %.4f, \"lc_solo_p99_ms\": %.4f, "
                        "\"qos_bound_ms\": %.4f, \"mixable_layers\": %d, \"fused_layers\": %d, \"blocks_per_fused_query\": %lld, "
                        "\"lc_graph_ms\": %.4f, \"lc_fused_graph_ms\": %.4f, "
                        "\"timesliced\": {\"lc_p50_ms\": %.4f, \"lc_p99_ms\": %.4f, \"qos_met\": %s, \"be_blocks\": %lld, "
                        "\"be_blocks_per_s\": %.1f}, "
                        "\"fused\": {\"lc_p50_ms\": %.4f, \"lc_p99_ms\": %.4f, \"qos_met\": %s, \"be_blocks\": %lld, "
                        "\"be_blocks_in_lc\": %lld, \"fused_queries\": %lld, \"plain_queries\": %lld, \"be_blocks_per_s\": %.1f}}\n",
                        device_no, model.c_str(), r.be_kernel.c_str(), r.be_blocks_per_job, r.seconds, qps, r.lc_served,
                        r.lc_solo_p50_ms, r.lc_solo_p99_ms, r.qos_bound_ms, r.mixable_layers, r.fused_layers,
                        r.blocks_per_fused_query, r.lc_graph_ms, r.lc_fused_graph_ms, r.ts_lc_p50_ms, r.ts_lc_p99_ms,
                        r.ts_qos_met ? "true" : "false", r.ts_be_blocks, r.ts_be_blocks_per_s, r.fu_lc_p50_ms, r.fu_lc_p99_ms,
                        r.fu_qos_met ? "true" : "false", r.fu_be_blocks, r.fu_be_blocks_in_lc, r.fu_fused_queries,
                        r.fu_plain_queries, r.fu_be_blocks_per_s);
        } else if (one_cd) {
            if (system_name == "aker" || system_name == "both") taskManager.execute_with_one_cd_kernel(ExecutionMode::Aker, streams[0]);
            if (system_name == "tacker" || system_name == "both") taskManager.execute_with_one_cd_kernel(ExecutionMode::Tacker, streams[1]);
        } else {
            if (system_name == "aker" || system_name == "both") taskManager.executeAllTasks(ExecutionMode::Aker, streams[0]);
            if (system_name == "tacker" || system_name == "both") taskManager.executeAllTasks(ExecutionMode::Tacker, streams[1]);
        }
        if (generatedLaunchers > 0)
            std::printf("[Result] fused kernels launched through generated modules: %d\n", generatedLaunchers);
        const unsigned status = be->deviceStatus();
        if (status != 0) logger.WARNING("device status word: " + std::to_string(status));
        recorder.text();
        releaseFusedKernels();
        lc_task.reset();
        destroyCreatedKernels();
        tzgemmScratch.release();
    } catch (const std::exception& e) {
        std::cerr << "[ERROR] " << e.what() << std::endl;
        rc = 1;
    }
    return rc;
}
