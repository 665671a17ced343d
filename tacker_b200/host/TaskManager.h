// TaskManager.h -- QoS-aware co-location of a latency-critical task with best-effort kernels
// (reference: src/TaskManager.h, src/TaskManager.cu:92-123, 125-400, 413-714).
#pragma once
#include <string>
#include <vector>

#include "Creator.h"
#include "Task.h"
#include "dnn/layers.h"

// {M, N, K} of the GEMM a convolution becomes (src/TaskManager.cu:92-123)
std::vector<int> get_mnk_from_cudnn_args(std::vector<int>& cudnn_args);

// One LC layer fused with best-effort blocks [cd_start_blk, cd_end_blk) of a CUDA-core kernel: the layer's
// operand preparation, then one MixKernel launch "tzgemm_<cd>" (src/TaskManager.cu:125-306, 309-400).
// The MixKernel is cached per (layer, pair) instead of being rebuilt and leaked on every call.
void mixcudnnConvolutionForward(TzLayer* layer, GPTBKernel* gptb_cd_kernel, int cd_start_blk, int cd_end_blk,
                                stream_t stream);
void mixcublasSgemm(TzLayer* layer, GPTBKernel* gptb_cd_kernel, int cd_start_blk, int cd_end_blk, stream_t stream);

// how many cached fused kernels launch through a generated module instead of the library's kernel
extern int generatedLaunchers;

// forget the cached fused kernels (call before destroying the tasks or the best-effort kernels they were built from)
void releaseFusedKernels();

struct ScheduleResult {
    float lc_solo_ms = 0;        // sum of the profiled solo kernel times
    float lc_colocated_ms = 0;   // LC time of the last scheduling pass
    float qos_headroom_left = 0;
    long long be_blocks = 0;     // best-effort virtual blocks executed inside the LC task
    int mix_times = 0, mixable_times = 0;
    float time_earned = 0;       // ms saved against running the same work unfused
    float be1_ms = 0, be2_ms = 0;  // solo time of one full launch of each best-effort kernel
    float stage1_be_ms = 0, stage2_be_ms = 0;   // stage 2: device time of the solo launches that ran in the leftover budget
    int stage2_launches = 0;
    long long stage2_blocks1 = 0, stage2_blocks2 = 0;  // virtual blocks of each best-effort kernel run in stage 2
};

struct ColocationResult {
    double seconds = 0;
    long long lc_served = 0, be_queries = 0;
    double lc_p50_ms = 0, lc_p99_ms = 0, lc_solo_p50_ms = 0, lc_solo_p99_ms = 0;
    double be_qps = 0, qos_bound_ms = 0;
    bool qos_met = false;
};

// Request-driven co-location with a benchmark kernel as the best-effort job, run twice under the same arrivals:
// time-sliced (best-effort blocks only while no query is in flight) and fused (the same, plus best-effort blocks
// riding inside the LC layers' fused kernels whenever the query's latency budget allows it).
struct FusedColocationResult {
    double seconds = 0, qos_bound_ms = 0, lc_solo_p50_ms = 0, lc_solo_p99_ms = 0;
    long long lc_served = 0;
    std::string be_kernel;
    int be_blocks_per_job = 0;
    int fused_layers = 0, mixable_layers = 0;   // layers whose fused launch paid off when measured / layers that could be fused
    long long blocks_per_fused_query = 0;       // best-effort blocks one fused LC pass carries
    double lc_graph_ms = 0, lc_fused_graph_ms = 0;  // one LC pass alone: plain and fused
    // time-sliced phase
    double ts_lc_p50_ms = 0, ts_lc_p99_ms = 0, ts_be_blocks_per_s = 0;
    long long ts_be_blocks = 0;
    bool ts_qos_met = false;
    // fused phase
    double fu_lc_p50_ms = 0, fu_lc_p99_ms = 0, fu_be_blocks_per_s = 0;
    long long fu_be_blocks = 0, fu_be_blocks_in_lc = 0, fu_fused_queries = 0, fu_plain_queries = 0;
    bool fu_qos_met = false;
};

class TaskManager {
public:
    TaskManager(Task* lc_task, const std::string& be_task1_name, const std::string& be_task2_name);
    ~TaskManager() { releaseFusedKernels(); }  // they point into lc_task's layers
    // The reference's experiment: profile the LC task kernel by kernel, then walk it under a latency budget and
    // fuse every mixable layer that still has headroom with best-effort blocks.
    //   Tacker: all blocks of the best-effort kernel with every layer;
    //   Aker:   tiles x block_ratio[K] blocks (JSON "tzgemm_<be>"."<K_GLOBAL>", scaled from "4096" when absent).
    ScheduleResult executeAllTasks(ExecutionMode mode, stream_t stream);
    // The variant with one best-effort kernel (src/TaskManager.cu:717-1005): every fused launch takes the first
    // tiles x block_ratio[K] blocks, rounded to whole rounds of the SM count; no second kernel, no stage 2.
    ScheduleResult execute_with_one_cd_kernel(ExecutionMode mode, stream_t stream);
    // Request-driven co-location: LC queries arrive as a Poisson process of rate `qps`; between queries the GPU
    // runs the best-effort task kernel by kernel.  QoS: p99 <= qos_factor x solo p99.  `be_queries_per_pass` =
    // queries one pass over the best-effort task completes (its batch size).
    ColocationResult runColocation(Task* be_task, int be_queries_per_pass, double seconds, double qps,
                                   double qos_factor, uint64_t seed, stream_t stream);

    // The reference's co-location (src/TaskManager.cu:569-656: best-effort blocks inside the LC layers) under
    // request-driven load: best-effort job = the benchmark kernel `be_task1_name`, measured against time slicing.
    FusedColocationResult runFusedColocation(double seconds, double qps, double qos_factor, uint64_t seed, stream_t stream);

    Task* lc_task;
    std::string be_task1_name, be_task2_name;
    float qos_budget_ms = 50.0f;  // src/TaskManager.cu:571
    float qos_guard_ms = 4.0f;    // src/TaskManager.cu:586
    int profile_passes = 10, schedule_passes = 5, warmup_passes = 5;
    float ride_scale = 1.0f;    // fused co-location: a layer carries best-effort blocks worth this many layer times
    double be_chunk_ms = 0.15;  // best-effort work enqueued at once while idle (bounds the extra LC wait)

private:
    ScheduleResult schedule(ExecutionMode mode, stream_t stream, bool one_cd);
    float blockRatio(const std::string& pair, int k_global);
    float timedBlocks(GPTBKernel* kernel, int start, int end, stream_t stream);
};
