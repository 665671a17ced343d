// Task.h -- a named, ordered list of kernels (reference: src/Task.h:7-37, src/Task.cu:17-63).
#pragma once
#include <string>
#include <vector>

#include "Kernel.h"

enum ExecutionMode { Aker = 0, Tacker };
enum TaskType { LC = 0, BE };

class Task {
public:
    Task(int taskId, std::string taskName) : taskId(taskId), taskName(std::move(taskName)) {}
    explicit Task(int taskId) : taskId(taskId) {}
    virtual ~Task();
    void addKernel(Kernel* kernel) { kernels.emplace_back(kernel); }
    // runs every kernel with per-kernel event timing; in Aker mode the times go to the Recorder
    void executeTask(ExecutionMode mode, stream_t stream);
    void executeTask(ExecutionMode mode, int idx, stream_t stream);
    // runs every kernel back to back without per-kernel synchronisation; returns nothing, times nothing
    void enqueue(stream_t stream);
    // the same through CUDA graphs: kernels [begin, end) are captured once per (range, stream) and replayed
    // afterwards; falls back to plain launches when the backend cannot capture
    void enqueueGraph(stream_t stream) { enqueueGraph(0, kernels.size(), stream); }
    void enqueueGraph(size_t begin, size_t end, stream_t stream);
    void dropGraphs();
    virtual void initExecution() = 0;  // bring the task's input to the device

    int taskId;
    std::string taskName;
    std::vector<Kernel*> kernels;
    TaskType taskType = LC;
    // Stream on which initExecution() queues the upload of the task's input: the stream its kernels run on.
    stream_t execStream = nullptr;
    void* Input[3] = {nullptr, nullptr, nullptr};
    void** Result = nullptr;
    void* InputHost[3] = {nullptr, nullptr, nullptr};
    int InputSize[3] = {0, 0, 0};

private:
    struct CapturedRange {
        size_t begin, end;
        stream_t stream;
        void* graph;
    };
    std::vector<CapturedRange> graphs;
    void* evStart = nullptr;  // created once, destroyed with the task (the reference leaks a pair per call)
    void* evStop = nullptr;
};
