#include "Task.h"

#include "Logger.h"
#include "Recorder.h"

Task::~Task() {
    dropGraphs();
    if (evStart) backend().eventDestroy(evStart);
    if (evStop) backend().eventDestroy(evStop);
    logger.DEBUG("task name: " + taskName + ", id: " + std::to_string(taskId) + " is destroyed!");
}

void Task::executeTask(ExecutionMode mode, stream_t stream) {
    for (size_t i = 0; i < kernels.size(); ++i) executeTask(mode, static_cast<int>(i), stream);
    if (mode == ExecutionMode::Aker) recorder.recordTask(taskId, taskName);
}

void Task::executeTask(ExecutionMode mode, int idx, stream_t stream) {
    if (!evStart) {
        evStart = backend().eventCreate();
        evStop = backend().eventCreate();
    }
    Kernel* kernel = kernels.at(static_cast<size_t>(idx));
    logger.DEBUG("kernel name: " + kernel->kernelName + ", id: " + std::to_string(kernel->Id) + " is executing ...");
    backend().eventRecord(evStart, stream);  // on the kernel's stream (the reference records on stream 0)
    kernel->execute(stream);
    backend().eventRecord(evStop, stream);
    const float kernel_time = backend().eventElapsedMs(evStart, evStop);
    if (mode == ExecutionMode::Aker) recorder.recordKernel(taskId, kernel->Id, kernel->kernelName, kernel_time);
}

void Task::enqueue(stream_t stream) {
    for (auto& kernel : kernels) kernel->execute(stream);
}

void Task::enqueueGraph(size_t begin, size_t end, stream_t stream) {
    for (auto& g : graphs)
        if (g.begin == begin && g.end == end && g.stream == stream) {
            if (g.graph) backend().graphLaunch(g.graph, stream);
            else
                for (size_t k = begin; k < end; ++k) kernels[k]->execute(stream);
            return;
        }
    // first use: one plain pass (lazy set-up inside the library must not happen during capture), then capture
    for (size_t k = begin; k < end; ++k) kernels[k]->execute(stream);
    backend().streamSync(stream);
    void* graph = backend().graphCapture(stream, [this, begin, end, stream] {
        for (size_t k = begin; k < end; ++k) kernels[k]->execute(stream);
    });
    graphs.push_back(CapturedRange{begin, end, stream, graph});  // this call's work was done by the plain pass
}

void Task::dropGraphs() {
    for (auto& g : graphs)
        if (g.graph) backend().graphDestroy(g.graph);
    graphs.clear();
}
