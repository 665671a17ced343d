#include "Task.h"

#include "Logger.h"
#include "Recorder.h"

Task::~Task() {
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
