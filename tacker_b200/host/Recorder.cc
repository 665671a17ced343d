#include "Recorder.h"

#include <fstream>
#include <iostream>

Recorder recorder;

float Recorder::taskTime(int taskId) const {
    const auto it = tasks.find(taskId);
    if (it == tasks.end()) return 0.0f;
    float total = 0.0f;
    for (const KernelRecord& k : it->second.kernels) total += k.ms;
    return total;
}

size_t Recorder::text(const std::string& filename) {
    std::ofstream file(filename);
    if (!file) {
        std::cerr << "cannot open file: " << filename << std::endl;
        return 0;
    }
    size_t written = 0;
    for (const auto& entry : tasks) {
        const TaskRecord& task = entry.second;
        file << "taskID: " << entry.first << ", taskName: " << task.name << "\n";
        for (const KernelRecord& k : task.kernels) {
            file << "    kernelID: " << k.kernelId << ", kernelName: " << k.kernelName << ", execTime: " << k.ms << "ms\n";
            ++written;
        }
        file << "    task running time: " << taskTime(entry.first) << "ms\n\n";
    }
    return written;
}
