#include "Recorder.h"

#include <fstream>
#include <iostream>

Recorder recorder;

float Recorder::taskTime(int taskId) const {
    auto it = task_time_map.find(taskId);
    float total = 0.0f;
    if (it != task_time_map.end())
        for (float t : it->second) total += t;
    return total;
}

size_t Recorder::text(const std::string& filename) {
    std::ofstream file(filename);
    if (!file.is_open()) {
        std::cerr << "cannot open file: " << filename << std::endl;
        return 0;
    }
    size_t n = 0;
    for (auto& task_pair : task_time_map) {
        const int taskId = task_pair.first;
        auto& times = task_pair.second;
        auto& kernelIds = task_kernel_map[taskId];
        file << "taskID: " << taskId << ", taskName: " << task_name_map[taskId] << "\n";
        float total = 0.0f;
        for (size_t i = 0; i < times.size(); ++i, ++n) {
            total += times[i];
            file << "    kernelID: " << kernelIds[i] << ", kernelName: " << task_kernel_name_vec[taskId][i]
                 << ", execTime: " << times[i] << "ms\n";
        }
        file << "    task running time: " << total << "ms\n\n";
    }
    return n;
}
