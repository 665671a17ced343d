// Recorder.h -- per-task kernel ids / names / times, written out at exit
// (reference: src/Recorder.h:7-27, src/Recorder.cc:12-44).
#pragma once
#include <map>
#include <string>
#include <vector>

class Recorder {
public:
    void recordKernel(int taskId, int kernelId, const std::string& kernelName, float executionTime) {
        task_time_map[taskId].push_back(executionTime);
        task_kernel_map[taskId].push_back(kernelId);
        task_kernel_name_vec[taskId].push_back(kernelName);
    }
    void recordTask(int taskId, const std::string& taskName) { task_name_map[taskId] = taskName; }
    // writes recorder_output.txt-style text; returns the number of kernel records written
    size_t text(const std::string& filename = "recorder_output.txt");
    float taskTime(int taskId) const;

private:
    std::map<int, std::vector<float>> task_time_map;
    std::map<int, std::vector<int>> task_kernel_map;
    std::map<int, std::vector<std::string>> task_kernel_name_vec;
    std::map<int, std::string> task_name_map;
};

extern Recorder recorder;
