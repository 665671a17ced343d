// Recorder.h -- what ran and how long it took, per task; dumped as text when the run ends
// (the role of the reference's Recorder: src/Recorder.h:7-27, src/Recorder.cc:12-44).
#pragma once
#include <map>
#include <string>
#include <vector>

class Recorder {
public:
    struct KernelRecord {
        int kernelId;
        std::string kernelName;
        float ms;
    };
    void recordKernel(int taskId, int kernelId, const std::string& kernelName, float executionTime) {
        tasks[taskId].kernels.push_back(KernelRecord{kernelId, kernelName, executionTime});
    }
    void recordTask(int taskId, const std::string& taskName) { tasks[taskId].name = taskName; }
    // One block per task: a header line, one line per kernel record, the task's total.  Returns the number of
    // kernel records written.
    size_t text(const std::string& filename = "recorder_output.txt");
    float taskTime(int taskId) const;

private:
    struct TaskRecord {
        std::string name;
        std::vector<KernelRecord> kernels;
    };
    std::map<int, TaskRecord> tasks;  // ordered by task id, so the dump is stable
};

extern Recorder recorder;
