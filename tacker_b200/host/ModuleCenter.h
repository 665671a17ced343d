// ModuleCenter.h -- registry of loadable kernel modules (reference: src/ModuleCenter.h, ModuleCenter.cu:8-52,
// where a module is a cubin opened with cuModuleLoad and a function is a CUfunction).  Here a module is a
// shared library that exports C-ABI launchers (libtacker_b200.so itself, or a library emitted by the
// fused-kernel generator); a function is a tk_launch_fn found by symbol name.
#pragma once
#include <map>
#include <string>

#include "tacker_b200.h"

class ModuleCenter {
public:
    ~ModuleCenter();
    // dlopen()s `path` under `moduleName`; returns false (and keeps the old state) when it cannot be opened
    bool registerModule(const std::string& moduleName, const std::string& path);
    bool hasModule(const std::string& moduleName) const;
    // launcher exported as `symbol` by the module, nullptr when absent
    tk_launch_fn getFunction(const std::string& moduleName, const std::string& symbol);
    void* getSymbol(const std::string& moduleName, const std::string& symbol);
    // Name of the launcher a generated module exports: "tk_launch_<kernel name>", where the kernel name is the file
    // name of the module without directory and extension (tzgemm_mriq_1_16.so -> tk_launch_tzgemm_mriq_1_16).
    std::string launcherOf(const std::string& moduleName) const;
    size_t size() const { return modules.size(); }

private:
    std::map<std::string, void*> modules;
    std::map<std::string, std::string> paths;
};

extern ModuleCenter moduleCenter;
