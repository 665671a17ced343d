#include "ModuleCenter.h"

#include <dlfcn.h>

#include "Logger.h"

ModuleCenter moduleCenter;

ModuleCenter::~ModuleCenter() {
    for (auto& m : modules)
        if (m.second) dlclose(m.second);
}

bool ModuleCenter::registerModule(const std::string& moduleName, const std::string& path) {
    void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) {
        logger.WARNING("module {" + moduleName + "}: cannot open " + path + ": " + dlerror());
        return false;
    }
    auto it = modules.find(moduleName);
    if (it != modules.end() && it->second) dlclose(it->second);
    modules[moduleName] = h;
    return true;
}

bool ModuleCenter::hasModule(const std::string& moduleName) const { return modules.count(moduleName) != 0; }

tk_launch_fn ModuleCenter::getFunction(const std::string& moduleName, const std::string& symbol) {
    auto it = modules.find(moduleName);
    if (it == modules.end()) return nullptr;
    return reinterpret_cast<tk_launch_fn>(dlsym(it->second, symbol.c_str()));
}
