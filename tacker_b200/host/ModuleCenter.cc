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
    paths[moduleName] = path;
    return true;
}

bool ModuleCenter::hasModule(const std::string& moduleName) const { return modules.count(moduleName) != 0; }

tk_launch_fn ModuleCenter::getFunction(const std::string& moduleName, const std::string& symbol) {
    auto it = modules.find(moduleName);
    if (it == modules.end()) return nullptr;
    return reinterpret_cast<tk_launch_fn>(dlsym(it->second, symbol.c_str()));
}

void* ModuleCenter::getSymbol(const std::string& moduleName, const std::string& symbol) {
    auto it = modules.find(moduleName);
    if (it == modules.end()) return nullptr;
    return dlsym(it->second, symbol.c_str());
}

std::string ModuleCenter::launcherOf(const std::string& moduleName) const {
    auto it = paths.find(moduleName);
    std::string file = it == paths.end() ? moduleName : it->second;
    const size_t slash = file.find_last_of('/');
    if (slash != std::string::npos) file = file.substr(slash + 1);
    const size_t dot = file.find_last_of('.');
    if (dot != std::string::npos) file = file.substr(0, dot);
    if (file.compare(0, 3, "lib") == 0) file = file.substr(3);
    return "tk_launch_" + file;
}
