#include "Backend.h"

#include <stdexcept>

namespace {
Backend* g_backend = nullptr;
}

Backend& backend() {
    if (!g_backend) throw std::runtime_error("no backend installed: call setBackend(makeCudaBackend()) first");
    return *g_backend;
}

void setBackend(Backend* b) { g_backend = b; }
