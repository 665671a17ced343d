// util.h -- small helpers shared by the host runtime (reference: src/util.h:25-84).
// The reference aborts or throws from its CUDA_SAFE_CALL macros; here every failure becomes a
// std::runtime_error that the CLI reports, so that library users never lose the process.
#pragma once
#include <cstdint>
#include <sstream>
#include <stdexcept>
#include <string>

struct dim3h {  // host-side stand-in for dim3: the host is plain C++ and includes no CUDA header
    unsigned x, y, z;
    dim3h(unsigned x_ = 1, unsigned y_ = 1, unsigned z_ = 1) : x(x_), y(y_), z(z_) {}
};

typedef void* stream_t;  // cudaStream_t travels as an opaque pointer

#define TK_HOST_CHECK(expr)                                                                  \
    do {                                                                                     \
        int _rc = (expr);                                                                    \
        if (_rc != 0) {                                                                      \
            std::ostringstream _s;                                                           \
            _s << "error: " #expr " failed with status " << _rc << " (" << __FILE__ << ":" << __LINE__ << ")"; \
            throw std::runtime_error(_s.str());                                              \
        }                                                                                    \
    } while (0)

// counter-based SplitMix64 draws in [0, 1): the same generator the test-suite's inputs use
inline float tk_unit_draw(uint64_t seed, uint64_t i) {
    uint64_t z = seed * 0xD1342543DE82EF95ull + i + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return static_cast<float>(z >> 40) * (1.0f / 16777216.0f);
}
