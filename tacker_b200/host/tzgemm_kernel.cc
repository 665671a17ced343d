#include "tzgemm_kernel.h"

#include <cstdint>
#include <vector>

TZGEMMScratch tzgemmScratch;

namespace {
// fp32 -> fp16 bits, round to nearest even (values here are in [-1, 1): normal halves or zero)
uint16_t to_half_bits(float f) {
    uint32_t x;
    static_assert(sizeof(x) == sizeof(f), "float is 32 bits");
    __builtin_memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u, absx = x & 0x7fffffffu;
    if (absx < 0x38800000u) {  // below the smallest normal half
        if (absx < 0x33000000u) return static_cast<uint16_t>(sign);
        const uint32_t e = absx >> 23, m = (absx & 0x7fffffu) | 0x800000u, shift = 126u - e;
        uint32_t h = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1u), mid = 1u << (shift - 1u);
        if (rem > mid || (rem == mid && (h & 1u))) ++h;
        return static_cast<uint16_t>(sign | h);
    }
    uint32_t h = (((absx >> 23) - 112u) << 10) | ((absx & 0x7fffffu) >> 13);
    const uint32_t rem = absx & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
    return static_cast<uint16_t>(sign | h);
}

void* seeded_half(long long bytes, uint64_t seed) {
    const size_t n = static_cast<size_t>(bytes / 2);
    std::vector<uint16_t> h(n);
    for (size_t i = 0; i < n; ++i) h[i] = to_half_bits(tk_unit_draw(seed, i) * 2.0f - 1.0f);
    void* d = backend().deviceAlloc(static_cast<size_t>(bytes));
    backend().upload(d, h.data(), n * 2, nullptr);
    backend().streamSync(nullptr);
    return d;
}
}  // namespace

void TZGEMMScratch::reserve(long long a_bytes, long long b_bytes, long long c_bytes) {
    if (a_bytes > bytesA) {
        backend().deviceFree(A);
        A = seeded_half(a_bytes, 1337);
        bytesA = a_bytes;
    }
    if (b_bytes > bytesB) {
        backend().deviceFree(B);
        B = seeded_half(b_bytes, 1338);
        bytesB = b_bytes;
    }
    if (c_bytes > bytesC) {
        backend().deviceFree(C);
        C = static_cast<float*>(backend().deviceAlloc(static_cast<size_t>(c_bytes)));
        backend().fillZero(C, static_cast<size_t>(c_bytes), nullptr);
        backend().streamSync(nullptr);
        bytesC = c_bytes;
    }
}

void TZGEMMScratch::release() {
    backend().deviceFree(A);
    backend().deviceFree(B);
    backend().deviceFree(C);
    A = B = nullptr;
    C = nullptr;
    bytesA = bytesB = bytesC = 0;
}
