// Host-side seeded streams for synthetic weights and batches (no GPU involved).
// One counter-based generator: word i of stream `key` is splitmix64(key + i*phi),
// so any slice of any stream can be produced independently, by any rank, on any
// number of threads, with the same bits.
#include <cmath>
#include <thread>

#include "common.h"

namespace {

constexpr uint64_t kGolden = 0x9E3779B97F4A7C15ull;

inline uint64_t word(uint64_t key, uint64_t index) {
    uint64_t z = key + index * kGolden + kGolden;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

inline double unit(uint64_t w) { return (double)(w >> 11) * (1.0 / 9007199254740992.0); }  // [0,1), 53 bits

template <class F>
void parallel_for(uint64_t n, F body) {
    unsigned hw = std::thread::hardware_concurrency();
    uint64_t threads = hw ? hw : 4;
    if (threads > 64) threads = 64;
    if (n < (1u << 16)) threads = 1;
    if (threads <= 1) { body(0, n); return; }
    std::vector<std::thread> pool;
    uint64_t per = (n + threads - 1) / threads;
    for (uint64_t t = 0; t < threads; ++t) {
        uint64_t lo = t * per, hi = lo + per < n ? lo + per : n;
        if (lo >= hi) break;
        pool.emplace_back([=] { body(lo, hi); });
    }
    for (auto& th : pool) th.join();
}

}  // namespace

extern "C" int rst_synth_uniform(uint64_t key, uint64_t n, uint64_t offset, double* out) {
    if (n && !out) return rst::fail(nullptr, RST_ERR_INVALID_ARG, "out is NULL");
    parallel_for(n, [=](uint64_t lo, uint64_t hi) {
        for (uint64_t i = lo; i < hi; ++i) out[i] = unit(word(key, offset + i));
    });
    return RST_OK;
}

// Box-Muller: element i uses words 2i and 2i+1 of the stream.
extern "C" int rst_synth_normal(uint64_t key, uint64_t n, uint64_t offset, double mean, double stddev,
                                double* out) {
    if (n && !out) return rst::fail(nullptr, RST_ERR_INVALID_ARG, "out is NULL");
    const double two_pi = 6.283185307179586476925286766559;
    parallel_for(n, [=](uint64_t lo, uint64_t hi) {
        for (uint64_t i = lo; i < hi; ++i) {
            const uint64_t e = offset + i;
            const double u1 = 1.0 - unit(word(key, 2 * e));       // (0, 1]
            const double u2 = unit(word(key, 2 * e + 1));
            out[i] = mean + stddev * (std::sqrt(-2.0 * std::log(u1)) * std::cos(two_pi * u2));
        }
    });
    return RST_OK;
}
