// The random values of random_fill.cuh computed on the host, for model folders written by the
// random-weights mode and for whoever wants a tensor (or a few rows of one) without a GPU.
// Compiled with -ffp-contract=off (the values must not depend on fused multiply-adds).
#include "random_fill.cuh"

#include <stdio.h>
#include <algorithm>
#include <thread>
#include <vector>

static thread_local char ri_errbuf[256];
extern "C" const char* ri_last_error() { return ri_errbuf; }

static inline uint16_t bf16_bits(float f) {          // round to nearest even; the values here are finite
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

// out[i] = value of element first + i, i < count.  kind 0: N(0, a); kind 1: a + U(-b/2, b/2).
// dtype 0: float32, 1: bfloat16.
extern "C" int ri_random_fill_host(void* out, unsigned long long key, unsigned long long first, unsigned long long count,
                                   int kind, double a, double b, int dtype, int threads) {
    if (count == 0) return 0;
    if (!out || (kind != 0 && kind != 1) || (dtype != 0 && dtype != 1)) {
        snprintf(ri_errbuf, sizeof(ri_errbuf), "random_fill_host: bad arguments (kind %d, dtype %d)", kind, dtype);
        return -1;
    }
    auto work = [=](unsigned long long lo, unsigned long long hi) {
        for (unsigned long long i = lo; i < hi; i++) {
            const float v = kind == 0 ? rf_normal(key, first + i, a) : rf_uniform(key, first + i, a, b);
            if (dtype == 0) ((float*)out)[i] = v;
            else ((uint16_t*)out)[i] = bf16_bits(v);
        }
    };
    unsigned n = threads > 0 ? (unsigned)threads : std::max(1u, std::thread::hardware_concurrency());
    n = (unsigned)std::min<unsigned long long>(n, (count + 65535) / 65536);
    if (n <= 1) {
        work(0, count);
        return 0;
    }
    std::vector<std::thread> pool;
    const unsigned long long per = (count + n - 1) / n;
    for (unsigned t = 0; t < n; t++) {
        const unsigned long long lo = t * per, hi = std::min(count, lo + per);
        if (lo < hi) pool.emplace_back(work, lo, hi);
    }
    for (auto& t : pool) t.join();
    return 0;
}
