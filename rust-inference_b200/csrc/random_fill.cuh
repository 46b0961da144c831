// Random weights as a function of (key, element index): the same value, bit for bit, from the host
// (host_random.cpp) and from the device (random_fill.cu), in any order and for any subset of a tensor.
//
// The key is made by the caller from the seed and the tensor's name.  Element i takes 64 bits
//     h = mix64(key + (i + 1) * 0x9E3779B97F4A7C15)        (the splitmix64 finalizer)
// and turns them into
//   * a normal deviate by Box-Muller: u1 = (h >> 32 + 1/2) / 2^32 in (0, 1), u2 = (h & 2^32-1) / 2^32,
//     z = sqrt(-2 ln u1) cos(2 pi u2), value = float(z * std);
//   * a uniform deviate: u = (h >> 40) / 2^24 in [0, 1), value = float(mid + (u * width - width / 2)).
// ln and cos are evaluated here from their series with additions, multiplications, one division and
// one square root of IEEE double precision, each rounded on its own (no fused multiply-add, no
// library function), so that every machine gets the same bits: ln through the exponent and
// 2 atanh((m - 1) / (m + 1)) with m in [sqrt(1/2), sqrt(2)), cos through the quadrant (exact, from
// the top bits of u2) and the Taylor series of sin and cos on [0, pi/4].
//
// The distributions are the ones of thanhauco/rust-inference's scripts/synthetic_checkpoint.py:135-152
// (matrices and the embedding N(0, 0.02)); norm gains are 1 + U(-0.1, 0.1).
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDA_ARCH__)
#define RF_FN __device__ __forceinline__
#define RF_ADD(a, b) __dadd_rn((a), (b))
#define RF_MUL(a, b) __dmul_rn((a), (b))
#define RF_DIV(a, b) __ddiv_rn((a), (b))
#define RF_SQRT(a) __dsqrt_rn(a)
#define RF_BITS(x) ((uint64_t)__double_as_longlong(x))
#define RF_FROM_BITS(b) __longlong_as_double((long long)(b))
#else
#include <math.h>
#define RF_FN static inline
// the host file is compiled with -ffp-contract=off: every operation below is rounded on its own
#define RF_ADD(a, b) ((a) + (b))
#define RF_MUL(a, b) ((a) * (b))
#define RF_DIV(a, b) ((a) / (b))
#define RF_SQRT(a) sqrt(a)
static inline uint64_t rf_bits_(double x) { uint64_t b; memcpy(&b, &x, 8); return b; }
static inline double rf_from_bits_(uint64_t b) { double x; memcpy(&x, &b, 8); return x; }
#define RF_BITS(x) rf_bits_(x)
#define RF_FROM_BITS(b) rf_from_bits_(b)
#endif

RF_FN uint64_t rf_mix64(uint64_t z) {
    z ^= z >> 30;
    z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27;
    z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

RF_FN uint64_t rf_element_bits(uint64_t key, uint64_t index) { return rf_mix64(key + (index + 1) * 0x9E3779B97F4A7C15ull); }

// ln x for a normal double x in (0, 1]
RF_FN double rf_ln(double x) {
    uint64_t b = RF_BITS(x);
    int e = (int)((b >> 52) & 0x7ff) - 1022;                                      // x = m 2^e, m in [1/2, 1)
    double m = RF_FROM_BITS((b & 0x000fffffffffffffull) | 0x3fe0000000000000ull);
    if (m < 0.70710678118654752) {
        m = RF_MUL(m, 2.0);
        e -= 1;
    }
    const double z = RF_DIV(RF_ADD(m, -1.0), RF_ADD(m, 1.0));
    const double z2 = RF_MUL(z, z);
    // 2 atanh z = z (2 + z^2 (2/3 + z^2 (2/5 + ... + z^2 2/21)))
    double s = 2.0 / 21.0;
    s = RF_ADD(RF_MUL(s, z2), 2.0 / 19.0);
    s = RF_ADD(RF_MUL(s, z2), 2.0 / 17.0);
    s = RF_ADD(RF_MUL(s, z2), 2.0 / 15.0);
    s = RF_ADD(RF_MUL(s, z2), 2.0 / 13.0);
    s = RF_ADD(RF_MUL(s, z2), 2.0 / 11.0);
    s = RF_ADD(RF_MUL(s, z2), 2.0 / 9.0);
    s = RF_ADD(RF_MUL(s, z2), 2.0 / 7.0);
    s = RF_ADD(RF_MUL(s, z2), 2.0 / 5.0);
    s = RF_ADD(RF_MUL(s, z2), 2.0 / 3.0);
    s = RF_ADD(RF_MUL(s, z2), 2.0);
    return RF_ADD(RF_MUL((double)e, 0.69314718055994531), RF_MUL(s, z));
}

// cos(2 pi k / 2^32)
RF_FN double rf_cos_turn(uint32_t k) {
    const uint32_t quadrant = k >> 30;
    uint32_t f = k & 0x3fffffffu;                          // the angle inside the quadrant, in units of (pi/2) / 2^30
    const bool mirror = f > 0x20000000u;                   // past pi/4: take the complement, swap sin and cos
    if (mirror) f = 0x40000000u - f;
    const double x = RF_MUL((double)f, 1.5707963267948966 / 1073741824.0);      // in [0, pi/4]
    const double x2 = RF_MUL(x, x);
    double c = 1.0 / 20922789888000.0;                     // 1/16!
    c = RF_ADD(RF_MUL(c, x2), -1.0 / 87178291200.0);       // 1/14!
    c = RF_ADD(RF_MUL(c, x2), 1.0 / 479001600.0);          // 1/12!
    c = RF_ADD(RF_MUL(c, x2), -1.0 / 3628800.0);           // 1/10!
    c = RF_ADD(RF_MUL(c, x2), 1.0 / 40320.0);              // 1/8!
    c = RF_ADD(RF_MUL(c, x2), -1.0 / 720.0);
    c = RF_ADD(RF_MUL(c, x2), 1.0 / 24.0);
    c = RF_ADD(RF_MUL(c, x2), -0.5);
    c = RF_ADD(RF_MUL(c, x2), 1.0);
    double s = 1.0 / 355687428096000.0;                    // 1/17!
    s = RF_ADD(RF_MUL(s, x2), -1.0 / 1307674368000.0);     // 1/15!
    s = RF_ADD(RF_MUL(s, x2), 1.0 / 6227020800.0);         // 1/13!
    s = RF_ADD(RF_MUL(s, x2), -1.0 / 39916800.0);          // 1/11!
    s = RF_ADD(RF_MUL(s, x2), 1.0 / 362880.0);             // 1/9!
    s = RF_ADD(RF_MUL(s, x2), -1.0 / 5040.0);
    s = RF_ADD(RF_MUL(s, x2), 1.0 / 120.0);
    s = RF_ADD(RF_MUL(s, x2), -1.0 / 6.0);
    s = RF_ADD(RF_MUL(s, x2), 1.0);
    s = RF_MUL(s, x);
    const double cos_a = mirror ? s : c, sin_a = mirror ? c : s;     // of the angle inside the quadrant
    switch (quadrant) {
        case 0: return cos_a;
        case 1: return -sin_a;
        case 2: return -cos_a;
        default: return sin_a;
    }
}

// N(0, std) for element `index` of the tensor with this key
RF_FN float rf_normal(uint64_t key, uint64_t index, double std) {
    const uint64_t h = rf_element_bits(key, index);
    const double u1 = RF_MUL(RF_ADD((double)(uint32_t)(h >> 32), 0.5), 1.0 / 4294967296.0);
    const double r = RF_SQRT(RF_MUL(-2.0, rf_ln(u1)));
    return (float)RF_MUL(RF_MUL(r, rf_cos_turn((uint32_t)h)), std);
}

// mid + U(-width/2, width/2)
RF_FN float rf_uniform(uint64_t key, uint64_t index, double mid, double width) {
    const uint64_t h = rf_element_bits(key, index);
    const double u = RF_MUL((double)(uint32_t)(h >> 40), 1.0 / 16777216.0);
    return (float)RF_ADD(mid, RF_ADD(RF_MUL(u, width), RF_MUL(width, -0.5)));
}
