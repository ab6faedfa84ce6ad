// The random numbers of random-weights models, defined bit by bit so that the device fill kernel
// (utility.cu), the host code that writes model folders, and the numpy twin of the tests
// (tests/random_twin.py) produce the same tensors from the same seed.
//
//   key(seed, name)   = fnv1a64(name) ^ (seed * 0x9E3779B97F4A7C15)             (64-bit wrap-around)
//   base              = fin(key + G),  G = 0x9E3779B97F4A7C15, fin = the splitmix64 finaliser
//   r_j(i)            = fin(base + (3 i + j + 1) G),  j = 0, 1, 2                  (a splitmix64 stream)
//   S(i)              = the sum of the twelve 16-bit fields of r_0, r_1, r_2      (0 .. 12 * 65535)
//   z(i)              = S(i) - 393210                                            (an integer, mean 0)
//   value(i)          = float32(z(i)) * (std / 65536)  [+ mean]                   (each operation rounded once)
//
// A sum of twelve uniform numbers has variance 1 and is normal to well within what random
// initial weights need (no value beyond 6 standard deviations); unlike Box-Muller it uses integer
// arithmetic and one float32 multiplication only, so every platform gets the same bits.
// The reference has no random models (its tests randomise per operator, test/checker.cpp:162-204).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define ILLM_HD __host__ __device__ __forceinline__
#else
#define ILLM_HD inline
#endif

#define ILLM_RANDOM_GAMMA 0x9E3779B97F4A7C15ull

ILLM_HD unsigned long long illm_random_fin(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

inline unsigned long long illm_random_key(unsigned long long seed, const char* name) {
    unsigned long long h = 0xCBF29CE484222325ull;
    for (const unsigned char* p = (const unsigned char*)name; *p; p++) {
        h ^= *p;
        h *= 0x100000001B3ull;
    }
    return h ^ (seed * ILLM_RANDOM_GAMMA);
}

ILLM_HD unsigned long long illm_random_base(unsigned long long key) { return illm_random_fin(key + ILLM_RANDOM_GAMMA); }

// z(i): the centred sum of twelve 16-bit uniform numbers, |z| <= 393210.
ILLM_HD int illm_random_centered_sum(unsigned long long base, unsigned long long i) {
    unsigned sum = 0;
    for (unsigned long long j = 1; j <= 3; j++) {
        const unsigned long long r = illm_random_fin(base + (3ull * i + j) * ILLM_RANDOM_GAMMA);
        sum += (unsigned)(r & 0xFFFF) + (unsigned)((r >> 16) & 0xFFFF) + (unsigned)((r >> 32) & 0xFFFF) +
               (unsigned)(r >> 48);
    }
    return (int)sum - 393210;
}
