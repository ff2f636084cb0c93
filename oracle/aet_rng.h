/*
 * TEST INFRASTRUCTURE ONLY -- deterministic synthetic-tensor generator shared
 * by the CPU oracle and its timing driver.  The product library never includes
 * this header; the Python package carries an identical numpy generator
 * (synth.py) and a test keeps the two in lock-step.
 *
 * Stream definition
 *   state_i = (seed ^ tensor_id) + (i + 1) * 0x9E3779B97F4A7C15   (mod 2^64)
 *   z       = splitmix64 finaliser(state_i)
 *   u_i     = (z >> 40) * 2^-24            in [0, 1)
 * Normals use Box-Muller on consecutive pairs (u_2j, u_2j+1), cosine branch
 * only, evaluated in float:  g_j = sqrtf(-2 logf(max(u_2j, 2^-24))) * cosf(2 pi u_2j+1).
 */
#ifndef AET_ORACLE_RNG_H
#define AET_ORACLE_RNG_H
#include <stdint.h>
#include <math.h>

static inline uint64_t aet_rng_mix(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

static inline float aet_rng_uniform(uint64_t seed, uint64_t tensor_id, uint64_t i) {
    uint64_t s = (seed ^ tensor_id) + (i + 1) * 0x9E3779B97F4A7C15ULL;
    return (float)(aet_rng_mix(s) >> 40) * (1.0f / 16777216.0f);
}

static inline float aet_rng_normal(uint64_t seed, uint64_t tensor_id, uint64_t j) {
    float u1 = aet_rng_uniform(seed, tensor_id, 2 * j);
    float u2 = aet_rng_uniform(seed, tensor_id, 2 * j + 1);
    if (u1 < 1.0f / 16777216.0f) u1 = 1.0f / 16777216.0f;
    return sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
}

static inline void aet_rng_fill_uniform(float *dst, uint64_t n, uint64_t seed, uint64_t tensor_id) {
    for (uint64_t i = 0; i < n; ++i) dst[i] = aet_rng_uniform(seed, tensor_id, i);
}

static inline void aet_rng_fill_normal(float *dst, uint64_t n, uint64_t seed, uint64_t tensor_id,
                                       float mean, float stddev) {
    for (uint64_t i = 0; i < n; ++i) dst[i] = mean + stddev * aet_rng_normal(seed, tensor_id, i);
}
#endif
