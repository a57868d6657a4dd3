/* Portable counter-based generator for the seeded synthetic inputs of the MLP
 * benchmark configurations (weights U(lo,hi) or N(0,s), inputs N(0,1), targets +-1).
 *
 * The reference fills its matrices from an MKL VSL quasi-random stream
 * (Rand.cc:14-49, mlp_bench_common.cc:16-33), which cannot be reproduced
 * without MKL.  Every consumer here (CPU oracle, the MKL stand-in used to build
 * the reference, the C++ host driver, the tests) includes this header instead,
 * so all of them see identical bits.  Element i of stream `seed` depends only
 * on (seed, i): fills can be split across threads or ranks in any order.
 *
 * Plain C99; no state.
 */
#ifndef B2_RNG_H
#define B2_RNG_H

#include <math.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

static inline uint64_t b2_mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

/* 64 random bits for element `idx` of stream `seed`. */
static inline uint64_t b2_rng_bits(uint64_t seed, uint64_t idx) {
  return b2_mix64(b2_mix64(seed) + idx);
}

/* Uniform in [0,1) with 24 random mantissa bits (exact in float). */
static inline float b2_rng_unit(uint64_t seed, uint64_t idx) {
  return (float)(b2_rng_bits(seed, idx) >> 40) * (1.0f / 16777216.0f);
}

/* Uniform in [lo,hi): the affine map is done in double so that no compiler
 * contraction can change the rounded float. */
static inline float b2_rng_uniform(uint64_t seed, uint64_t idx, float lo, float hi) {
  double u = (double)(b2_rng_bits(seed, idx) >> 40) * (1.0 / 16777216.0);
  return (float)((double)lo + ((double)hi - (double)lo) * u);
}

/* Standard normal by Box-Muller in double; element idx consumes counters
 * 2*idx and 2*idx+1 of the stream. */
static inline float b2_rng_normal(uint64_t seed, uint64_t idx) {
  double u1 = (double)((b2_rng_bits(seed, 2 * idx) >> 11) + 1) * (1.0 / 9007199254740992.0);
  double u2 = (double)(b2_rng_bits(seed, 2 * idx + 1) >> 11) * (1.0 / 9007199254740992.0);
  return (float)(sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2));
}

/* +1 / -1 with equal probability. */
static inline float b2_rng_sign(uint64_t seed, uint64_t idx) {
  return (b2_rng_bits(seed, idx) & 1ull) ? 1.0f : -1.0f;
}

/* Row-major fills of an nrows x ncols block with leading dimension ld; the
 * counter of element (i,j) is i*ncols+j, independent of ld. */
static inline void b2_fill_uniform(float* a, int nrows, int ncols, size_t ld,
                                   uint64_t seed, float lo, float hi) {
  for (int i = 0; i < nrows; ++i)
    for (int j = 0; j < ncols; ++j)
      a[(size_t)i * ld + j] = b2_rng_uniform(seed, (uint64_t)i * ncols + j, lo, hi);
}

static inline void b2_fill_normal(float* a, int nrows, int ncols, size_t ld,
                                  uint64_t seed, float stddev) {
  for (int i = 0; i < nrows; ++i)
    for (int j = 0; j < ncols; ++j)
      a[(size_t)i * ld + j] = stddev * b2_rng_normal(seed, (uint64_t)i * ncols + j);
}

static inline void b2_fill_sign(float* a, int nrows, int ncols, size_t ld, uint64_t seed) {
  for (int i = 0; i < nrows; ++i)
    for (int j = 0; j < ncols; ++j)
      a[(size_t)i * ld + j] = b2_rng_sign(seed, (uint64_t)i * ncols + j);
}

#ifdef __cplusplus
}
#endif
#endif /* B2_RNG_H */
