/* mugraph_rng.h - counter-based generator shared by device fills and host checkers.
 * value(seed, index) depends on nothing else, so a host loop and a CUDA grid produce the
 * same tensors without copying them.  splitmix64 finaliser over (seed, index); normal
 * deviates by Box-Muller on two 24-bit uniforms. */
#ifndef MUGRAPH_RNG_H_
#define MUGRAPH_RNG_H_
#include <math.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define MG_RNG_FN static __host__ __device__ __forceinline__
#else
#define MG_RNG_FN static inline
#endif

MG_RNG_FN uint64_t mg_rng_mix(uint64_t seed, uint64_t index) {
  uint64_t z = seed * 0x9E3779B97F4A7C15ull + index * 0xD1B54A32D192ED03ull + 0x632BE59BD9B4E019ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

/* uniform integer in [0, modulus), modulus <= 65536 */
MG_RNG_FN uint32_t mg_rng_uniform(uint64_t seed, uint64_t index, uint32_t modulus) {
  return (uint32_t)((mg_rng_mix(seed, index) >> 32) % modulus);
}

/* standard normal deviate.  logf/cosf are not bit-identical between the host and the device
 * math libraries, so a checker that needs the exact tensor downloads it instead of regenerating it;
 * the integer generators above are exact everywhere. */
MG_RNG_FN float mg_rng_normal(uint64_t seed, uint64_t index) {
  uint64_t r = mg_rng_mix(seed, index);
  float u1 = ((float)((r >> 40) & 0xFFFFFF) + 1.0f) * (1.0f / 16777216.0f); /* (0, 1] */
  float u2 = (float)((r >> 16) & 0xFFFFFF) * (1.0f / 16777216.0f);           /* [0, 1) */
  return sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
}

#endif /* MUGRAPH_RNG_H_ */
