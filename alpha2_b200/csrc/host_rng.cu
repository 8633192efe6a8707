// Host-side seeded generator used for parameter initialisation, so that a model created
// through this backend starts from the same weights as one created by the reference.
// Stream definition: packages/core/src/rng.ts:6-68 — xorshift128+ on two 32-bit lanes
// seeded with (seed, seed ^ 0xdeadbeef), twenty discarded draws, uniform = (s0+s1 mod 2^32)
// / 2^32; Gaussian by the polar method, returning u*f and keeping v*f for the next call.
// Weight fill: packages/model/src/gpt.ts:53-58, value = float(gauss * std).
#include <math.h>

#include "common.cuh"

static inline uint32_t step(alpha_host_rng_t *r) {
  uint32_t a = r->s0;
  const uint32_t b = r->s1;
  r->s0 = b;
  a ^= a << 23;
  a ^= a >> 17;
  a ^= b ^ (b >> 26);
  r->s1 = a;
  return r->s0 + r->s1;
}

extern "C" {

int alpha_rng_seed(alpha_host_rng_t *r, uint32_t seed) {
  r->s0 = seed;
  r->s1 = seed ^ 0xdeadbeefu;
  r->has_spare = 0;
  r->spare = 0.0;
  for (int i = 0; i < 20; i++) step(r);
  return 0;
}

double alpha_rng_next(alpha_host_rng_t *r) { return (double)step(r) * (1.0 / 4294967296.0); }

double alpha_rng_gauss(alpha_host_rng_t *r) {
  if (r->has_spare) {
    r->has_spare = 0;
    return r->spare;
  }
  double u, v, s;
  for (;;) {
    u = alpha_rng_next(r) * 2 - 1;
    v = alpha_rng_next(r) * 2 - 1;
    s = u * u + v * v;
    if (s < 1 && s != 0) break;
  }
  const double f = sqrt(-2.0 * log(s) / s);
  r->spare = v * f;
  r->has_spare = 1;
  return u * f;
}

int alpha_rng_fill_gauss(alpha_host_rng_t *r, float *host_out, int64_t n, double std) {
  for (int64_t i = 0; i < n; i++) host_out[i] = (float)(alpha_rng_gauss(r) * std);
  return 0;
}

}  // extern "C"
