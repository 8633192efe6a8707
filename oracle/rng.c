/*
 * TEST INFRASTRUCTURE ONLY (checker): CPU restatement of the reference's seeded RNG
 * and of the hot scalar loops of its CPU optimizer. Never linked into the product
 * library.
 *
 * Follows packages/core/src/rng.ts:6-68 (SeededRng): xorshift128+ on two 32-bit lanes
 * with JavaScript int32 shift semantics, 20 warm-up draws after seeding, and the
 * Marsaglia polar method with one cached spare for Gaussian samples.
 * fill_gauss_f32 follows packages/model/src/gpt.ts:53-58 (initWeight):
 * data[i] = (float) (nextGauss() * std).
 * adamw_f32 follows packages/train/src/optimizers.ts:84-92 (the CPU loop of
 * AdamW.stepParamEntries): f64 arithmetic, f32 stores after every assignment.
 *
 * Parity of the RNG stream is unpinned by the reference's own tests: rng.test.ts
 * holds no literal values (only determinism / range / mean checks, which
 * tests/test_oracle_rng.py repeats).
 */
#include <math.h>
#include <stdint.h>

typedef struct {
  uint32_t s0, s1;
  int32_t has_spare;
  double spare;
} alpha_rng;

static double rng_next(alpha_rng *r) {
  uint32_t s1 = r->s0;
  const uint32_t s0 = r->s1;
  r->s0 = s0;
  s1 ^= s1 << 23;
  s1 ^= s1 >> 17;
  s1 ^= s0;
  s1 ^= s0 >> 26;
  r->s1 = s1;
  return (double)(uint32_t)(r->s0 + r->s1) / 4294967296.0;
}

void alpha_rng_seed(alpha_rng *r, uint32_t seed) {
  r->s0 = seed;
  r->s1 = seed ^ 0xdeadbeefu;
  r->has_spare = 0;
  r->spare = 0.0;
  for (int i = 0; i < 20; i++) (void)rng_next(r);
}

double alpha_rng_next(alpha_rng *r) { return rng_next(r); }

double alpha_rng_gauss(alpha_rng *r) {
  if (r->has_spare) {
    r->has_spare = 0;
    return r->spare;
  }
  double u, v, s;
  do {
    u = rng_next(r) * 2 - 1;
    v = rng_next(r) * 2 - 1;
    s = u * u + v * v;
  } while (s >= 1 || s == 0);
  const double mul = sqrt(-2.0 * log(s) / s);
  r->spare = v * mul;
  r->has_spare = 1;
  return u * mul;
}

void alpha_rng_fill_gauss_f32(alpha_rng *r, float *out, int64_t n, double std) {
  for (int64_t i = 0; i < n; i++) out[i] = (float)(alpha_rng_gauss(r) * std);
}

void alpha_rng_fill_uniform_i32(alpha_rng *r, int32_t *out, int64_t n, int32_t hi) {
  for (int64_t i = 0; i < n; i++) out[i] = (int32_t)floor(rng_next(r) * hi);
}

/* packages/train/src/optimizers.ts:84-92 */
void alpha_oracle_adamw_f32(float *p, const float *g, float *m, float *v, int64_t n,
                            double lr, double beta1, double beta2, double eps, double wd,
                            double bc1, double bc2, double grad_scale) {
  for (int64_t j = 0; j < n; j++) {
    const double gj = (double)g[j] * grad_scale;
    if (wd > 0) p[j] = (float)((double)p[j] - lr * wd * (double)p[j]);
    m[j] = (float)(beta1 * (double)m[j] + (1 - beta1) * gj);
    v[j] = (float)(beta2 * (double)v[j] + (1 - beta2) * gj * gj);
    const double mhat = (double)m[j] / bc1;
    const double vhat = (double)v[j] / bc2;
    p[j] = (float)((double)p[j] - lr * mhat / (sqrt(vhat) + eps));
  }
}

/* packages/autograd/src/ops.ts:495-505: sequential f32 scatter-add of rows. */
void alpha_oracle_embedding_bwd_f32(float *dw, const int32_t *idx, const float *g,
                                    int64_t n_idx, int64_t dim) {
  for (int64_t i = 0; i < n_idx; i++) {
    float *row = dw + (int64_t)idx[i] * dim;
    const float *gi = g + i * dim;
    for (int64_t d = 0; d < dim; d++) row[d] = (float)((double)row[d] + (double)gi[d]);
  }
}

/* packages/tensor/src/cpu_ref.ts:246-254: the reference's sequential f64 dot product
 * GEMM (C = A[M,K] * B[K,N]), one f32 rounding per output. Kept as the literal loop
 * order so that the BLAS-backed numpy restatement can be validated against it and so
 * that the timed CPU baseline runs the reference's own algorithm. */
void alpha_oracle_matmul_f32(const float *a, const float *b, float *c, int64_t M, int64_t K,
                             int64_t N) {
  for (int64_t m = 0; m < M; m++)
    for (int64_t n = 0; n < N; n++) {
      double sum = 0;
      for (int64_t k = 0; k < K; k++) sum += (double)a[m * K + k] * (double)b[k * N + n];
      c[m * N + n] = (float)sum;
    }
}

/* packages/autograd/src/ops.ts:523-569: the CPU fallback of layerNorm backward.
 * Statistics and per-row sums are doubles; dw/db are Float32Array accumulators that
 * round after every row (":547-548"), dx is stored once per element. */
void alpha_oracle_layernorm_bwd_f32(const float *x, const float *w, const float *g, float *dx,
                                    float *dw, float *db, int64_t n, int64_t dim, double eps) {
  for (int64_t j = 0; j < dim; j++) { dw[j] = 0.f; db[j] = 0.f; }
  for (int64_t i = 0; i < n; i++) {
    const float *xr = x + i * dim;
    const float *gr = g + i * dim;
    float *dxr = dx + i * dim;
    double mu = 0;
    for (int64_t j = 0; j < dim; j++) mu += (double)xr[j];
    mu /= (double)dim;
    double variance = 0;
    for (int64_t j = 0; j < dim; j++) {
      const double d = (double)xr[j] - mu;
      variance += d * d;
    }
    variance /= (double)dim;
    const double inv_std = 1 / sqrt(variance + eps);
    for (int64_t j = 0; j < dim; j++) {
      const double xhat = ((double)xr[j] - mu) * inv_std;
      dw[j] = (float)((double)dw[j] + (double)gr[j] * xhat);
      db[j] = (float)((double)db[j] + (double)gr[j]);
    }
    double sum1 = 0, sum2 = 0;
    for (int64_t j = 0; j < dim; j++) {
      const double dy = (double)gr[j] * (double)w[j];
      sum1 += dy;
      sum2 += dy * ((double)xr[j] - mu) * inv_std;
    }
    for (int64_t j = 0; j < dim; j++) {
      const double xhat = ((double)xr[j] - mu) * inv_std;
      const double dy = (double)gr[j] * (double)w[j];
      dxr[j] = (float)(inv_std * (dy - (sum1 + xhat * sum2) / (double)dim));
    }
  }
}
