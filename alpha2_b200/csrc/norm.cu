// LayerNorm / RMSNorm forward and backward.  HBM-bound: each row is read once with 16-byte
// loads into registers (one warp per row), statistics by warp shuffles in two passes over
// the registers, outputs stored with 16-byte stores.
//
// Reference semantics: packages/tensor/src/cpu_ref.ts:387-420 (forward: biased variance,
// y = (x-mean)*rsqrt(var+eps)*w + b) and packages/autograd/src/ops.ts:523-569 (backward:
// dx = rstd*(dy - (sum(dy) + xhat*sum(dy*xhat))/dim) with dy = g*w; dw = sum_rows g*xhat;
// db = sum_rows g).  Weights, biases and their gradients are always f32.
//
// Backward reduces dw/db in two deterministic stages: every block keeps per-lane column
// sums over the rows it walks, writes one partial row to scratch, and a second kernel adds
// the partial rows in block order.  Algorithmic bytes per row: forward 2*dim*e, backward
// 3*dim*e (e = element size) — the scratch adds 2*grid*dim*4 bytes per call.
#include <stdlib.h>
#include "tc_common.cuh"

namespace alpha {

constexpr int LN_WARPS = 4;

template <typename T, int NV, bool RMS>
__global__ void __launch_bounds__(LN_WARPS * 32) ln_fwd_warp(const T *__restrict__ x, const float *__restrict__ w,
                                                             const float *__restrict__ b, T *__restrict__ y,
                                                             int64_t rows, int dim, float eps) {
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int nvec = dim / V;
  const int64_t warp_global = (int64_t)blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
  const int64_t warp_stride = (int64_t)gridDim.x * LN_WARPS;
  for (int64_t r = warp_global; r < rows; r += warp_stride) {
    float xv[NV][V];
    const T *xr = x + r * dim;
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < NV; v++) {
      const int iv = v * 32 + lane;
      if (iv < nvec) {
        Vec16<T> t;
        t.load(xr + iv * V);
        t.get(xv[v]);
#pragma unroll
        for (int j = 0; j < V; j++) s += RMS ? xv[v][j] * xv[v][j] : xv[v][j];
      }
    }
    s = warp_sum(s);
    float mean = 0.f, rstd;
    if (RMS) {
      rstd = rsqrtf(s / dim + eps);
    } else {
      mean = s / dim;
      float q = 0.f;
#pragma unroll
      for (int v = 0; v < NV; v++)
        if (v * 32 + lane < nvec) {
#pragma unroll
          for (int j = 0; j < V; j++) {
            const float d = xv[v][j] - mean;
            q += d * d;
          }
        }
      q = warp_sum(q);
      rstd = 1.f / sqrtf(q / dim + eps);
    }
    T *yr = y + r * dim;
#pragma unroll
    for (int v = 0; v < NV; v++) {
      const int iv = v * 32 + lane;
      if (iv < nvec) {
        float o[V];
#pragma unroll
        for (int j = 0; j < V; j++) {
          const int c = iv * V + j;
          o[j] = (xv[v][j] - mean) * rstd * w[c] + (RMS ? 0.f : b[c]);
        }
        Vec16<T> t;
        t.set(o);
        t.store(yr + iv * V);
      }
    }
  }
}

// Backward, one warp per row, persistent over rows.  part: [gridDim.x, 2, dim] f32.
template <typename T, int NV, bool RMS>
__global__ void __launch_bounds__(LN_WARPS * 32) ln_bwd_warp(const T *__restrict__ x, const float *__restrict__ w,
                                                             const T *__restrict__ g, const T *dx_add, T *dx,
                                                             float *__restrict__ part, int64_t rows, int dim,
                                                             float eps) {
  constexpr int V = Vec16<T>::N;
  extern __shared__ float sm[];  // [LN_WARPS][2][dim]
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nvec = dim / V;
  float dw_acc[NV][V], db_acc[NV][V], wv[NV][V];
#pragma unroll
  for (int v = 0; v < NV; v++) {
    const int iv = v * 32 + lane;
#pragma unroll
    for (int j = 0; j < V; j++) {
      dw_acc[v][j] = 0.f;
      db_acc[v][j] = 0.f;
      wv[v][j] = iv < nvec ? w[iv * V + j] : 0.f;
    }
  }
  const int64_t warp_global = (int64_t)blockIdx.x * LN_WARPS + wid;
  const int64_t warp_stride = (int64_t)gridDim.x * LN_WARPS;
  for (int64_t r = warp_global; r < rows; r += warp_stride) {
    float xv[NV][V], gv[NV][V];
    const T *xr = x + r * dim, *gr = g + r * dim;
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < NV; v++) {
      const int iv = v * 32 + lane;
      if (iv < nvec) {
        Vec16<T> t, u;
        t.load(xr + iv * V);
        u.load(gr + iv * V);
        t.get(xv[v]);
        u.get(gv[v]);
#pragma unroll
        for (int j = 0; j < V; j++) s += RMS ? xv[v][j] * xv[v][j] : xv[v][j];
      }
    }
    s = warp_sum(s);
    float mean = 0.f, rstd;
    if (RMS) {
      rstd = rsqrtf(s / dim + eps);
    } else {
      mean = s / dim;
      float q = 0.f;
#pragma unroll
      for (int v = 0; v < NV; v++)
        if (v * 32 + lane < nvec) {
#pragma unroll
          for (int j = 0; j < V; j++) {
            const float d = xv[v][j] - mean;
            q += d * d;
          }
        }
      q = warp_sum(q);
      rstd = 1.f / sqrtf(q / dim + eps);
    }
    float sum1 = 0.f, sum2 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; v++)
      if (v * 32 + lane < nvec) {
#pragma unroll
        for (int j = 0; j < V; j++) {
          const float xhat = (xv[v][j] - mean) * rstd;
          const float dy = gv[v][j] * wv[v][j];
          dw_acc[v][j] += gv[v][j] * xhat;
          db_acc[v][j] += gv[v][j];
          sum1 += dy;
          sum2 += dy * xhat;
          xv[v][j] = xhat;  // keep xhat
          gv[v][j] = dy;    // keep dy
        }
      }
    sum1 = warp_sum(sum1);
    sum2 = warp_sum(sum2);
    if (RMS) sum1 = 0.f;  // no mean subtraction in RMSNorm
    T *dr = dx + r * dim;
#pragma unroll
    for (int v = 0; v < NV; v++) {
      const int iv = v * 32 + lane;
      if (iv < nvec) {
        float o[V];
#pragma unroll
        for (int j = 0; j < V; j++) o[j] = rstd * (gv[v][j] - (sum1 + xv[v][j] * sum2) / dim);
        if (dx_add) {  // dx = dx_add + result (dx may alias dx_add: each element is read, then written, by one thread)
          Vec16<T> u;
          float e[V];
          u.load(dx_add + r * dim + iv * V);
          u.get(e);
#pragma unroll
          for (int j = 0; j < V; j++) o[j] += e[j];
        }
        Vec16<T> t;
        t.set(o);
        t.store(dr + iv * V);
      }
    }
  }
  // block-level reduce of the per-warp column sums, fixed warp order
  float *my = sm + (size_t)wid * 2 * dim;
#pragma unroll
  for (int v = 0; v < NV; v++) {
    const int iv = v * 32 + lane;
    if (iv < nvec) {
#pragma unroll
      for (int j = 0; j < V; j++) {
        my[iv * V + j] = dw_acc[v][j];
        my[dim + iv * V + j] = db_acc[v][j];
      }
    }
  }
  __syncthreads();
  float *out = part + (size_t)blockIdx.x * 2 * dim;
  for (int c = threadIdx.x; c < 2 * dim; c += blockDim.x) {
    float a = 0.f;
#pragma unroll
    for (int k = 0; k < LN_WARPS; k++) a += sm[(size_t)k * 2 * dim + c];
    out[c] = a;
  }
}

// dw[c] (+)= sum_p part[p][0][c]; db[c] (+)= sum_p part[p][1][c].  Block = 32 columns x 32 row
// groups: each thread adds every 32nd partial row of its column, four independent loads at a
// time, then the 32 group sums are added in fixed order, so the result does not depend on
// scheduling.
constexpr int LN_RED_GROUPS = 32;
__global__ void __launch_bounds__(32 * LN_RED_GROUPS) ln_reduce_partials(const float *__restrict__ part, float *dw,
                                                                         float *db, int n_part, int dim,
                                                                         int accumulate) {
  __shared__ float sm[LN_RED_GROUPS][33];
  grid_dependency_trigger();
  grid_dependency_wait();
  const int c = blockIdx.x * 32 + threadIdx.x;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  if (c < 2 * dim) {
    const size_t ld = (size_t)2 * dim;
    int p = threadIdx.y;
    for (; p + 3 * LN_RED_GROUPS < n_part; p += 4 * LN_RED_GROUPS) {
      a0 += part[(size_t)p * ld + c];
      a1 += part[(size_t)(p + LN_RED_GROUPS) * ld + c];
      a2 += part[(size_t)(p + 2 * LN_RED_GROUPS) * ld + c];
      a3 += part[(size_t)(p + 3 * LN_RED_GROUPS) * ld + c];
    }
    for (; p < n_part; p += LN_RED_GROUPS) a0 += part[(size_t)p * ld + c];
  }
  sm[threadIdx.y][threadIdx.x] = (a0 + a1) + (a2 + a3);
  __syncthreads();
  if (threadIdx.y == 0 && c < 2 * dim) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < LN_RED_GROUPS; k++) t += sm[k][threadIdx.x];
    float *dst = c < dim ? dw + c : (db ? db + (c - dim) : nullptr);
    if (dst) *dst = accumulate ? *dst + t : t;
  }
}

// ── a CTA per group of R rows (the fast path) ────────────────────────────────────────────
// Up to 128 threads walk groups of R rows; thread t owns the 16-byte column vectors t and
// t + blockDim.x of every row, so its slice of the weight / bias (and, backward, of the
// dw / db sums) stays in registers for the whole kernel and only the rows themselves move,
// every access a fully coalesced 16-byte load or store.  The next group is fetched into
// registers before the current one is reduced, so each CTA keeps 2·R rows of loads in flight
// across the block reductions (warp shuffle + one partial per warp in shared memory, one
// __syncthreads each; the slots alternate between groups so no second barrier is needed).
constexpr int LN_CTA = 128;

// sums of R values over the block; slot is [R][4] floats private to this reduction instance
// (entries of warps that do not exist stay zero from the kernel prologue)
template <int R>
__device__ __forceinline__ void cta_sum_rows(float (&v)[R], float (*slot)[4]) {
#pragma unroll
  for (int k = 0; k < R; k++) v[k] = warp_sum(v[k]);
  if ((threadIdx.x & 31) == 0) {
#pragma unroll
    for (int k = 0; k < R; k++) slot[k][threadIdx.x >> 5] = v[k];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < R; k++) v[k] = (slot[k][0] + slot[k][1]) + (slot[k][2] + slot[k][3]);
}

template <typename T, int NV, int R, bool RMS>
__global__ void __launch_bounds__(LN_CTA) ln_fwd_cta(const T *__restrict__ x, const float *__restrict__ w,
                                                     const float *__restrict__ b, T *__restrict__ y, int64_t rows,
                                                     int dim, float eps) {
  constexpr int V = Vec16<T>::N;
  __shared__ float red[2][2][R][4];
  for (int i = threadIdx.x; i < 2 * 2 * R * 4; i += blockDim.x) (&red[0][0][0][0])[i] = 0.f;
  __syncthreads();
  const int nvec = dim / V, nt = blockDim.x;
  bool act[NV];
  float wv[NV][V], bv[NV][V];
#pragma unroll
  for (int v = 0; v < NV; v++) {
    const int iv = v * nt + threadIdx.x;
    act[v] = iv < nvec;
#pragma unroll
    for (int j = 0; j < V; j += 4) {
      const float4 a = act[v] ? *reinterpret_cast<const float4 *>(w + iv * V + j) : make_float4(0, 0, 0, 0);
      const float4 c = (!RMS && act[v]) ? *reinterpret_cast<const float4 *>(b + iv * V + j) : make_float4(0, 0, 0, 0);
      wv[v][j] = a.x; wv[v][j + 1] = a.y; wv[v][j + 2] = a.z; wv[v][j + 3] = a.w;
      bv[v][j] = c.x; bv[v][j + 1] = c.y; bv[v][j + 2] = c.z; bv[v][j + 3] = c.w;
    }
  }
  const int64_t ngroups = (rows + R - 1) / R;
  Vec16<T> nxt[R][NV];
  auto fetch = [&](int64_t grp) {
#pragma unroll
    for (int k = 0; k < R; k++) {
      const int64_t r = grp * R + k;
      if (r < rows) {
#pragma unroll
        for (int v = 0; v < NV; v++)
          if (act[v]) nxt[k][v].load(x + r * dim + (v * nt + threadIdx.x) * V);
      }
    }
  };
  if (blockIdx.x < ngroups) fetch(blockIdx.x);
  int par = 0;
  for (int64_t grp = blockIdx.x; grp < ngroups; grp += gridDim.x, par ^= 1) {
    float xv[R][NV][V];
    float s[R];
#pragma unroll
    for (int k = 0; k < R; k++) {
      s[k] = 0.f;
      const bool rv = grp * R + k < rows;
#pragma unroll
      for (int v = 0; v < NV; v++) {
        if (rv && act[v]) {
          nxt[k][v].get(xv[k][v]);
        } else {
#pragma unroll
          for (int j = 0; j < V; j++) xv[k][v][j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < V; j++) s[k] += RMS ? xv[k][v][j] * xv[k][v][j] : xv[k][v][j];
      }
    }
    if (grp + gridDim.x < ngroups) fetch(grp + gridDim.x);
    cta_sum_rows<R>(s, red[par][0]);
    float mean[R], rstd[R];
    if (RMS) {
#pragma unroll
      for (int k = 0; k < R; k++) {
        mean[k] = 0.f;
        rstd[k] = rsqrtf(s[k] / dim + eps);
      }
    } else {
      float q[R];
#pragma unroll
      for (int k = 0; k < R; k++) {
        mean[k] = s[k] / dim;
        q[k] = 0.f;
#pragma unroll
        for (int v = 0; v < NV; v++)
          if (act[v]) {
#pragma unroll
            for (int j = 0; j < V; j++) {
              const float d = xv[k][v][j] - mean[k];
              q[k] += d * d;
            }
          }
      }
      cta_sum_rows<R>(q, red[par][1]);
#pragma unroll
      for (int k = 0; k < R; k++) rstd[k] = 1.f / sqrtf(q[k] / dim + eps);
    }
#pragma unroll
    for (int k = 0; k < R; k++) {
      const int64_t r = grp * R + k;
      if (r < rows) {
#pragma unroll
        for (int v = 0; v < NV; v++)
          if (act[v]) {
            float o[V];
#pragma unroll
            for (int j = 0; j < V; j++) o[j] = (xv[k][v][j] - mean[k]) * rstd[k] * wv[v][j] + bv[v][j];
            Vec16<T> t;
            t.set(o);
            t.store(y + r * dim + (v * nt + threadIdx.x) * V);
          }
      }
    }
  }
}

// part: [gridDim.x][2][dim] f32 partial column sums (dw, db), written once per CTA.
template <typename T, int NV, int R, bool RMS>
__global__ void __launch_bounds__(LN_CTA) ln_bwd_cta(const T *__restrict__ x, const float *__restrict__ w,
                                                     const T *__restrict__ g, const T *dx_add, T *dx,
                                                     float *__restrict__ part, int64_t rows, int dim, float eps) {
  constexpr int V = Vec16<T>::N;
  __shared__ float red[2][4][R][4];
  for (int i = threadIdx.x; i < 2 * 4 * R * 4; i += blockDim.x) (&red[0][0][0][0])[i] = 0.f;
  __syncthreads();
  const int nvec = dim / V, nt = blockDim.x;
  bool act[NV];
  float wv[NV][V], dw_acc[NV][V], db_acc[NV][V];
#pragma unroll
  for (int v = 0; v < NV; v++) {
    const int iv = v * nt + threadIdx.x;
    act[v] = iv < nvec;
#pragma unroll
    for (int j = 0; j < V; j += 4) {
      const float4 a = act[v] ? *reinterpret_cast<const float4 *>(w + iv * V + j) : make_float4(0, 0, 0, 0);
      wv[v][j] = a.x; wv[v][j + 1] = a.y; wv[v][j + 2] = a.z; wv[v][j + 3] = a.w;
    }
#pragma unroll
    for (int j = 0; j < V; j++) dw_acc[v][j] = db_acc[v][j] = 0.f;
  }
  const int64_t ngroups = (rows + R - 1) / R;
  Vec16<T> nx[R][NV], ng[R][NV], na[R][NV];
  auto fetch = [&](int64_t grp) {
#pragma unroll
    for (int k = 0; k < R; k++) {
      const int64_t r = grp * R + k;
      if (r < rows) {
#pragma unroll
        for (int v = 0; v < NV; v++)
          if (act[v]) {
            const int64_t off = r * dim + (v * nt + threadIdx.x) * V;
            nx[k][v].load(x + off);
            ng[k][v].load(g + off);
            if (dx_add) na[k][v].load(dx_add + off);
          }
      }
    }
  };
  if (blockIdx.x < ngroups) fetch(blockIdx.x);
  int par = 0;
  for (int64_t grp = blockIdx.x; grp < ngroups; grp += gridDim.x, par ^= 1) {
    float xv[R][NV][V], gv[R][NV][V];
    Vec16<T> av[R][NV];
    float s[R];
#pragma unroll
    for (int k = 0; k < R; k++) {
      s[k] = 0.f;
      const bool rv = grp * R + k < rows;
#pragma unroll
      for (int v = 0; v < NV; v++) {
        if (rv && act[v]) {
          nx[k][v].get(xv[k][v]);
          ng[k][v].get(gv[k][v]);
          av[k][v] = na[k][v];
        } else {
#pragma unroll
          for (int j = 0; j < V; j++) xv[k][v][j] = gv[k][v][j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < V; j++) s[k] += RMS ? xv[k][v][j] * xv[k][v][j] : xv[k][v][j];
      }
    }
    if (grp + gridDim.x < ngroups) fetch(grp + gridDim.x);
    cta_sum_rows<R>(s, red[par][0]);
    float mean[R], rstd[R];
    if (RMS) {
#pragma unroll
      for (int k = 0; k < R; k++) {
        mean[k] = 0.f;
        rstd[k] = rsqrtf(s[k] / dim + eps);
      }
    } else {
      float q[R];
#pragma unroll
      for (int k = 0; k < R; k++) {
        mean[k] = s[k] / dim;
        q[k] = 0.f;
#pragma unroll
        for (int v = 0; v < NV; v++)
          if (act[v]) {
#pragma unroll
            for (int j = 0; j < V; j++) {
              const float d = xv[k][v][j] - mean[k];
              q[k] += d * d;
            }
          }
      }
      cta_sum_rows<R>(q, red[par][1]);
#pragma unroll
      for (int k = 0; k < R; k++) rstd[k] = 1.f / sqrtf(q[k] / dim + eps);
    }
    float s1[R], s2[R];
#pragma unroll
    for (int k = 0; k < R; k++) {
      s1[k] = s2[k] = 0.f;
#pragma unroll
      for (int v = 0; v < NV; v++)
        if (act[v]) {
#pragma unroll
          for (int j = 0; j < V; j++) {
            const float xhat = (xv[k][v][j] - mean[k]) * rstd[k];
            const float dy = gv[k][v][j] * wv[v][j];
            dw_acc[v][j] += gv[k][v][j] * xhat;  // rows past the end carry g == 0
            db_acc[v][j] += gv[k][v][j];
            s1[k] += dy;
            s2[k] += dy * xhat;
            xv[k][v][j] = xhat;
            gv[k][v][j] = dy;
          }
        }
    }
    // the two sums share one barrier
    {
      float both[2 * R];
#pragma unroll
      for (int k = 0; k < R; k++) {
        both[k] = s1[k];
        both[R + k] = s2[k];
      }
      cta_sum_rows<2 * R>(both, reinterpret_cast<float(*)[4]>(&red[par][2][0][0]));
#pragma unroll
      for (int k = 0; k < R; k++) {
        s1[k] = RMS ? 0.f : both[k];
        s2[k] = both[R + k];
      }
    }
#pragma unroll
    for (int k = 0; k < R; k++) {
      const int64_t r = grp * R + k;
      if (r < rows) {
#pragma unroll
        for (int v = 0; v < NV; v++)
          if (act[v]) {
            float o[V];
#pragma unroll
            for (int j = 0; j < V; j++) o[j] = rstd[k] * (gv[k][v][j] - (s1[k] + xv[k][v][j] * s2[k]) / dim);
            if (dx_add) {
              float e[V];
              av[k][v].get(e);
#pragma unroll
              for (int j = 0; j < V; j++) o[j] += e[j];
            }
            Vec16<T> t;
            t.set(o);
            t.store(dx + r * dim + (v * nt + threadIdx.x) * V);
          }
      }
    }
  }
  float *out = part + (size_t)blockIdx.x * 2 * dim;
#pragma unroll
  for (int v = 0; v < NV; v++) {
    if (act[v]) {
      const int iv = v * nt + threadIdx.x;
#pragma unroll
      for (int j = 0; j < V; j += 4) {
        *reinterpret_cast<float4 *>(out + iv * V + j) =
            make_float4(dw_acc[v][j], dw_acc[v][j + 1], dw_acc[v][j + 2], dw_acc[v][j + 3]);
        *reinterpret_cast<float4 *>(out + dim + iv * V + j) =
            make_float4(db_acc[v][j], db_acc[v][j + 1], db_acc[v][j + 2], db_acc[v][j + 3]);
      }
    }
  }
}

// ── backward, a warp per row fed by a bulk-copy ring (the fastest path) ──────────────────
// Four worker warps each own one row of a 4-row group; a fifth warp streams the groups
// (x, g and the optional residual gradient are contiguous 4-row slabs) into a 3-stage
// shared-memory ring with one bulk copy per slab, so the loads of the next groups are in
// flight while the workers compute and nothing depends on how the compiler schedules
// loads.  A lane owns the 16-byte vectors lane, lane + 32, ... of its row: row statistics
// are warp shuffles only (no block barrier in the loop), dw / db sums stay in registers
// and are combined across the four warps once at the end, in fixed order.
constexpr int LR_WARPS = 4, LR_STAGES = 3, LR_THREADS = (LR_WARPS + 1) * 32;
// The ring kernels keep a row as packed fp32 pairs (two values per 64-bit register) and use
// the packed add / mul / fma of sm_100: half the issue slots of scalar fp32 for the same,
// equally rounded, arithmetic.  Pair i of a 16-byte vector holds its elements 2i and 2i + 1.
template <typename T> struct RowPairs;
template <> struct RowPairs<float> {
  static constexpr int NP = 2;
  static __device__ __forceinline__ void get(const Vec16<float> &v, uint64_t *p) {
    p[0] = tc::f2_pack(v.raw.x, v.raw.y);
    p[1] = tc::f2_pack(v.raw.z, v.raw.w);
  }
  static __device__ __forceinline__ void set(Vec16<float> &v, const uint64_t *p) {
    tc::f2_unpack(p[0], v.raw.x, v.raw.y);
    tc::f2_unpack(p[1], v.raw.z, v.raw.w);
  }
};
template <> struct RowPairs<__nv_bfloat16> {
  static constexpr int NP = 4;
  static __device__ __forceinline__ void get(const Vec16<__nv_bfloat16> &v, uint64_t *p) {
    p[0] = tc::bf16x2_to_f2(v.raw.x);
    p[1] = tc::bf16x2_to_f2(v.raw.y);
    p[2] = tc::bf16x2_to_f2(v.raw.z);
    p[3] = tc::bf16x2_to_f2(v.raw.w);
  }
  static __device__ __forceinline__ void set(Vec16<__nv_bfloat16> &v, const uint64_t *p) {
    float a, b;
    tc::f2_unpack(p[0], a, b); v.raw.x = tc::bf16x2_pack(a, b);
    tc::f2_unpack(p[1], a, b); v.raw.y = tc::bf16x2_pack(a, b);
    tc::f2_unpack(p[2], a, b); v.raw.z = tc::bf16x2_pack(a, b);
    tc::f2_unpack(p[3], a, b); v.raw.w = tc::bf16x2_pack(a, b);
  }
};
__device__ __forceinline__ float pair_total(uint64_t v) {
  float a, b;
  tc::f2_unpack(v, a, b);
  return a + b;
}
__device__ __forceinline__ uint64_t pair_of(float v) { return tc::f2_pack(v, v); }
// Mean (0 for RMSNorm) and 1/std of a row held as NP2 pairs per lane; on return the pairs are
// centred (x - mean).
template <int NP2, bool RMS>
__device__ __forceinline__ void row_stats(uint64_t (&xp)[NP2], float inv_dim, float eps, float &rstd) {
  using namespace tc;
  if (RMS) {
    uint64_t acc = f2_mul(xp[0], xp[0]);
#pragma unroll
    for (int j = 1; j < NP2; j++) acc = f2_fma(xp[j], xp[j], acc);
    rstd = rsqrtf(warp_sum(pair_total(acc)) * inv_dim + eps);
  } else {
    uint64_t acc = xp[0];
#pragma unroll
    for (int j = 1; j < NP2; j++) acc = f2_add(acc, xp[j]);
    const float mean = warp_sum(pair_total(acc)) * inv_dim;
    const uint64_t nm = pair_of(-mean);
    xp[0] = f2_add(xp[0], nm);
    uint64_t q = f2_mul(xp[0], xp[0]);
#pragma unroll
    for (int j = 1; j < NP2; j++) {
      xp[j] = f2_add(xp[j], nm);
      q = f2_fma(xp[j], xp[j], q);
    }
    rstd = 1.f / sqrtf(warp_sum(pair_total(q)) * inv_dim + eps);
  }
}

// Position of per-column constant c (weight, bias) in shared memory: a lane owns V consecutive
// columns per vector and reads them as float4s, so the float4s of one (vector, quarter) are laid
// side by side across the 32 lanes (16-byte lane stride: no bank conflicts) instead of V*4 bytes apart.
template <int V>
__device__ __forceinline__ int lr_const_pos(int c) {
  const int j = c % V, lane = (c / V) & 31, v = c / (32 * V);
  return ((v * (V / 4) + j / 4) * 32 + lane) * 4 + (j & 3);
}

// 32 elements per lane need more registers than three resident blocks leave (and their ring
// takes a third of the shared memory anyway): two blocks per SM there.
template <typename T, int NV>
constexpr int lr_bwd_blocks() { return NV * (16 / (int)sizeof(T)) > 24 ? 2 : 3; }

template <typename T, int NV, bool RMS, bool HAS_ADD>
__global__ void __launch_bounds__(LR_THREADS, lr_bwd_blocks<T, NV>())
ln_bwd_ring(const T *__restrict__ x, const float *__restrict__ w, const T *__restrict__ g,
            const T *__restrict__ dx_add, T *__restrict__ dx, float *__restrict__ part, int64_t rows, int dim, float eps,
            uint32_t *err) {
  using namespace tc;
  constexpr int V = Vec16<T>::N;
  constexpr int NS = HAS_ADD ? 3 : 2;
  extern __shared__ __align__(128) uint8_t lr_smem[];
  const uint32_t row_bytes = (uint32_t)dim * sizeof(T);
  const uint32_t slab = LR_WARPS * row_bytes, stage_bytes = NS * slab;
  const uint32_t ring = smem_u32(lr_smem);
  const uint32_t bar = ring + LR_STAGES * stage_bytes;
  auto full_bar = [&](int s) { return bar + 8u * s; };
  auto empty_bar = [&](int s) { return bar + 8u * (LR_STAGES + s); };
  volatile uint32_t *abort_flag = (volatile uint32_t *)(lr_smem + LR_STAGES * stage_bytes + 16 * LR_STAGES);
  float *w_sm = reinterpret_cast<float *>(lr_smem + LR_STAGES * stage_bytes + 64);  // the weight row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n_groups = (rows + LR_WARPS - 1) / LR_WARPS;
  auto load_group = [&](int s, int64_t grp) {
    const int64_t r0 = grp * LR_WARPS;
    const uint32_t bytes = (uint32_t)min((int64_t)LR_WARPS, rows - r0) * row_bytes;
    const uint32_t dst = ring + s * stage_bytes;
    if (elect_one()) {
      mbar_expect_tx(full_bar(s), NS * bytes);
      bulk_load_1d(dst, x + r0 * dim, bytes, full_bar(s));
      bulk_load_1d(dst + slab, g + r0 * dim, bytes, full_bar(s));
      if (HAS_ADD) bulk_load_1d(dst + 2 * slab, dx_add + r0 * dim, bytes, full_bar(s));
    }
    __syncwarp();
  };
  // The producer warp sets the barriers up and fills the whole ring before the block's first
  // barrier, so that the first rows are on their way while the workers fetch the weight row.
  if (warp == LR_WARPS) {
    if (lane == 0) {
      for (int s = 0; s < LR_STAGES; s++) {
        mbar_init(full_bar(s), 1);
        mbar_init(empty_bar(s), LR_WARPS);
      }
      *abort_flag = 0;
      fence_barrier_init();
      fence_proxy_async();
    }
    __syncwarp();
  }
  grid_dependency_trigger();
  grid_dependency_wait();
  int p_i = 0;                     // producer cursor: groups issued so far, next group
  int64_t p_grp = blockIdx.x;
  if (warp == LR_WARPS)
    for (; p_i < LR_STAGES && p_grp < n_groups; p_i++, p_grp += gridDim.x) load_group(p_i, p_grp);
  {
    constexpr int TRIPS = (NV * 32 * V + LR_THREADS - 1) / LR_THREADS;  // dim <= NV * 32 * V: a fixed trip count
    float wv[TRIPS];
#pragma unroll
    for (int k = 0; k < TRIPS; k++) {
      const int c = threadIdx.x + k * LR_THREADS;
      wv[k] = c < dim ? w[c] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < TRIPS; k++) {
      const int c = threadIdx.x + k * LR_THREADS;
      if (c < dim) w_sm[lr_const_pos<V>(c)] = wv[k];
    }
  }
  __syncthreads();

  constexpr int NP = RowPairs<T>::NP, NP2 = NV * NP;  // pairs per vector, per lane and row
  uint64_t dw_acc[NP2], db_acc[NP2];
#pragma unroll
  for (int j = 0; j < NP2; j++) dw_acc[j] = db_acc[j] = 0ull;

  if (warp == LR_WARPS) {
    // producer: the rest of the groups, each into a slot the workers have released
    for (; p_grp < n_groups; p_grp += gridDim.x, p_i++) {
      const int s = p_i % LR_STAGES;
      if (!mbar_wait(empty_bar(s), ((p_i / LR_STAGES) & 1) ^ 1, abort_flag)) break;
      load_group(s, p_grp);
    }
  } else {
    const float inv_dim = 1.f / (float)dim;
    int i = 0;
    for (int64_t grp = blockIdx.x; grp < n_groups; grp += gridDim.x, i++) {
      const int s = i % LR_STAGES;
      if (!mbar_wait(full_bar(s), (i / LR_STAGES) & 1, abort_flag)) break;
      const int64_t r = grp * LR_WARPS + warp;
      const uint8_t *src = lr_smem + s * stage_bytes + warp * row_bytes;
      uint64_t xp[NP2], gp[NP2];
      Vec16<T> av[NV];
#pragma unroll
      for (int v = 0; v < NV; v++) {
        Vec16<T> t, u;
        t.load(reinterpret_cast<const T *>(src + (v * 32 + lane) * 16));
        u.load(reinterpret_cast<const T *>(src + slab + (v * 32 + lane) * 16));
        if (HAS_ADD) av[v].load(reinterpret_cast<const T *>(src + 2 * slab + (v * 32 + lane) * 16));
        RowPairs<T>::get(t, &xp[v * NP]);
        RowPairs<T>::get(u, &gp[v * NP]);
      }
      // The rows were read through the generic proxy and the slot's next contents arrive through
      // the async proxy (bulk copy): without this fence the refill may overtake the reads.
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(s));  // the row is in registers: the stage may be refilled
      if (r >= rows) continue;                   // warp-uniform (a short last group)
      float rstd;
      row_stats<NP2, RMS>(xp, inv_dim, eps, rstd);
      const uint64_t rs2 = pair_of(rstd);
      uint64_t s1 = 0ull, s2 = 0ull;
#pragma unroll
      for (int v = 0; v < NV; v++)
#pragma unroll
        for (int h = 0; h < NP / 2; h++) {   // one float4 of weights = two pairs
          const ulonglong2 w2 = *reinterpret_cast<const ulonglong2 *>(w_sm + ((v * (V / 4) + h) * 32 + lane) * 4);
          const uint64_t wq[2] = {w2.x, w2.y};
#pragma unroll
          for (int q = 0; q < 2; q++) {
            const int j = v * NP + h * 2 + q;
            const uint64_t xhat = f2_mul(xp[j], rs2);
            const uint64_t dy = f2_mul(gp[j], wq[q]);
            dw_acc[j] = f2_fma(gp[j], xhat, dw_acc[j]);
            db_acc[j] = f2_add(db_acc[j], gp[j]);
            s1 = f2_add(s1, dy);
            s2 = f2_fma(dy, xhat, s2);
            xp[j] = xhat;
            gp[j] = dy;
          }
        }
      const float s1t = RMS ? 0.f : warp_sum(pair_total(s1));
      const float s2t = warp_sum(pair_total(s2));
      const uint64_t s1p = pair_of(s1t), s2p = pair_of(s2t), ninv = pair_of(-inv_dim);
      T *dr = dx + r * dim;
#pragma unroll
      for (int v = 0; v < NV; v++) {
        uint64_t o[NP];
#pragma unroll
        for (int j = 0; j < NP; j++) {
          const uint64_t t = f2_fma(xp[v * NP + j], s2p, s1p);
          o[j] = f2_mul(f2_fma(t, ninv, gp[v * NP + j]), rs2);
        }
        if (HAS_ADD) {
          uint64_t e[NP];
          RowPairs<T>::get(av[v], e);
#pragma unroll
          for (int j = 0; j < NP; j++) o[j] = f2_add(o[j], e[j]);
        }
        Vec16<T> t;
        RowPairs<T>::set(t, o);
        t.store(dr + (v * 32 + lane) * V);
      }
    }
  }
  // combine the four warps' column sums in warp order through the (now idle) ring
  __syncthreads();
  float *red = reinterpret_cast<float *>(lr_smem);  // [LR_WARPS][2 * dim]
  if (warp < LR_WARPS) {
    float *mine = red + (size_t)warp * 2 * dim;
#pragma unroll
    for (int v = 0; v < NV; v++)
#pragma unroll
      for (int h = 0; h < NP / 2; h++) {
        const int c = (v * 32 + lane) * V + h * 4;
        *reinterpret_cast<ulonglong2 *>(mine + c) = make_ulonglong2(dw_acc[v * NP + 2 * h], dw_acc[v * NP + 2 * h + 1]);
        *reinterpret_cast<ulonglong2 *>(mine + dim + c) = make_ulonglong2(db_acc[v * NP + 2 * h], db_acc[v * NP + 2 * h + 1]);
      }
  }
  __syncthreads();
  float *out = part + (size_t)blockIdx.x * 2 * dim;
  for (int c = threadIdx.x; c < 2 * dim; c += LR_THREADS) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < LR_WARPS; k++) t += red[(size_t)k * 2 * dim + c];
    out[c] = t;
  }
  if (*abort_flag) {  // a bounded wait ran out: let copies in flight land before the block's memory goes away
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
    if (threadIdx.x == 0 && err) atomicExch(err, 0xB1000000u | (uint32_t)(blockIdx.x & 0xFFFF));
  }
}

// Forward with the same structure: four worker warps, one row each per group, x streamed
// through a 4-stage bulk-copy ring; weight and bias rows sit in shared memory.  Measured at
// 16384 x 768 bf16: a deeper ring (up to all of a block's rows in flight at once) is slower,
// 19.0 against 16.5 us, and five or six resident blocks per SM (72 / 64 registers) change
// nothing; a launch over 4 rows takes 7 us in the same harness and 4x the rows add data at
// 6-7 TB/s, so what is left at this size is the fixed cost of a launch.
constexpr int LRF_STAGES = 4;

template <typename T, int NV, bool RMS>
__global__ void __launch_bounds__(LR_THREADS, 4)
ln_fwd_ring(const T *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b, T *__restrict__ y,
            int64_t rows, int dim, float eps, uint32_t *err) {
  using namespace tc;
  constexpr int V = Vec16<T>::N;
  extern __shared__ __align__(128) uint8_t lr_smem[];
  const uint32_t row_bytes = (uint32_t)dim * sizeof(T);
  const uint32_t stage_bytes = LR_WARPS * row_bytes;
  const uint32_t ring = smem_u32(lr_smem);
  const uint32_t bar = ring + LRF_STAGES * stage_bytes;
  auto full_bar = [&](int s) { return bar + 8u * s; };
  auto empty_bar = [&](int s) { return bar + 8u * (LRF_STAGES + s); };
  volatile uint32_t *abort_flag = (volatile uint32_t *)(lr_smem + LRF_STAGES * stage_bytes + 16 * LRF_STAGES);
  float *w_sm = reinterpret_cast<float *>(lr_smem + LRF_STAGES * stage_bytes + 128);
  float *b_sm = w_sm + dim;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n_groups = (rows + LR_WARPS - 1) / LR_WARPS;
  auto load_group = [&](int s, int64_t grp) {
    const int64_t r0 = grp * LR_WARPS;
    const uint32_t bytes = (uint32_t)min((int64_t)LR_WARPS, rows - r0) * row_bytes;
    if (elect_one()) {
      mbar_expect_tx(full_bar(s), bytes);
      bulk_load_1d(ring + s * stage_bytes, x + r0 * dim, bytes, full_bar(s));
    }
    __syncwarp();
  };
  // as in the backward kernel: the producer fills the ring while the workers fetch weight and bias
  if (warp == LR_WARPS) {
    if (lane == 0) {
      for (int s = 0; s < LRF_STAGES; s++) {
        mbar_init(full_bar(s), 1);
        mbar_init(empty_bar(s), LR_WARPS);
      }
      *abort_flag = 0;
      fence_barrier_init();
      fence_proxy_async();
    }
    __syncwarp();
  }
  grid_dependency_trigger();
  grid_dependency_wait();
  int p_i = 0;
  int64_t p_grp = blockIdx.x;
  if (warp == LR_WARPS)
    for (; p_i < LRF_STAGES && p_grp < n_groups; p_i++, p_grp += gridDim.x) load_group(p_i, p_grp);
  {
    // dim <= NV * 32 * V: a fixed trip count lets all of a thread's loads be in flight together
    constexpr int TRIPS = (NV * 32 * V + LR_THREADS - 1) / LR_THREADS;
    float wv[TRIPS], bv[TRIPS];
#pragma unroll
    for (int k = 0; k < TRIPS; k++) {
      const int c = threadIdx.x + k * LR_THREADS;
      wv[k] = c < dim ? w[c] : 0.f;
      bv[k] = (!RMS && c < dim) ? b[c] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < TRIPS; k++) {
      const int c = threadIdx.x + k * LR_THREADS;
      if (c < dim) {
        w_sm[lr_const_pos<V>(c)] = wv[k];
        b_sm[lr_const_pos<V>(c)] = bv[k];
      }
    }
  }
  __syncthreads();
  if (warp == LR_WARPS) {
    for (; p_grp < n_groups; p_grp += gridDim.x, p_i++) {
      const int s = p_i % LRF_STAGES;
      if (!mbar_wait(empty_bar(s), ((p_i / LRF_STAGES) & 1) ^ 1, abort_flag)) break;
      load_group(s, p_grp);
    }
  } else {
    const float inv_dim = 1.f / (float)dim;
    int i = 0;
    for (int64_t grp = blockIdx.x; grp < n_groups; grp += gridDim.x, i++) {
      const int s = i % LRF_STAGES;
      if (!mbar_wait(full_bar(s), (i / LRF_STAGES) & 1, abort_flag)) break;
      const int64_t r = grp * LR_WARPS + warp;
      const uint8_t *src = lr_smem + s * stage_bytes + warp * row_bytes;
      constexpr int NP = RowPairs<T>::NP, NP2 = NV * NP;
      uint64_t xp[NP2];
#pragma unroll
      for (int v = 0; v < NV; v++) {
        Vec16<T> t;
        t.load(reinterpret_cast<const T *>(src + (v * 32 + lane) * 16));
        RowPairs<T>::get(t, &xp[v * NP]);
      }
      fence_proxy_async();  // generic-proxy reads before the async-proxy refill of the slot
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(s));  // the row is in registers: the slot can be refilled
      if (r >= rows) continue;
      float rstd;
      row_stats<NP2, RMS>(xp, inv_dim, eps, rstd);
      const uint64_t rs2 = pair_of(rstd);
      T *yr = y + r * dim;
#pragma unroll
      for (int v = 0; v < NV; v++) {
        uint64_t o[NP];
#pragma unroll
        for (int h = 0; h < NP / 2; h++) {   // one float4 of weight and of bias = two pairs
          const int cp = ((v * (V / 4) + h) * 32 + lane) * 4;
          const ulonglong2 w2 = *reinterpret_cast<const ulonglong2 *>(w_sm + cp);
          if (RMS) {
            o[2 * h] = f2_mul(f2_mul(xp[v * NP + 2 * h], rs2), w2.x);
            o[2 * h + 1] = f2_mul(f2_mul(xp[v * NP + 2 * h + 1], rs2), w2.y);
          } else {
            const ulonglong2 b2 = *reinterpret_cast<const ulonglong2 *>(b_sm + cp);
            o[2 * h] = f2_fma(f2_mul(xp[v * NP + 2 * h], rs2), w2.x, b2.x);
            o[2 * h + 1] = f2_fma(f2_mul(xp[v * NP + 2 * h + 1], rs2), w2.y, b2.y);
          }
        }
        Vec16<T> t;
        RowPairs<T>::set(t, o);
        t.store(yr + (v * 32 + lane) * V);
      }
    }
  }
  if (*abort_flag) {  // a bounded wait ran out: let copies in flight land before the block's memory goes away
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
    if (threadIdx.x == 0 && err) atomicExch(err, 0xB2000000u | (uint32_t)(blockIdx.x & 0xFFFF));
  }
}

template <typename T, int NV, bool RMS>
static int launch_fwd_ring_nv(alpha_buf x, alpha_buf w, alpha_buf b, alpha_buf y, int64_t rows, int64_t dim, float eps) {
  const size_t smem = (size_t)LRF_STAGES * LR_WARPS * dim * sizeof(T) + 128 + 2 * dim * sizeof(float);
  static int attr = -1;
  if (attr != g_init_epoch) {
    ALPHA_CUDA(cudaFuncSetAttribute(ln_fwd_ring<T, NV, RMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr = g_init_epoch;
  }
  ALPHA_CUDA(launch_overlapped(OVL_NORM_FWD, ln_fwd_ring<T, NV, RMS>, dim3(grid_for(rows, LR_WARPS, 4)), dim3(LR_THREADS), smem,
                               (const T *)ptr<T>(x), (const float *)ptr<float>(w),
                               (const float *)(RMS ? nullptr : ptr<float>(b)), ptr<T>(y), rows, (int)dim, eps,
                               tc::tc_error_word()));
  return 0;
}
template <typename T, bool RMS>
static int launch_fwd_ring(int nv, alpha_buf x, alpha_buf w, alpha_buf b, alpha_buf y, int64_t rows, int64_t dim,
                           float eps) {
  constexpr int K = sizeof(T) == 2 ? 1 : 2;
  switch (nv) {
    case 1 * K: return launch_fwd_ring_nv<T, 1 * K, RMS>(x, w, b, y, rows, dim, eps);
    case 2 * K: return launch_fwd_ring_nv<T, 2 * K, RMS>(x, w, b, y, rows, dim, eps);
    case 3 * K: return launch_fwd_ring_nv<T, 3 * K, RMS>(x, w, b, y, rows, dim, eps);
    case 4 * K: return launch_fwd_ring_nv<T, 4 * K, RMS>(x, w, b, y, rows, dim, eps);
  }
  return set_error("layernorm forward: unsupported vector count %d", nv);
}

// ── generic fallback (any dim / alignment): one block per row, scalar accesses ──────────
template <typename T, bool RMS>
__global__ void __launch_bounds__(256) ln_fwd_block(const T *x, const float *w, const float *b, T *y, int64_t rows,
                                                    int dim, float eps) {
  __shared__ float red[32];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T *xr = x + r * dim;
    float s = 0.f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      const float v = to_f32(xr[c]);
      s += RMS ? v * v : v;
    }
    s = block_sum(s, red);
    float mean = 0.f, rstd;
    if (RMS) {
      rstd = rsqrtf(s / dim + eps);
    } else {
      mean = s / dim;
      float q = 0.f;
      for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        const float d = to_f32(xr[c]) - mean;
        q += d * d;
      }
      q = block_sum(q, red);
      rstd = 1.f / sqrtf(q / dim + eps);
    }
    for (int c = threadIdx.x; c < dim; c += blockDim.x)
      y[r * dim + c] = from_f32<T>((to_f32(xr[c]) - mean) * rstd * w[c] + (RMS ? 0.f : b[c]));
  }
}

// dx per row; also stores (mean, rstd) per row for the column kernel.
template <typename T, bool RMS>
__global__ void __launch_bounds__(256) ln_bwd_block(const T *x, const float *w, const T *g, const T *dx_add, T *dx,
                                                    float *stats, int64_t rows, int dim, float eps) {
  __shared__ float red[32];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T *xr = x + r * dim, *gr = g + r * dim;
    float s = 0.f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      const float v = to_f32(xr[c]);
      s += RMS ? v * v : v;
    }
    s = block_sum(s, red);
    float mean = 0.f, rstd;
    if (RMS) {
      rstd = rsqrtf(s / dim + eps);
    } else {
      mean = s / dim;
      float q = 0.f;
      for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        const float d = to_f32(xr[c]) - mean;
        q += d * d;
      }
      q = block_sum(q, red);
      rstd = 1.f / sqrtf(q / dim + eps);
    }
    float s1 = 0.f, s2 = 0.f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      const float dy = to_f32(gr[c]) * w[c];
      s1 += dy;
      s2 += dy * (to_f32(xr[c]) - mean) * rstd;
    }
    s1 = block_sum(s1, red);
    s2 = block_sum(s2, red);
    if (RMS) s1 = 0.f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      const float xhat = (to_f32(xr[c]) - mean) * rstd;
      const float dy = to_f32(gr[c]) * w[c];
      const float extra = dx_add ? to_f32(dx_add[r * dim + c]) : 0.f;
      dx[r * dim + c] = from_f32<T>(rstd * (dy - (s1 + xhat * s2) / dim) + extra);
    }
    if (threadIdx.x == 0) {
      stats[2 * r] = mean;
      stats[2 * r + 1] = rstd;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) ln_dwdb_cols(const T *x, const T *g, const float *stats, float *dw, float *db,
                                                    int64_t rows, int dim, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= dim) return;
  float a = 0.f, bsum = 0.f;
  for (int64_t r = 0; r < rows; r++) {
    const float gv = to_f32(g[r * dim + c]);
    a += gv * (to_f32(x[r * dim + c]) - stats[2 * r]) * stats[2 * r + 1];
    bsum += gv;
  }
  dw[c] = accumulate ? dw[c] + a : a;
  if (db) db[c] = accumulate ? db[c] + bsum : bsum;
}

template <typename T, bool RMS>
static int norm_fwd(alpha_buf x, alpha_buf w, alpha_buf b, alpha_buf y, int64_t rows, int64_t dim, float eps) {
  if (rows == 0 || dim == 0) return 0;
  ProfScope prof(PROF_NORM, 2.0 * rows * dim * sizeof(T));
  constexpr int V = Vec16<T>::N;
  const bool fast = dim % V == 0 && (x & 15) == 0 && (y & 15) == 0 && dim / V <= 32 * 8;
  constexpr int RK = sizeof(T) == 2 ? 1 : 2;
  if (fast && dim % (32 * V * RK) == 0 && dim / (32 * V) <= 4 * RK && rows >= 4 * LR_WARPS) {
    if (launch_fwd_ring<T, RMS>((int)(dim / (32 * V)), x, w, b, y, rows, dim, eps)) return 1;
  } else if (fast && dim / V <= 2 * LN_CTA && (w & 15) == 0 && (RMS || (b & 15) == 0)) {
    const int nvec = (int)(dim / V);
    if (nvec <= LN_CTA) {
      const int nt = (nvec + 31) / 32 * 32;
      ln_fwd_cta<T, 1, 2, RMS><<<grid_for(rows, 2, 10), nt, 0, g_stream>>>(ptr<T>(x), ptr<float>(w), ptr<float>(b),
                                                                            ptr<T>(y), rows, (int)dim, eps);
    } else {
      const int nt = ((nvec + 1) / 2 + 31) / 32 * 32;
      ln_fwd_cta<T, 2, 1, RMS><<<grid_for(rows, 1, 12), nt, 0, g_stream>>>(ptr<T>(x), ptr<float>(w), ptr<float>(b),
                                                                            ptr<T>(y), rows, (int)dim, eps);
    }
  } else if (fast) {
    const int nv = (int)((dim / V + 31) / 32);
    const int grid = grid_for(rows, LN_WARPS, 16);
#define LN_FWD_CASE(NV)                                                                                     \
  case NV:                                                                                                  \
    ln_fwd_warp<T, NV, RMS><<<grid, LN_WARPS * 32, 0, g_stream>>>(ptr<T>(x), ptr<float>(w), ptr<float>(b),  \
                                                                  ptr<T>(y), rows, (int)dim, eps);           \
    break;
    switch (nv) {
      LN_FWD_CASE(1) LN_FWD_CASE(2) LN_FWD_CASE(3) LN_FWD_CASE(4) LN_FWD_CASE(5) LN_FWD_CASE(6) LN_FWD_CASE(7)
      LN_FWD_CASE(8)
    }
#undef LN_FWD_CASE
  } else {
    ln_fwd_block<T, RMS><<<grid_for(rows, 1, 8), 256, 0, g_stream>>>(ptr<T>(x), ptr<float>(w), ptr<float>(b),
                                                                     ptr<T>(y), rows, (int)dim, eps);
  }
  ALPHA_LAUNCHED();
  return 0;
}

template <typename T, int NV, bool RMS, bool HAS_ADD>
static int launch_bwd_ring_nv(alpha_buf x, alpha_buf w, alpha_buf g, alpha_buf dx_add, alpha_buf dx, float *part,
                              int64_t rows, int64_t dim, float eps, int grid) {
  const size_t smem = (size_t)LR_STAGES * (HAS_ADD ? 3 : 2) * LR_WARPS * dim * sizeof(T) + 64 + dim * sizeof(float);
  static int attr = -1;
  if (attr != g_init_epoch) {
    ALPHA_CUDA(cudaFuncSetAttribute(ln_bwd_ring<T, NV, RMS, HAS_ADD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    200 * 1024));
    attr = g_init_epoch;
  }
  ALPHA_CUDA(launch_overlapped(OVL_NORM_BWD, ln_bwd_ring<T, NV, RMS, HAS_ADD>, dim3(grid), dim3(LR_THREADS), smem,
                               (const T *)ptr<T>(x), (const float *)ptr<float>(w), (const T *)ptr<T>(g),
                               (const T *)(HAS_ADD ? ptr<T>(dx_add) : nullptr), ptr<T>(dx), part, rows, (int)dim, eps,
                               tc::tc_error_word()));
  return 0;
}
template <typename T, bool RMS, bool HAS_ADD>
static int launch_bwd_ring(int nv, alpha_buf x, alpha_buf w, alpha_buf g, alpha_buf dx_add, alpha_buf dx, float *part,
                           int64_t rows, int64_t dim, float eps, int grid) {
  constexpr int K = sizeof(T) == 2 ? 1 : 2;  // lanes hold up to 32 elements: 4 bf16 vectors or 8 f32 vectors
  switch (nv) {
    case 1 * K: return launch_bwd_ring_nv<T, 1 * K, RMS, HAS_ADD>(x, w, g, dx_add, dx, part, rows, dim, eps, grid);
    case 2 * K: return launch_bwd_ring_nv<T, 2 * K, RMS, HAS_ADD>(x, w, g, dx_add, dx, part, rows, dim, eps, grid);
    case 3 * K: return launch_bwd_ring_nv<T, 3 * K, RMS, HAS_ADD>(x, w, g, dx_add, dx, part, rows, dim, eps, grid);
    case 4 * K: return launch_bwd_ring_nv<T, 4 * K, RMS, HAS_ADD>(x, w, g, dx_add, dx, part, rows, dim, eps, grid);
  }
  return set_error("layernorm backward: unsupported vector count %d", nv);
}

template <typename T, bool RMS>
static int norm_bwd(alpha_buf x, alpha_buf w, alpha_buf g, alpha_buf dx_add, alpha_buf dx, alpha_buf dw, alpha_buf db,
                    int64_t rows, int64_t dim, float eps, int accumulate) {
  if (dim == 0) return 0;
  if (rows == 0) {
    if (!accumulate) {
      ALPHA_CUDA(cudaMemsetAsync(ptr<void>(dw), 0, dim * 4, g_stream));
      if (db) ALPHA_CUDA(cudaMemsetAsync(ptr<void>(db), 0, dim * 4, g_stream));
    }
    return 0;
  }
  ProfScope prof(PROF_NORM, 3.0 * rows * dim * sizeof(T));
  constexpr int V = Vec16<T>::N;
  const size_t smem = (size_t)LN_WARPS * 2 * dim * sizeof(float);
  const bool fast = dim % V == 0 && (x & 15) == 0 && (g & 15) == 0 && (dx & 15) == 0 && (dx_add & 15) == 0 &&
                    dim / V <= 32 * 8;
  constexpr int RK = sizeof(T) == 2 ? 1 : 2;  // 16-byte vectors per 8 elements
  if (fast && dim % (32 * V * RK) == 0 && dim / (32 * V) <= 4 * RK && rows >= 4 * LR_WARPS) {
    // ring-fed warp-per-row kernel: 8, 16, 24 or 32 elements per lane
    const int nv = (int)(dim / (32 * V));
    const int grid = grid_for(rows, LR_WARPS, nv * V > 24 ? 2 : 3);
    void *part = nullptr;
    if (pool_alloc((size_t)grid * 2 * dim * sizeof(float), &part)) return 1;
    int rc = dx_add ? launch_bwd_ring<T, RMS, true>(nv, x, w, g, dx_add, dx, (float *)part, rows, dim, eps, grid)
                    : launch_bwd_ring<T, RMS, false>(nv, x, w, g, dx_add, dx, (float *)part, rows, dim, eps, grid);
    if (rc) { pool_free(part); return 1; }
    g_launches++;
    cudaError_t e = launch_overlapped(OVL_NORM_BWD, ln_reduce_partials, dim3((unsigned)((2 * dim + 31) / 32)), dim3(32, LN_RED_GROUPS), 0,
                                      (const float *)part, ptr<float>(dw), db ? ptr<float>(db) : (float *)nullptr, grid,
                                      (int)dim, accumulate);
    pool_free(part);
    if (e != cudaSuccess) return set_error("layernorm partial reduce launch -> %s", cudaGetErrorString(e));
  } else if (fast && dim / V <= 2 * LN_CTA && (w & 15) == 0) {
    const int nvec = (int)(dim / V);
    const int grid = nvec <= LN_CTA ? grid_for(rows, 2, 5) : grid_for(rows, 1, 4);
    void *part = nullptr;
    if (pool_alloc((size_t)grid * 2 * dim * sizeof(float), &part)) return 1;
    if (nvec <= LN_CTA)
      ln_bwd_cta<T, 1, 2, RMS><<<grid, (nvec + 31) / 32 * 32, 0, g_stream>>>(
          ptr<T>(x), ptr<float>(w), ptr<T>(g), dx_add ? ptr<T>(dx_add) : nullptr, ptr<T>(dx), (float *)part, rows,
          (int)dim, eps);
    else
      ln_bwd_cta<T, 2, 1, RMS><<<grid, ((nvec + 1) / 2 + 31) / 32 * 32, 0, g_stream>>>(
          ptr<T>(x), ptr<float>(w), ptr<T>(g), dx_add ? ptr<T>(dx_add) : nullptr, ptr<T>(dx), (float *)part, rows,
          (int)dim, eps);
    g_launches++;
    ln_reduce_partials<<<(unsigned)((2 * dim + 31) / 32), dim3(32, LN_RED_GROUPS), 0, g_stream>>>(
        (const float *)part, ptr<float>(dw), db ? ptr<float>(db) : nullptr, grid, (int)dim, accumulate);
    pool_free(part);
  } else if (fast && smem <= 48 * 1024) {
    const int nv = (int)((dim / V + 31) / 32);
    int grid = grid_for(rows, LN_WARPS, 4);
    void *part = nullptr;
    if (pool_alloc((size_t)grid * 2 * dim * sizeof(float), &part)) return 1;
#define LN_BWD_CASE(NV)                                                                                    \
  case NV:                                                                                                 \
    ln_bwd_warp<T, NV, RMS><<<grid, LN_WARPS * 32, smem, g_stream>>>(ptr<T>(x), ptr<float>(w), ptr<T>(g),   \
                                                                     dx_add ? ptr<T>(dx_add) : nullptr,     \
                                                                     ptr<T>(dx), (float *)part, rows,       \
                                                                     (int)dim, eps);                        \
    break;
    switch (nv) {
      LN_BWD_CASE(1) LN_BWD_CASE(2) LN_BWD_CASE(3) LN_BWD_CASE(4) LN_BWD_CASE(5) LN_BWD_CASE(6) LN_BWD_CASE(7)
      LN_BWD_CASE(8)
    }
#undef LN_BWD_CASE
    g_launches++;
    ln_reduce_partials<<<(unsigned)((2 * dim + 31) / 32), dim3(32, LN_RED_GROUPS), 0, g_stream>>>(
        (const float *)part, ptr<float>(dw), db ? ptr<float>(db) : nullptr, grid, (int)dim, accumulate);
    pool_free(part);
  } else {
    void *stats = nullptr;
    if (pool_alloc((size_t)rows * 2 * sizeof(float), &stats)) return 1;
    ln_bwd_block<T, RMS><<<grid_for(rows, 1, 8), 256, 0, g_stream>>>(ptr<T>(x), ptr<float>(w), ptr<T>(g),
                                                                     dx_add ? ptr<T>(dx_add) : nullptr, ptr<T>(dx),
                                                                     (float *)stats, rows, (int)dim, eps);
    g_launches++;
    ln_dwdb_cols<T><<<(unsigned)((dim + 127) / 128), 128, 0, g_stream>>>(ptr<T>(x), ptr<T>(g), (const float *)stats,
                                                                         ptr<float>(dw), db ? ptr<float>(db) : nullptr,
                                                                         rows, (int)dim, accumulate);
    pool_free(stats);
  }
  ALPHA_LAUNCHED();
  return 0;
}

}  // namespace alpha

using namespace alpha;

extern "C" {

int alpha_layernorm_fwd(alpha_buf x, alpha_buf w, alpha_buf b, alpha_buf y, int64_t rows, int64_t dim, float eps,
                        int dtype) {
  ALPHA_REQUIRE_INIT();
  if (dtype == ALPHA_F32) return norm_fwd<float, false>(x, w, b, y, rows, dim, eps);
  if (dtype == ALPHA_BF16) return norm_fwd<__nv_bfloat16, false>(x, w, b, y, rows, dim, eps);
  return set_error("alpha_layernorm_fwd: unsupported dtype %d", dtype);
}

int alpha_layernorm_bwd(alpha_buf x, alpha_buf w, alpha_buf g, alpha_buf dx, alpha_buf dw, alpha_buf db, int64_t rows,
                        int64_t dim, float eps, int dtype, int accumulate, alpha_buf dx_add) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(dw != 0 && db != 0, "alpha_layernorm_bwd: dw and db are required");
  if (dtype == ALPHA_F32) return norm_bwd<float, false>(x, w, g, dx_add, dx, dw, db, rows, dim, eps, accumulate);
  if (dtype == ALPHA_BF16) return norm_bwd<__nv_bfloat16, false>(x, w, g, dx_add, dx, dw, db, rows, dim, eps, accumulate);
  return set_error("alpha_layernorm_bwd: unsupported dtype %d", dtype);
}

int alpha_rmsnorm_fwd(alpha_buf x, alpha_buf w, alpha_buf y, int64_t rows, int64_t dim, float eps, int dtype) {
  ALPHA_REQUIRE_INIT();
  if (dtype == ALPHA_F32) return norm_fwd<float, true>(x, w, 0, y, rows, dim, eps);
  if (dtype == ALPHA_BF16) return norm_fwd<__nv_bfloat16, true>(x, w, 0, y, rows, dim, eps);
  return set_error("alpha_rmsnorm_fwd: unsupported dtype %d", dtype);
}

int alpha_rmsnorm_bwd(alpha_buf x, alpha_buf w, alpha_buf g, alpha_buf dx, alpha_buf dw, int64_t rows, int64_t dim,
                      float eps, int dtype, int accumulate, alpha_buf dx_add) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(dw != 0, "alpha_rmsnorm_bwd: dw is required");
  if (dtype == ALPHA_F32) return norm_bwd<float, true>(x, w, g, dx_add, dx, dw, 0, rows, dim, eps, accumulate);
  if (dtype == ALPHA_BF16) return norm_bwd<__nv_bfloat16, true>(x, w, g, dx_add, dx, dw, 0, rows, dim, eps, accumulate);
  return set_error("alpha_rmsnorm_bwd: unsupported dtype %d", dtype);
}

}  // extern "C"
