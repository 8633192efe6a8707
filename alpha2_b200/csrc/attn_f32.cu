// Causal flash attention, forward and backward, with fp32 arithmetic on the FMA pipes.
// This is the full-precision mode (fp32 parity configurations) and it accepts bf16
// storage too; the tensor-core kernels for bf16 live in attn_tc.cu.
//
// Contract: Backend.flashAttention / flashAttentionBackward
// (packages/core/src/interfaces.ts:127-135).  Math as in the reference kernels
// (packages/helios/src/kernels/attention.ts:427-477 forward, :1217-1231 and :1411-1427
// backward): s = scale*q.k ; optional soft cap s = cap*tanh(s/cap) ; keys after the query
// are masked ; online softmax ; O = P V ; LSE = m + ln(l).  Backward rebuilds P from LSE,
// D_i = dO_i . O_i, dS = P*(dP - D_i)*(1 - tanh^2)*scale.
//
// q/k/v/o are addressed through (batch, head, time) element strides so the kernel reads
// the fused QKV projection in place and writes O already head-merged; nothing is
// transposed or copied around it.  Tiles are 64 queries x 64 keys; 256 threads as a 16x16
// grid, each owning a 4x4 patch of the score tile and a 4 x (D/16) patch of the outputs.
// dK/dV and dQ are separate kernels (each output tile has one owner, no atomics, so the
// gradients are deterministic).
#include "common.cuh"

namespace alpha {

constexpr int BQ = 64, BKV = 64, PAD = 4;

struct AttnArgs {
  const void *q, *k, *v, *o, *d_o;
  void *out_o, *dq, *dk, *dv;
  float *lse;
  const float *lse_in;
  float *delta;  // [B,H,T] scratch: D_i
  int64_t q_sb, q_sh, q_st, o_sb, o_sh, o_st;
  int H, T;
  float scale, cap;
};

// global [rows x D] (row stride st) -> shared row-major [64][D+PAD], zero-filled past T
template <typename T, int D>
__device__ __forceinline__ void load_rows(float *dst, const T *src, int64_t st, int t0, int Tlen) {
  for (int e = threadIdx.x; e < 64 * D; e += 256) {
    const int r = e / D, c = e - r * D;
    const int t = t0 + r;
    dst[r * (D + PAD) + c] = t < Tlen ? to_f32(src[(int64_t)t * st + c]) : 0.f;
  }
}
// global [rows x D] -> shared transposed [D][64+PAD]
template <typename T, int D>
__device__ __forceinline__ void load_rows_t(float *dst, const T *src, int64_t st, int t0, int Tlen) {
  for (int e = threadIdx.x; e < 64 * D; e += 256) {
    const int r = e / D, c = e - r * D;
    const int t = t0 + r;
    dst[c * (64 + PAD) + r] = t < Tlen ? to_f32(src[(int64_t)t * st + c]) : 0.f;
  }
}

// acc[i][j] = sum_d A[ty*4+i][d] * Bt[d][tx*4+j]   (A row-major [64][D+PAD], Bt [D][64+PAD])
template <int D>
__device__ __forceinline__ void tile_abt(float (&acc)[4][4], const float *A, const float *Bt, int ty, int tx) {
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
#pragma unroll 8
  for (int d = 0; d < D; d++) {
    const float4 b4 = *reinterpret_cast<const float4 *>(&Bt[d * (64 + PAD) + tx * 4]);
    const float b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float a = A[(ty * 4 + i) * (D + PAD) + d];
#pragma unroll
      for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a, b[j], acc[i][j]);
    }
  }
}

// out[i][j] += sum_r W[r][ty*4+i] * X[r][tx*CPT+j]  (W [64][64+PAD] indexed [r][row], X row-major)
template <int D, bool W_TRANSPOSED>
__device__ __forceinline__ void tile_wx(float (&out)[4][D / 16], const float *W, const float *X, int ty, int tx) {
  constexpr int CPT = D / 16;
#pragma unroll 4
  for (int r = 0; r < 64; r++) {
    float w[4];
#pragma unroll
    for (int i = 0; i < 4; i++)
      w[i] = W_TRANSPOSED ? W[r * (64 + PAD) + ty * 4 + i] : W[(ty * 4 + i) * (64 + PAD) + r];
#pragma unroll
    for (int j = 0; j < CPT; j++) {
      const float x = X[r * (D + PAD) + tx * CPT + j];
#pragma unroll
      for (int i = 0; i < 4; i++) out[i][j] = fmaf(w[i], x, out[i][j]);
    }
  }
}

__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T, int D>
__global__ void __launch_bounds__(256) attn_fwd_kernel(AttnArgs a) {
  extern __shared__ __align__(16) float sm[];
  constexpr int CPT = D / 16;
  float *Qs = sm;                          // [64][D+PAD]
  float *Kt = Qs + 64 * (D + PAD);         // [D][64+PAD]
  float *Vs = Kt + D * (64 + PAD);         // [64][D+PAD]
  float *Ps = Vs + 64 * (D + PAD);         // [64][64+PAD]
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int qb = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh - b * a.H;
  const int q0 = qb * BQ;
  const T *qp = (const T *)a.q + b * a.q_sb + h * a.q_sh;
  const T *kp = (const T *)a.k + b * a.q_sb + h * a.q_sh;
  const T *vp = (const T *)a.v + b * a.q_sb + h * a.q_sh;
  load_rows<T, D>(Qs, qp, a.q_st, q0, a.T);
  float m[4], l[4], o[4][CPT];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int j = 0; j < CPT; j++) o[i][j] = 0.f;
  }
  for (int kb = 0; kb <= qb; kb++) {
    const int k0 = kb * BKV;
    __syncthreads();
    load_rows_t<T, D>(Kt, kp, a.q_st, k0, a.T);
    load_rows<T, D>(Vs, vp, a.q_st, k0, a.T);
    __syncthreads();
    float s[4][4];
    tile_abt<D>(s, Qs, Kt, ty, tx);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int qi = q0 + ty * 4 + i;
      float mloc = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int kj = k0 + tx * 4 + j;
        float x = s[i][j] * a.scale;
        if (a.cap > 0.f) x = a.cap * tanhf(x / a.cap);
        if (kj > qi || kj >= a.T) x = -INFINITY;
        s[i][j] = x;
        mloc = fmaxf(mloc, x);
      }
      mloc = half_warp_max(mloc);
      const float mnew = fmaxf(m[i], mloc);
      const float corr = (mnew == -INFINITY) ? 1.f : expf(m[i] - mnew);
      float lsum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float p = (mnew == -INFINITY) ? 0.f : expf(s[i][j] - mnew);
        Ps[(ty * 4 + i) * (64 + PAD) + tx * 4 + j] = p;
        lsum += p;
      }
      lsum = half_warp_sum(lsum);
      l[i] = l[i] * corr + lsum;
      m[i] = mnew;
#pragma unroll
      for (int j = 0; j < CPT; j++) o[i][j] *= corr;
    }
    __syncthreads();
    tile_wx<D, false>(o, Ps, Vs, ty, tx);
  }
  T *op = (T *)a.out_o + b * a.o_sb + h * a.o_sh;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int qi = q0 + ty * 4 + i;
    if (qi >= a.T) continue;
    const float inv = 1.f / l[i];
#pragma unroll
    for (int j = 0; j < CPT; j++) op[(int64_t)qi * a.o_st + tx * CPT + j] = from_f32<T>(o[i][j] * inv);
    if (tx == 0) a.lse[(int64_t)bh * a.T + qi] = m[i] + logf(l[i]);
  }
}

// delta[bh, t] = sum_d dO[t,d] * O[t,d]; one warp per row
template <typename T>
__global__ void __launch_bounds__(256) attn_delta_kernel(AttnArgs a, int D, int64_t rows) {
  const int lane = threadIdx.x & 31;
  const int64_t wg = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  for (int64_t r = wg; r < rows; r += (int64_t)gridDim.x * 8) {
    const int64_t bh = r / a.T;
    const int t = (int)(r - bh * a.T);
    const int b = (int)(bh / a.H), h = (int)(bh - (int64_t)b * a.H);
    const T *op = (const T *)a.o + b * a.o_sb + h * a.o_sh + (int64_t)t * a.o_st;
    const T *dp = (const T *)a.d_o + b * a.o_sb + h * a.o_sh + (int64_t)t * a.o_st;
    float s = 0.f;
    for (int c = lane; c < D; c += 32) s += to_f32(op[c]) * to_f32(dp[c]);
    s = warp_sum(s);
    if (lane == 0) a.delta[r] = s;
  }
}

// Recomputes, for the tile (q0, k0): P -> Ps (optional) and dS -> dSs, both [q][key].
template <int D>
__device__ __forceinline__ void recompute_p_ds(const AttnArgs &a, const float *Qs, const float *Kt, const float *dOs,
                                               const float *Vt, const float *lse_s, const float *delta_s, float *Ps,
                                               float *dSs, int q0, int k0, int ty, int tx) {
  float s[4][4], dp[4][4];
  tile_abt<D>(s, Qs, Kt, ty, tx);
  tile_abt<D>(dp, dOs, Vt, ty, tx);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int qi = q0 + ty * 4 + i;
    const float lse = lse_s[ty * 4 + i], dl = delta_s[ty * 4 + i];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int kj = k0 + tx * 4 + j;
      float x = s[i][j] * a.scale, dcap = 1.f;
      if (a.cap > 0.f) {
        const float th = tanhf(x / a.cap);
        x = a.cap * th;
        dcap = 1.f - th * th;
      }
      const bool dead = kj > qi || kj >= a.T || qi >= a.T;
      const float p = dead ? 0.f : expf(x - lse);
      const float ds = p * (dp[i][j] - dl) * dcap * a.scale;
      if (Ps) Ps[(ty * 4 + i) * (64 + PAD) + tx * 4 + j] = p;
      dSs[(ty * 4 + i) * (64 + PAD) + tx * 4 + j] = ds;
    }
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(256) attn_bwd_dkv_kernel(AttnArgs a) {
  extern __shared__ __align__(16) float sm[];
  constexpr int CPT = D / 16;
  float *Kt = sm;                           // [D][64+PAD]
  float *Vt = Kt + D * (64 + PAD);          // [D][64+PAD]
  float *Qs = Vt + D * (64 + PAD);          // [64][D+PAD]
  float *dOs = Qs + 64 * (D + PAD);         // [64][D+PAD]
  float *Ps = dOs + 64 * (D + PAD);         // [64][64+PAD]
  float *dSs = Ps + 64 * (64 + PAD);        // [64][64+PAD]
  float *lse_s = dSs + 64 * (64 + PAD);     // [64]
  float *delta_s = lse_s + 64;              // [64]
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int kb = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh - b * a.H;
  const int k0 = kb * BKV;
  const int64_t qoff = b * a.q_sb + h * a.q_sh, ooff = b * a.o_sb + h * a.o_sh;
  load_rows_t<T, D>(Kt, (const T *)a.k + qoff, a.q_st, k0, a.T);
  load_rows_t<T, D>(Vt, (const T *)a.v + qoff, a.q_st, k0, a.T);
  float dk[4][CPT], dv[4][CPT];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < CPT; j++) dk[i][j] = dv[i][j] = 0.f;
  const int n_qb = (a.T + BQ - 1) / BQ;
  for (int qb = kb; qb < n_qb; qb++) {
    const int q0 = qb * BQ;
    __syncthreads();
    load_rows<T, D>(Qs, (const T *)a.q + qoff, a.q_st, q0, a.T);
    load_rows<T, D>(dOs, (const T *)a.d_o + ooff, a.o_st, q0, a.T);
    if (threadIdx.x < 64) {
      const int t = q0 + threadIdx.x;
      lse_s[threadIdx.x] = t < a.T ? a.lse_in[(int64_t)bh * a.T + t] : 0.f;
      delta_s[threadIdx.x] = t < a.T ? a.delta[(int64_t)bh * a.T + t] : 0.f;
    }
    __syncthreads();
    recompute_p_ds<D>(a, Qs, Kt, dOs, Vt, lse_s, delta_s, Ps, dSs, q0, k0, ty, tx);
    __syncthreads();
    tile_wx<D, true>(dv, Ps, dOs, ty, tx);   // dV[key] += sum_q P[q][key] dO[q]
    tile_wx<D, true>(dk, dSs, Qs, ty, tx);   // dK[key] += sum_q dS[q][key] Q[q]
  }
  T *dkp = (T *)a.dk + qoff, *dvp = (T *)a.dv + qoff;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int kj = k0 + ty * 4 + i;
    if (kj >= a.T) continue;
#pragma unroll
    for (int j = 0; j < CPT; j++) {
      dkp[(int64_t)kj * a.q_st + tx * CPT + j] = from_f32<T>(dk[i][j]);
      dvp[(int64_t)kj * a.q_st + tx * CPT + j] = from_f32<T>(dv[i][j]);
    }
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(256) attn_bwd_dq_kernel(AttnArgs a) {
  extern __shared__ __align__(16) float sm[];
  constexpr int CPT = D / 16;
  float *Kt = sm;                           // [D][64+PAD]
  float *Vt = Kt + D * (64 + PAD);          // [D][64+PAD]
  float *Qs = Vt + D * (64 + PAD);          // [64][D+PAD]
  float *dOs = Qs + 64 * (D + PAD);         // [64][D+PAD]
  float *Ks = dOs + 64 * (D + PAD);         // [64][D+PAD]
  float *dSs = Ks + 64 * (D + PAD);         // [64][64+PAD]
  float *lse_s = dSs + 64 * (64 + PAD);
  float *delta_s = lse_s + 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int qb = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh - b * a.H;
  const int q0 = qb * BQ;
  const int64_t qoff = b * a.q_sb + h * a.q_sh, ooff = b * a.o_sb + h * a.o_sh;
  load_rows<T, D>(Qs, (const T *)a.q + qoff, a.q_st, q0, a.T);
  load_rows<T, D>(dOs, (const T *)a.d_o + ooff, a.o_st, q0, a.T);
  if (threadIdx.x < 64) {
    const int t = q0 + threadIdx.x;
    lse_s[threadIdx.x] = t < a.T ? a.lse_in[(int64_t)bh * a.T + t] : 0.f;
    delta_s[threadIdx.x] = t < a.T ? a.delta[(int64_t)bh * a.T + t] : 0.f;
  }
  float dq[4][CPT];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < CPT; j++) dq[i][j] = 0.f;
  for (int kb = 0; kb <= qb; kb++) {
    const int k0 = kb * BKV;
    __syncthreads();
    load_rows_t<T, D>(Kt, (const T *)a.k + qoff, a.q_st, k0, a.T);
    load_rows_t<T, D>(Vt, (const T *)a.v + qoff, a.q_st, k0, a.T);
    load_rows<T, D>(Ks, (const T *)a.k + qoff, a.q_st, k0, a.T);
    __syncthreads();
    recompute_p_ds<D>(a, Qs, Kt, dOs, Vt, lse_s, delta_s, nullptr, dSs, q0, k0, ty, tx);
    __syncthreads();
    tile_wx<D, false>(dq, dSs, Ks, ty, tx);  // dQ[q] += sum_key dS[q][key] K[key]
  }
  T *dqp = (T *)a.dq + qoff;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int qi = q0 + ty * 4 + i;
    if (qi >= a.T) continue;
#pragma unroll
    for (int j = 0; j < CPT; j++) dqp[(int64_t)qi * a.q_st + tx * CPT + j] = from_f32<T>(dq[i][j]);
  }
}

template <int D> constexpr size_t fwd_smem() { return sizeof(float) * (2 * 64 * (D + PAD) + D * (64 + PAD) + 64 * (64 + PAD)); }
template <int D> constexpr size_t dkv_smem() {
  return sizeof(float) * (2 * D * (64 + PAD) + 2 * 64 * (D + PAD) + 2 * 64 * (64 + PAD) + 128);
}
template <int D> constexpr size_t dq_smem() {
  return sizeof(float) * (2 * D * (64 + PAD) + 3 * 64 * (D + PAD) + 64 * (64 + PAD) + 128);
}

template <typename T, int D>
static int fwd_launch(const AttnArgs &a, int64_t batch) {
  static int attr = -1;
  if (attr != g_init_epoch) {
    ALPHA_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fwd_smem<D>()));
    attr = g_init_epoch;
  }
  dim3 grid((unsigned)((a.T + BQ - 1) / BQ), (unsigned)(batch * a.H));
  attn_fwd_kernel<T, D><<<grid, 256, fwd_smem<D>(), g_stream>>>(a);
  ALPHA_LAUNCHED();
  return 0;
}

template <typename T, int D>
static int bwd_launch(const AttnArgs &a, int64_t batch) {
  static int attr = -1;
  if (attr != g_init_epoch) {
    ALPHA_CUDA(cudaFuncSetAttribute(attn_bwd_dkv_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dkv_smem<D>()));
    ALPHA_CUDA(cudaFuncSetAttribute(attn_bwd_dq_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dq_smem<D>()));
    attr = g_init_epoch;
  }
  const int64_t rows = batch * a.H * a.T;
  attn_delta_kernel<T><<<grid_for(rows, 8, 8), 256, 0, g_stream>>>(a, D, rows);
  g_launches++;
  dim3 grid((unsigned)((a.T + BQ - 1) / BQ), (unsigned)(batch * a.H));
  attn_bwd_dkv_kernel<T, D><<<grid, 256, dkv_smem<D>(), g_stream>>>(a);
  g_launches++;
  attn_bwd_dq_kernel<T, D><<<grid, 256, dq_smem<D>(), g_stream>>>(a);
  ALPHA_LAUNCHED();
  return 0;
}

static int check_params(const alpha_attn_params_t *p, const char *who) {
  ALPHA_CHECK(p != nullptr, "%s: null params", who);
  ALPHA_CHECK(p->D == 16 || p->D == 32 || p->D == 64 || p->D == 128, "%s: head dim %lld not in {16,32,64,128}", who,
              (long long)p->D);
  ALPHA_CHECK(p->dtype == ALPHA_F32 || p->dtype == ALPHA_BF16, "%s: unsupported dtype %d", who, p->dtype);
  ALPHA_CHECK(p->batch * p->heads <= 65535, "%s: batch*heads > 65535", who);
  return 0;
}

int attn_f32_fwd(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf o, alpha_buf lse, const alpha_attn_params_t *p) {
  if (check_params(p, "alpha_flash_attn_fwd")) return 1;
  if (p->batch * p->heads * p->T == 0) return 0;
  ProfScope prof(PROF_ATTN_FWD, 4.0 * p->batch * p->heads * (double)p->T * p->T * p->D);
  AttnArgs a{};
  a.q = ptr<void>(q); a.k = ptr<void>(k); a.v = ptr<void>(v); a.out_o = ptr<void>(o); a.lse = ptr<float>(lse);
  a.q_sb = p->q_sb; a.q_sh = p->q_sh; a.q_st = p->q_st; a.o_sb = p->o_sb; a.o_sh = p->o_sh; a.o_st = p->o_st;
  a.H = (int)p->heads; a.T = (int)p->T; a.scale = p->scale; a.cap = p->soft_cap;
#define FWD_CASE(DD)                                                                      \
  case DD:                                                                                \
    return p->dtype == ALPHA_F32 ? fwd_launch<float, DD>(a, p->batch) : fwd_launch<__nv_bfloat16, DD>(a, p->batch);
  switch (p->D) { FWD_CASE(16) FWD_CASE(32) FWD_CASE(64) FWD_CASE(128) }
#undef FWD_CASE
  return 1;
}

int attn_f32_bwd(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf o, alpha_buf d_o, alpha_buf lse, alpha_buf dq,
                 alpha_buf dk, alpha_buf dv, const alpha_attn_params_t *p) {
  if (check_params(p, "alpha_flash_attn_bwd")) return 1;
  if (p->batch * p->heads * p->T == 0) return 0;
  ProfScope prof(PROF_ATTN_BWD, 8.0 * p->batch * p->heads * (double)p->T * p->T * p->D);
  AttnArgs a{};
  a.q = ptr<void>(q); a.k = ptr<void>(k); a.v = ptr<void>(v); a.o = ptr<void>(o); a.d_o = ptr<void>(d_o);
  a.lse_in = ptr<float>(lse); a.dq = ptr<void>(dq); a.dk = ptr<void>(dk); a.dv = ptr<void>(dv);
  a.q_sb = p->q_sb; a.q_sh = p->q_sh; a.q_st = p->q_st; a.o_sb = p->o_sb; a.o_sh = p->o_sh; a.o_st = p->o_st;
  a.H = (int)p->heads; a.T = (int)p->T; a.scale = p->scale; a.cap = p->soft_cap;
  void *delta = nullptr;
  if (pool_alloc((size_t)p->batch * p->heads * p->T * sizeof(float), &delta)) return 1;
  a.delta = (float *)delta;
  int rc = 1;
#define BWD_CASE(DD)                                                                                      \
  case DD:                                                                                                \
    rc = p->dtype == ALPHA_F32 ? bwd_launch<float, DD>(a, p->batch) : bwd_launch<__nv_bfloat16, DD>(a, p->batch); \
    break;
  switch (p->D) { BWD_CASE(16) BWD_CASE(32) BWD_CASE(64) BWD_CASE(128) }
#undef BWD_CASE
  pool_free(delta);
  return rc;
}

}  // namespace alpha
