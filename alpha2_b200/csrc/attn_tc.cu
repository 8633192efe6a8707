// Causal flash attention for bf16 on the tcgen05 tensor cores (head dim 64).
//
// Contract and math: Backend.flashAttention / flashAttentionBackward
// (packages/core/src/interfaces.ts:127-135; packages/helios/src/kernels/attention.ts:427-477,
// 552-558 forward, :1217-1231, 1411-1427 backward) — s = scale*q.k, optional soft cap
// cap*tanh(s/cap), keys after the query masked, online softmax, O = P V, LSE = m + ln(l);
// backward rebuilds P from LSE, D_i = dO_i.O_i, dS = P*(dP - D_i)*(1 - tanh^2)*scale.
// q/k/v are read in place from the fused QKV projection through (batch, head, time)
// strides by 4-D TMA tensor maps; O is written head-merged.
//
// Forward, one CTA per (batch, head, 128 queries); 192 threads:
//   warp 0     TMA producer: Q once, then K (2 stages) and V (1 stage) per 128-key block
//   warp 1     MMA issuer:   S = Q K^T  (128x128x64, both operands K-major) into TMEM,
//                            O += P V   (128x64x128, P K-major from shared memory,
//                                        V as an N-major operand read in place)
//   warps 2-5  softmax: one query row per thread (= one TMEM lane): row max, exp2, row sum,
//              P -> bf16 -> 128B-swizzled shared memory; O is rescaled in TMEM only when the
//              running max has moved by more than 2^8 (the stale max keeps P <= 2^8).
// Two CTAs fit on an SM (96 KB shared memory, 256 TMEM columns each), so one CTA's softmax
// overlaps the other's MMAs.  Single CTAs (no cluster).  Every wait is bounded.
// Model work: forward 4*B*H*T^2*D flop (causal tiles are skipped, so about half is executed).
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "tc_common.cuh"

namespace alpha {

using namespace tc;

constexpr int AT_THREADS = 192;
constexpr int AT_TILE = 128 * 64 * 2;  // one 128-row x 64-col bf16 tile, 16 KB

struct AttnTcArgs {
  void *o;
  float *lse;
  int64_t o_sb, o_sh, o_st;
  int H, T;
  float scale, cap;
  uint32_t *err;
};

// shared-memory map (bytes from the 1024-aligned base)
constexpr int AF_Q = 0;
constexpr int AF_K = AT_TILE;                 // 2 stages
constexpr int AF_V = AF_K + 2 * AT_TILE;      // 1 stage
constexpr int AF_P = AF_V + AT_TILE;          // 2 tiles: keys 0-63, 64-127
constexpr int AF_BAR = AF_P + 2 * AT_TILE;
constexpr int AF_TOTAL = AF_BAR + 128;
constexpr int AF_DYN = AF_TOTAL + 1024;

__global__ void __launch_bounds__(AT_THREADS, 2)
attn_tc_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, AttnTcArgs a) {
  extern __shared__ uint8_t at_smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)at_smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sb = smem_u32(smem);
  const uint32_t bar = sb + AF_BAR;
  const uint32_t q_full = bar, k_full0 = bar + 8, k_empty0 = bar + 24, v_full = bar + 40, v_empty = bar + 48,
                 s_full = bar + 56, p_ready = bar + 64, pv_done = bar + 72;
  uint32_t *tmem_slot = (uint32_t *)(smem + AF_BAR + 80);
  volatile uint32_t *abort_flag = (volatile uint32_t *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qb = (a.T + 127) / 128;
  const int qb = n_qb - 1 - (int)blockIdx.x;  // long rows first
  const int bh = blockIdx.y;
  const int b = bh / a.H, h = bh - b * a.H;
  const int q0 = qb * 128;
  const int nb = qb + 1;  // key blocks 0..qb
  constexpr uint32_t TMEM_COLS = 256;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full0, 1); mbar_init(k_full0 + 8, 1);
    mbar_init(k_empty0, 1); mbar_init(k_empty0 + 8, 1);
    mbar_init(v_full, 1); mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 4);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  grid_dependency_trigger();
  grid_dependency_wait();  // set-up above is SM-local; global memory is touched from here on
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tO = tmem_base + 128;

  if (warp == 0) {
    // TMA producer: the warp runs the loop, one elected lane issues
    if (elect_one()) {
      tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
      mbar_expect_tx(q_full, AT_TILE);
      tma_load_4d(sb + AF_Q, &tmap_q, q_full, 0, q0, h, b);
    }
    __syncwarp();
    for (int j = 0; j < nb; j++) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(k_empty0 + 8 * st, ph ^ 1, abort_flag)) break;
      if (elect_one()) {
        mbar_expect_tx(k_full0 + 8 * st, AT_TILE);
        tma_load_4d(sb + AF_K + st * AT_TILE, &tmap_k, k_full0 + 8 * st, 0, j * 128, h, b);
      }
      __syncwarp();
      if (!mbar_wait(v_empty, (j & 1) ^ 1, abort_flag)) break;
      if (elect_one()) {
        mbar_expect_tx(v_full, AT_TILE);
        tma_load_4d(sb + AF_V, &tmap_v, v_full, 0, j * 128, h, b);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // MMA issuer: warp-uniform control flow and descriptors, one elected lane issues
    constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false);
    constexpr uint32_t idesc_pv = make_idesc_bf16(128, 64, false, true);
    const uint64_t d_q = make_smem_desc(sb + AF_Q, 16, 1024), d_k = make_smem_desc(sb + AF_K, 16, 1024);
    const uint64_t d_p = make_smem_desc(sb + AF_P, 16, 1024), d_v = make_smem_desc(sb + AF_V, AT_TILE, 1024);
    bool ok = mbar_wait(q_full, 0, abort_flag);
    auto issue_pv = [&](int j) -> bool {  // O (+)= P(j) V(j)
      if (!mbar_wait(p_ready, j & 1, abort_flag)) return false;
      if (!mbar_wait(v_full, j & 1, abort_flag)) return false;
      tc_fence_after();
      const uint32_t first = j > 0 ? 1u : 0u;
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < 8; kk++)
          mma_bf16_ss(tO, d_p + (uint64_t)(((kk >> 2) * AT_TILE + (kk & 3) * 32) >> 4), d_v + kk * 128, idesc_pv,
                      kk > 0 ? 1u : first);
        mma_commit(v_empty);
        mma_commit(pv_done);
      }
      __syncwarp();
      return true;
    };
    for (int j = 0; j < nb && ok; j++) {
      if (j > 0 && !issue_pv(j - 1)) { ok = false; break; }
      const int st = j & 1;
      if (!mbar_wait(k_full0 + 8 * st, (j >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint64_t kd = d_k + (uint64_t)((st * AT_TILE) >> 4);
      const uint32_t freed = k_empty0 + 8 * st;
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < 4; kk++) mma_bf16_ss(tS, d_q + kk * 2, kd + kk * 2, idesc_qk, kk > 0 ? 1u : 0u);
        mma_commit(freed);
        mma_commit(s_full);
      }
      __syncwarp();
    }
    if (ok) issue_pv(nb - 1);
  } else {
    // ── softmax warps: thread <-> query row <-> TMEM lane ────────────────────
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    const bool capped = a.cap > 0.f;
    const float c1 = capped ? a.scale / a.cap : a.scale * LOG2E;  // argument scale
    const float c2 = a.cap * LOG2E;                               // capped: x2 = c2 * tanh(c1 * s)
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    uint8_t *p_row = smem + AF_P + row * 128;
    for (int j = 0; j < nb && ok; j++) {
      if (!mbar_wait(s_full, j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool diag = (j == qb);
      // pass 1: row max of the raw scores (the score transform is monotonic)
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; c++) {
        uint32_t r[32];
        tmem_ld_32x32(tS + lane_off + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i++) {
          const float s = __uint_as_float(r[i]);
          if (!diag || c * 32 + i <= row) mx = fmaxf(mx, s);
        }
      }
      const float m_blk = capped ? c2 * tanh_approx(c1 * mx) : c1 * mx;
      const float m_new = fmaxf(m_used, m_blk);
      const bool need = m_new > m_used + 8.f;  // also true while m_used is -inf
      if (j > 0) {
        if (!mbar_wait(pv_done, (j - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, need)) {
          const float alpha = need ? ex2_approx(m_used - m_new) : 1.f;
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < 2; c++) {
            uint32_t r[32];
            tmem_ld_32x32(tO + lane_off + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32(tO + lane_off + c * 32, r);
          }
          tmem_st_wait();
        }
      }
      if (need) m_used = m_new;
      // pass 2: P = exp2(x2 - m_used) -> bf16 -> swizzled shared memory
      float lsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; c++) {
        uint32_t r[32];
        tmem_ld_32x32(tS + lane_off + c * 32, r);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0, p1;
          {
            const float s = __uint_as_float(r[i]);
            const float x2 = capped ? c2 * tanh_approx(c1 * s) : c1 * s;
            p0 = (diag && c * 32 + i > row) ? 0.f : ex2_approx(x2 - m_used);
          }
          {
            const float s = __uint_as_float(r[i + 1]);
            const float x2 = capped ? c2 * tanh_approx(c1 * s) : c1 * s;
            p1 = (diag && c * 32 + i + 1 > row) ? 0.f : ex2_approx(x2 - m_used);
          }
          const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
          // the row sum uses the rounded values that the tensor core will multiply
          const float2 back = __bfloat1622float2(pk);
          lsum += back.x + back.y;
          packed[i >> 1] = *reinterpret_cast<const uint32_t *>(&pk);
        }
        uint8_t *tile_row = p_row + (c >> 1) * AT_TILE;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const int chunk = ((c & 1) * 4 + q) ^ (row & 7);
          *reinterpret_cast<uint4 *>(tile_row + chunk * 16) =
              make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        }
      }
      l += lsum;
      fence_proxy_async();  // generic-proxy stores -> visible to the tensor core's reads
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    if (ok && mbar_wait(pv_done, (nb - 1) & 1, abort_flag)) {
      tc_fence_after();
      const int qi = q0 + row;
      const float inv = 1.f / l;
      __nv_bfloat16 *orow = (__nv_bfloat16 *)a.o + (int64_t)b * a.o_sb + (int64_t)h * a.o_sh + (int64_t)qi * a.o_st;
#pragma unroll 1
      for (int c = 0; c < 2; c++) {
        uint32_t r[32];
        tmem_ld_32x32(tO + lane_off + c * 32, r);
        tmem_ld_wait();
        if (qi < a.T) {
#pragma unroll
          for (int q = 0; q < 4; q++) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = __uint_as_float(r[q * 8 + i]) * inv;
            Vec16<__nv_bfloat16> v;
            v.set(f);
            v.store(orow + c * 32 + q * 8);
          }
        }
      }
      if (qi < a.T) a.lse[(int64_t)bh * a.T + qi] = (m_used + log2f(l)) * 0.6931471805599453f;
    }
  }

  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
    if (threadIdx.x == 0 && a.err) atomicExch(a.err, 0xA7000000u | (uint32_t)(blockIdx.x & 0xFFFF));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ── backward ────────────────────────────────────────────────────────────────
// One pass over the causal (query block, key block) tiles; every output element has one owner
// and nothing is added with atomics, so gradients are bit-reproducible:
//   main kernel: CTA = (batch, head, 128 keys), loops over the query blocks at or after it.
//     Per tile it computes S = Q K^T and dP = dO V^T on the tensor cores into TMEM; sixteen math
//     warps (32 query rows x 32 key columns each) turn them into P = exp2(x2 - lse2) and
//     dS = P*(dP - D)*(1 - tanh^2)*scale, round to bf16 and store them as
//     [query rows][key columns] 128B-swizzled tiles; three products follow: dV += P^T dO and
//     dK += dS^T Q (accumulated in TMEM over the item, the tiles read M-major: the tensor core
//     transposes through the descriptor) and the tile's contribution to dQ, dS K (dS read
//     K-major, K read N-major), which goes out as fp32 to a workspace slab per (query block,
//     key block) — 5 products and one pass of the score arithmetic per tile;
//   reduce kernel: dQ[query block] = the slabs of its key blocks added in key-block order.
// Q, dO, K, V tiles are used both K-major (score products) and N-major (gradient products)
// from the same bytes.  (Q, dO) pairs stream through a 3-stage TMA ring.
struct AttnBwdArgs {
  void *dq, *dk, *dv;
  float *dq_part;   // fp32 dQ contributions, [batch*head][pair(qb, kb) = qb(qb+1)/2 + kb][128 rows][64]
  const float *lse, *delta;
  int64_t q_sb, q_sh, q_st;
  int H, T;
  float scale, cap;
  uint32_t *err;
};

// delta[bh*T + t] = sum_d dO[t,d] * O[t,d]; eight threads per row (64 elements), one 16-byte
// load of O and of dO each, shuffle-sum inside the group of eight; rows are walked grid-stride
// so that many loads are in flight per SM.
__global__ void __launch_bounds__(256) attn_tc_delta_kernel(const __nv_bfloat16 *__restrict__ o,
                                                            const __nv_bfloat16 *__restrict__ d_o, float *delta,
                                                            int64_t o_sb, int64_t o_sh, int64_t o_st, int H, int T,
                                                            int64_t rows) {
  const int sub = threadIdx.x & 7;
  const int64_t stride = (int64_t)gridDim.x * 32;
  grid_dependency_trigger();
  grid_dependency_wait();
  for (int64_t r0 = (int64_t)blockIdx.x * 32; r0 < rows; r0 += stride) {  // warp-uniform trip count
    const int64_t r = r0 + (threadIdx.x >> 3);
    float s = 0.f;
    if (r < rows) {
      const int64_t bh = r / T;
      const int t = (int)(r - bh * T);
      const int b = (int)(bh / H), h = (int)(bh - (int64_t)b * H);
      const int64_t off = b * o_sb + h * o_sh + (int64_t)t * o_st + sub * 8;
      Vec16<__nv_bfloat16> vo, vd;
      vo.load(o + off);
      vd.load(d_o + off);
      float x[8], y[8];
      vo.get(x);
      vd.get(y);
#pragma unroll
      for (int i = 0; i < 8; i++) s += x[i] * y[i];
    }
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if (sub == 0 && r < rows) delta[r] = s;
  }
}

// Work items of the persistent kernels are sorted longest first; round k hands item
// k*G + c to CTA c in even rounds and item k*G + (G-1-c) in odd rounds, so every CTA gets
// nearly the same number of tiles.
__device__ __forceinline__ int snake_item(int k) {
  const int G = (int)gridDim.x, c = (int)blockIdx.x;
  return k * G + ((k & 1) ? G - 1 - c : c);
}

// ── backward math warps ─────────────────────────────────────────────────────────────────
// Sixteen math warps work on one 128 x 128 (query x key) tile: warp w owns the TMEM lane
// quadrant w % 4 (32 query rows, one per thread) and the key-column quarter (w - 2) / 4, so a
// thread handles 32 scores and an SM sub-partition has four math warps to switch between.  The work is split in two phases so that the tensor core can run
// ahead: phase A needs only S (scores -> P and the factor P * (1 - tanh^2)), phase B needs dP
// (-> dS) and stores the bf16 P / dS rows into the 128B-swizzled tiles.
//
// Soft cap: tanh(x) for |x| <= 0.35 comes from an odd polynomial on the FMA pipes
// (x + x^3 (p1 + p2 x^2 + p3 x^4), truncation error < 2e-6), which halves the load
// on the special-function unit that exp2 also needs; a warp whose tile holds a larger
// argument redoes the tile with the hardware tanh.
constexpr int AB_MATH_WARPS = 16;
constexpr int AB_THREADS = 64 + 32 * AB_MATH_WARPS;  // TMA warp, MMA warp, math warps
constexpr int AB_NC = 128 / (AB_MATH_WARPS / 4);     // score columns per math thread (32)
constexpr float TANH_POLY_LIMIT2 = 0.1225f;  // x^2 bound of the polynomial branch (|x| <= 0.35)

struct BwdRowConsts {
  float c1, c2, lse2, scale, delta;  // lse2 = +inf for a query row past the end (its P becomes 0)
  // polynomial tanh on the raw score s: tanh(c1*s) = s*(c1 + u*(a1 + u*(a2 + u*a3))), u = s^2,
  // a_k = p_k * c1^(2k+1); u_limit is the largest u it accepts (|c1*s| <= 0.35)
  float a1, a2, a3, u_limit;
};

// Phase A for AB_NC scores of one row.  pk: P as packed bf16 pairs; fk: -P * dcap as packed
// bf16 pairs (dcap = 1 - tanh^2, or 1 without a cap).  The scores are read 16 columns at a
// time to keep registers free for interleaving the per-pair dependency chains.
// Returns the largest squared score seen by the polynomial branch (0 otherwise).
template <bool DIAG, bool CAPPED, bool POLY>
__device__ __forceinline__ float bwd_phase_a(uint32_t t_s, int row, int col0, const BwdRowConsts &k,
                                             uint32_t (&pk)[AB_NC / 2], uint32_t (&fk)[AB_NC / 2]) {
  float big = 0.f;
  const uint64_t c1 = f2_pack(k.c1, k.c1), c2 = f2_pack(k.c2, k.c2), nl = f2_pack(-k.lse2, -k.lse2);
  const uint64_t m1 = f2_pack(-1.f, -1.f);
  const uint64_t a1 = f2_pack(k.a1, k.a1), a2 = f2_pack(k.a2, k.a2), a3 = f2_pack(k.a3, k.a3);
#pragma unroll
  for (int part = 0; part < AB_NC / 16; part++) {
    uint32_t r[16];
    tmem_ld_32x16(t_s + part * 16, r);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const uint64_t s = f2_pack(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
      uint64_t e, ndcap = m1;  // ndcap = tanh^2 - 1
      if (CAPPED) {
        uint64_t th;
        if (POLY) {
          const uint64_t u = f2_mul(s, s);
          float ua, ub;
          f2_unpack(u, ua, ub);
          big = fmax3(big, ua, ub);
          uint64_t t = f2_fma(u, a3, a2);
          t = f2_fma(t, u, a1);
          t = f2_fma(t, u, c1);
          th = f2_mul(s, t);
        } else {
          float xa, xb;
          f2_unpack(f2_mul(s, c1), xa, xb);
          th = f2_pack(tanh_approx(xa), tanh_approx(xb));
        }
        e = f2_fma(th, c2, nl);
        ndcap = f2_fma(th, th, m1);
      } else {
        e = f2_fma(s, c1, nl);
      }
      float ea, eb;
      f2_unpack(e, ea, eb);
      float pa = ex2_approx(ea), pb = ex2_approx(eb);
      if (DIAG) {
        const int c = col0 + part * 16 + i;
        if (c > row) pa = 0.f;
        if (c + 1 > row) pb = 0.f;
      }
      const uint32_t pp = bf16x2_pack(pa, pb);
      pk[part * 8 + (i >> 1)] = pp;
      if (CAPPED) {
        float fa, fb;
        f2_unpack(f2_mul(f2_pack(pa, pb), ndcap), fa, fb);
        fk[part * 8 + (i >> 1)] = bf16x2_pack(fa, fb);
      } else {
        fk[part * 8 + (i >> 1)] = pp ^ 0x80008000u;
      }
    }
  }
  return big;
}

// Phase B: dS = (-P dcap) * (-(dP - delta) * scale) for the same columns (the second factor is
// rounded to bf16 and the product taken in packed bf16), then the row's P (optional) and dS
// chunks go to shared memory.  p_row / ds_row point at this thread's 128-byte row in the
// 64-column tile that holds its columns; chunk0 is its first 16-byte chunk there (0 or 4).
template <bool WRITE_P>
__device__ __forceinline__ void bwd_phase_b(uint32_t t_dp, int row, int chunk0, const BwdRowConsts &k,
                                            const uint32_t (&pk)[AB_NC / 2], const uint32_t (&fk)[AB_NC / 2],
                                            uint8_t *p_row, uint8_t *ds_row) {
  const uint64_t nsc = f2_pack(-k.scale, -k.scale), ds0 = f2_pack(k.delta * k.scale, k.delta * k.scale);
#pragma unroll
  for (int part = 0; part < AB_NC / 16; part++) {
    uint32_t d[16];
    tmem_ld_32x16(t_dp + part * 16, d);
    tmem_ld_wait();
    uint32_t dd[8];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      float ga, gb;
      f2_unpack(f2_fma(f2_pack(__uint_as_float(d[i]), __uint_as_float(d[i + 1])), nsc, ds0), ga, gb);
      dd[i >> 1] = bf16x2_mul(fk[part * 8 + (i >> 1)], bf16x2_pack(ga, gb));
    }
#pragma unroll
    for (int q = 0; q < 2; q++) {
      const int off = ((chunk0 + part * 2 + q) ^ (row & 7)) * 16;
      if (WRITE_P)
        *reinterpret_cast<uint4 *>(p_row + off) =
            make_uint4(pk[part * 8 + 4 * q], pk[part * 8 + 4 * q + 1], pk[part * 8 + 4 * q + 2], pk[part * 8 + 4 * q + 3]);
      *reinterpret_cast<uint4 *>(ds_row + off) = make_uint4(dd[4 * q], dd[4 * q + 1], dd[4 * q + 2], dd[4 * q + 3]);
    }
  }
}

// Phase A with the branch selection: diagonal tile or not, capped or not, and for capped
// scores the polynomial tanh unless some argument in the warp's part of the tile is too large.
__device__ __forceinline__ void bwd_phase_a_any(uint32_t t_s, int row, int col0, bool diag, bool capped,
                                                const BwdRowConsts &k, uint32_t (&pk)[AB_NC / 2],
                                                uint32_t (&fk)[AB_NC / 2]) {
  if (!capped) {
    if (diag) bwd_phase_a<true, false, false>(t_s, row, col0, k, pk, fk);
    else bwd_phase_a<false, false, false>(t_s, row, col0, k, pk, fk);
    return;
  }
  const float big = diag ? bwd_phase_a<true, true, true>(t_s, row, col0, k, pk, fk)
                         : bwd_phase_a<false, true, true>(t_s, row, col0, k, pk, fk);
  if (__any_sync(0xffffffffu, !(big <= k.u_limit))) {  // also catches NaN
    if (diag) bwd_phase_a<true, true, false>(t_s, row, col0, k, pk, fk);
    else bwd_phase_a<false, true, false>(t_s, row, col0, k, pk, fk);
  }
}

// shared-memory map of the dK/dV kernel
constexpr int AK_STAGES = 3;                               // ring of (Q, dO) tiles
constexpr int AK_K = 0;                                    // 2 buffers (items alternate)
constexpr int AK_V = 2 * AT_TILE;
constexpr int AK_Q = 3 * AT_TILE;
constexpr int AK_DO = AK_Q + AK_STAGES * AT_TILE;
constexpr int AK_P = AK_DO + AK_STAGES * AT_TILE;          // 2 tiles (key halves)
constexpr int AK_DS = AK_P + 2 * AT_TILE;                  // 2 tiles
constexpr int AK_STG = AK_DS + 2 * AT_TILE;                // dQ staging: 4 epilogue warps x (32 rows x 128 bytes)
constexpr int AK_BAR = AK_STG + 4 * 4096;
constexpr int AK_DYN = AK_BAR + 256 + 1024;
constexpr int ABP_THREADS = AB_THREADS + 128;              // + four epilogue warps

// Pipeline of the backward kernel.  One CTA per SM walks (batch*head, key block) items, longest
// first; inside an item the tile index `it` walks the query blocks of the key block:
//   tensor core, on "tile it-1 stored" : dP(it) -> dQ(it-1), dV,dK += (P,dS)(it-1) -> S(it+1)
//   math warps                          : phase A(it) from S(it) | wait dP(it) and the end of
//                                         the products of tile it-1 | phase B(it) stores P,dS
//   epilogue warps (one per lane quadrant): every tile they move its dQ contribution TMEM ->
//                                         swizzled shared memory -> TMA store to the workspace;
//                                         when an item's last products are done they write
//                                         dV, dK while everybody else is on the next item
// S has two TMEM buffers, so the scores of the next tile are ready before the math warps ask
// for them; the dQ contribution of a tile is written over that tile's (long consumed) scores
// and the buffer takes new scores once the epilogue warps have read it out.  K has two
// buffers: the item's last dQ product still reads it when the next item begins, so the next K
// is fetched with the item's last (Q, dO) pair; V is free after the item's last dP.  All
// barrier phases are running counters over items (n) and tiles (t).
__global__ void __launch_bounds__(ABP_THREADS, 1)
attn_tc_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                       const __grid_constant__ CUtensorMap tmap_part, AttnBwdArgs a, int n_items, int BH) {
  extern __shared__ uint8_t at_smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)at_smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sb = smem_u32(smem);
  const uint32_t bar = sb + AK_BAR;
  const uint32_t v_full = bar, v_empty = bar + 8, s_full0 = bar + 16, dp_full = bar + 32, pds_ready = bar + 40,
                 acc_done = bar + 48, acc_final = bar + 56, acc_free = bar + 64, dq_full0 = bar + 72,
                 dq_free0 = bar + 88, k_full0 = bar + 104, k_empty0 = bar + 120, q_full0 = bar + 136,
                 q_empty0 = q_full0 + 8 * AK_STAGES;
  uint32_t *tmem_slot = (uint32_t *)(smem + AK_BAR + 136 + 16 * AK_STAGES);
  volatile uint32_t *abort_flag = (volatile uint32_t *)(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qb = (a.T + 127) / 128;
  constexpr uint32_t TMEM_COLS = 512;

  if (threadIdx.x == 0) {
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(k_full0, 1); mbar_init(k_full0 + 8, 1);
    mbar_init(k_empty0, 1); mbar_init(k_empty0 + 8, 1);
    mbar_init(s_full0, 1); mbar_init(s_full0 + 8, 1);
    mbar_init(dp_full, 1);
    mbar_init(pds_ready, AB_MATH_WARPS);
    mbar_init(acc_done, 1);
    mbar_init(acc_final, 1);
    mbar_init(acc_free, 4);
    mbar_init(dq_full0, 1); mbar_init(dq_full0 + 8, 1);
    mbar_init(dq_free0, 4); mbar_init(dq_free0 + 8, 4);
    for (int s = 0; s < AK_STAGES; s++) {
      mbar_init(q_full0 + 8 * s, 1);
      mbar_init(q_empty0 + 8 * s, 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  grid_dependency_trigger();
  grid_dependency_wait();  // set-up above is SM-local; global memory is touched from here on
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS0 = tmem_base, tdP = tmem_base + 256, tdV = tmem_base + 384, tdK = tmem_base + 448;
  const int n_pairs = n_qb * (n_qb + 1) / 2;

  // item -> (batch*head, key block): key block 0 has the most query blocks to visit
  auto decode = [&](int item, int &bh, int &kb) {
    kb = item / BH;
    bh = item - kb * BH;
  };

  if (warp == 0) {
    // TMA producer: the warp runs the loops, one elected lane issues
    int t = 0, n = 0;
    bool ok = true;
    for (int item = snake_item(0); item < n_items && ok; item = snake_item(++n)) {
      int bh, kb;
      decode(item, bh, kb);
      const int b = bh / a.H, h = bh - b * a.H, n_it = n_qb - kb;
      // K has two buffers (items alternate): the item's last dQ product still reads it while the
      // next item starts, so the next K is fetched ahead, with this item's last tile (below); the
      // very first K is fetched here.  V is free after the item's last dP and has one buffer.
      if (n == 0) {
        if (elect_one()) {
          mbar_expect_tx(k_full0, AT_TILE);
          tma_load_4d(sb + AK_K, &tmap_k, k_full0, 0, kb * 128, h, b);
        }
        __syncwarp();
      }
      if (!mbar_wait(v_empty, (n & 1) ^ 1, abort_flag)) break;
      if (elect_one()) {
        mbar_expect_tx(v_full, AT_TILE);
        tma_load_4d(sb + AK_V, &tmap_v, v_full, 0, kb * 128, h, b);
      }
      __syncwarp();
      for (int it = 0; it < n_it; it++, t++) {
        const int st = t % AK_STAGES;
        if (!mbar_wait(q_empty0 + 8 * st, ((t / AK_STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
        const int q0 = (kb + it) * 128;
        if (elect_one()) {
          mbar_expect_tx(q_full0 + 8 * st, 2 * AT_TILE);
          tma_load_4d(sb + AK_Q + st * AT_TILE, &tmap_q, q_full0 + 8 * st, 0, q0, h, b);
          tma_load_4d(sb + AK_DO + st * AT_TILE, &tmap_do, q_full0 + 8 * st, 0, q0, h, b);
        }
        __syncwarp();
        if (it == n_it - 1) {   // all of this item's tiles are on their way: now the next item's K
          const int nxt = snake_item(n + 1);
          if (nxt < n_items) {
            int bh2, kb2;
            decode(nxt, bh2, kb2);
            const int b2 = bh2 / a.H, h2 = bh2 - b2 * a.H, kbuf = (n + 1) & 1;
            // the buffer's previous tenant was item n - 1
            if (!mbar_wait(k_empty0 + 8 * kbuf, (((n + 1) >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
            if (elect_one()) {
              mbar_expect_tx(k_full0 + 8 * kbuf, AT_TILE);
              tma_load_4d(sb + AK_K + kbuf * AT_TILE, &tmap_k, k_full0 + 8 * kbuf, 0, kb2 * 128, h2, b2);
            }
            __syncwarp();
          }
        }
      }
    }
  } else if (warp == 1) {
    // MMA issuer: warp-uniform control flow and descriptors, one elected lane issues
    constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);   // [q x k] = A[q,d] B[k,d]^T
    constexpr uint32_t idesc_g = make_idesc_bf16(128, 64, true, true);      // [k x d] = A[q,k]^T B[q,d]
    const uint64_t d_k0 = make_smem_desc(sb + AK_K, 16, 1024), d_v = make_smem_desc(sb + AK_V, 16, 1024);
    const uint64_t d_q_k = make_smem_desc(sb + AK_Q, 16, 1024), d_do_k = make_smem_desc(sb + AK_DO, 16, 1024);
    const uint64_t d_q_n = make_smem_desc(sb + AK_Q, AT_TILE, 1024), d_do_n = make_smem_desc(sb + AK_DO, AT_TILE, 1024);
    const uint64_t d_p = make_smem_desc(sb + AK_P, AT_TILE, 1024), d_ds = make_smem_desc(sb + AK_DS, AT_TILE, 1024);
    // dQ(tile) = dS K, [q x d] = A[q,k] B[k,d]: dS read K-major, K read N-major
    constexpr uint32_t idesc_dq = make_idesc_bf16(128, 64, false, true);
    const uint64_t d_ds_k = make_smem_desc(sb + AK_DS, 16, 1024), d_k_n0 = make_smem_desc(sb + AK_K, AT_TILE, 1024);
    int t = 0, n = 0;
    bool ok = true;
    for (int item = snake_item(0); item < n_items && ok; item = snake_item(++n)) {
      int bh, kb;
      decode(item, bh, kb);
      const int n_it = n_qb - kb;
      const uint64_t d_k = d_k0 + (uint64_t)(((n & 1) * AT_TILE) >> 4), d_k_n = d_k_n0 + (uint64_t)(((n & 1) * AT_TILE) >> 4);
      auto issue_s = [&](int it) -> bool {   // S(it) = Q(it) K^T into buffer (t + it) & 1 (waits for the tile's loads)
        const int tt = t + it, st = tt % AK_STAGES;
        if (!mbar_wait(q_full0 + 8 * st, (tt / AK_STAGES) & 1, abort_flag)) return false;
        // the buffer last held the dQ contribution of tile tt - 2; it must have been read out
        if (tt >= 2 && !mbar_wait(dq_free0 + 8 * (tt & 1), ((tt - 2) >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint64_t qd = d_q_k + (uint64_t)((st * AT_TILE) >> 4);
        const uint32_t ts = tS0 + (tt & 1) * 128, done = s_full0 + 8 * (tt & 1);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; kk++) mma_bf16_ss(ts, qd + kk * 2, d_k + kk * 2, idesc_s, kk > 0 ? 1u : 0u);
          mma_commit(done);
        }
        __syncwarp();
        return true;
      };
      auto issue_dp = [&](int it) {          // dP(it) = dO(it) V^T (loads already awaited by issue_s(it))
        const uint64_t dd = d_do_k + (uint64_t)((((t + it) % AK_STAGES) * AT_TILE) >> 4);
        const bool last = it == n_it - 1;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; kk++) mma_bf16_ss(tdP, dd + kk * 2, d_v + kk * 2, idesc_s, kk > 0 ? 1u : 0u);
          mma_commit(dp_full);
          if (last) mma_commit(v_empty);       // V is not read after the item's last dP
        }
        __syncwarp();
      };
      ok = mbar_wait(k_full0 + 8 * (n & 1), (n >> 1) & 1, abort_flag) && mbar_wait(v_full, n & 1, abort_flag);
      if (ok) ok = issue_s(0);
      if (ok) issue_dp(0);
      if (ok && n_it > 1) ok = issue_s(1);
      for (int it = 0; it < n_it && ok; it++) {
        const int tt = t + it;
        if (!mbar_wait(pds_ready, tt & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (it + 1 < n_it) issue_dp(it + 1);
        // the epilogue warps must have read the previous item's dV / dK before they are overwritten
        if (it == 0 && n > 0 && !mbar_wait(acc_free, (n - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const int st = tt % AK_STAGES;
        const uint64_t qn = d_q_n + (uint64_t)((st * AT_TILE) >> 4), don = d_do_n + (uint64_t)((st * AT_TILE) >> 4);
        const uint32_t first = it > 0 ? 1u : 0u, freed = q_empty0 + 8 * st;
        const bool last = it == n_it - 1;
        if (elect_one()) {
          {
            // this tile's dQ contribution goes where its scores were: phase A has long consumed them
            const uint32_t tdq = tS0 + (tt & 1) * 128;
#pragma unroll
            for (int kk = 0; kk < 8; kk++)  // 16 keys per step; dS tile (kk >> 2), 32 bytes per step inside it
              mma_bf16_ss(tdq, d_ds_k + (uint64_t)(((kk >> 2) * AT_TILE + (kk & 3) * 32) >> 4), d_k_n + kk * 128,
                          idesc_dq, kk > 0 ? 1u : 0u);
            mma_commit(dq_full0 + 8 * (tt & 1));
          }
#pragma unroll
          for (int kk = 0; kk < 8; kk++)  // 16 query rows per step
            mma_bf16_ss(tdV, d_p + kk * 128, don + kk * 128, idesc_g, kk > 0 ? 1u : first);
#pragma unroll
          for (int kk = 0; kk < 8; kk++) mma_bf16_ss(tdK, d_ds + kk * 128, qn + kk * 128, idesc_g, kk > 0 ? 1u : first);
          mma_commit(freed);
          mma_commit(acc_done);
          if (last) {
            mma_commit(acc_final);
            mma_commit(k_empty0 + 8 * (n & 1));  // the last dQ product was the last reader of K
          }
        }
        __syncwarp();
        if (it + 2 < n_it) ok = issue_s(it + 2);
      }
      t += n_it;
    }
  } else if (warp < 2 + AB_MATH_WARPS) {
    const int quad = warp & 3, colq = (warp - 2) >> 2;  // lane quadrant, 32-column quarter
    const int col0 = colq * AB_NC;
    const int row = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    const bool capped = a.cap > 0.f;
    BwdRowConsts k;
    k.c1 = capped ? a.scale / a.cap : a.scale * LOG2E;
    k.c2 = a.cap * LOG2E;
    k.scale = a.scale;
    {
      const float q = k.c1 * k.c1;
      k.a1 = k.c1 * q * -0.3333333333f;
      k.a2 = k.c1 * q * q * 0.1333333333f;
      k.a3 = k.c1 * q * q * q * -0.0539682540f;
      k.u_limit = TANH_POLY_LIMIT2 / q;
    }
    uint8_t *p_row = smem + AK_P + (colq >> 1) * AT_TILE + row * 128;
    uint8_t *ds_row = smem + AK_DS + (colq >> 1) * AT_TILE + row * 128;
    int t = 0;
    bool ok = true;
    for (int rnd = 0, item = snake_item(0); item < n_items && ok; item = snake_item(++rnd)) {
      int bh, kb;
      decode(item, bh, kb);
      const int n_it = n_qb - kb;
      // the row's LSE and delta for the next tile are fetched one tile ahead, so that their
      // global-memory latency is not paid at the start of every tile
      auto fetch_row = [&](int it, float &lse_raw, float &dl) {
        const int qi = (kb + it) * 128 + row;
        const bool valid = qi < a.T;
        lse_raw = valid ? a.lse[(int64_t)bh * a.T + qi] : INFINITY;
        dl = valid ? a.delta[(int64_t)bh * a.T + qi] : 0.f;
      };
      float lse_nxt, dl_nxt;
      fetch_row(0, lse_nxt, dl_nxt);
      for (int it = 0; it < n_it; it++) {
        const int tt = t + it;
        k.lse2 = lse_nxt * LOG2E;
        k.delta = dl_nxt;
        if (it + 1 < n_it) fetch_row(it + 1, lse_nxt, dl_nxt);
        uint32_t pk[AB_NC / 2], fk[AB_NC / 2];
        if (!mbar_wait(s_full0 + 8 * (tt & 1), (tt >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        bwd_phase_a_any(tS0 + (tt & 1) * 128 + lane_off + col0, row, col0, it == 0, capped, k, pk, fk);
        if (!mbar_wait(dp_full, tt & 1, abort_flag)) { ok = false; break; }
        // the gradient products of the previous tile must have finished reading the P / dS tiles
        if (tt > 0 && !mbar_wait(acc_done, (tt - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        bwd_phase_b<true>(tdP + lane_off + col0, row, (colq & 1) * 4, k, pk, fk, p_row, ds_row);
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(pds_ready);
      }
      t += n_it;
    }
  } else {
    // epilogue warps: quadrant q writes rows 32q .. 32q+31 of dV and dK of every finished item
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    int n = 0, t = 0;
    bool ok = true;
    uint8_t *stg = smem + AK_STG + quad * 4096;
    const uint32_t stg_u32 = sb + AK_STG + quad * 4096;
    if (lane == 0) tma_prefetch_desc(&tmap_part);
    for (int item = snake_item(0); item < n_items && ok; item = snake_item(++n)) {
      int bh, kb;
      decode(item, bh, kb);
      const int b = bh / a.H, h = bh - b * a.H;
      {
        // every tile: this quadrant's 32 query rows of the tile's dQ contribution, fp32, to the
        // workspace slab of (query block, key block); the TMEM columns go back to the scores at once
        const int n_it = n_qb - kb;
        for (int it = 0; it < n_it; it++) {
          const int tt = t + it, qb = kb + it;
          if (!mbar_wait(dq_full0 + 8 * (tt & 1), (tt >> 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t tdq = tS0 + (tt & 1) * 128 + lane_off;
          // workspace row of this warp's first query row: slab (bh, pair(qb, kb)), 128 rows each
          const int part_row0 = (bh * n_pairs + (qb * (qb + 1) / 2 + kb)) * 128 + quad * 32;
#pragma unroll 1
          for (int c = 0; c < 2; c++) {         // columns 0-31, 32-63: one 128B-swizzled box of 32 rows each
            uint32_t r[32];
            tmem_ld_32x32(tdq + c * 32, r);
            tmem_ld_wait();
            if (c == 1) {   // both halves have been read: the columns may take new scores
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(dq_free0 + 8 * (tt & 1));
            }
            if (lane == 0) bulk_wait_read<0>();   // the previous box has left the staging buffer
            __syncwarp();
            uint8_t *bp = stg + lane * 128;
#pragma unroll
            for (int q = 0; q < 8; q++)
              *reinterpret_cast<uint4 *>(bp + ((q ^ (lane & 7)) << 4)) = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmap_part, stg_u32, c * 32, part_row0);
              bulk_commit();
            }
          }
        }
        t += n_it;
        if (!ok) break;
      }
      if (!mbar_wait(acc_final, n & 1, abort_flag)) break;
      tc_fence_after();
      const int kj = kb * 128 + row;  // accumulator lanes are keys
      const int64_t off = (int64_t)b * a.q_sb + (int64_t)h * a.q_sh + (int64_t)kj * a.q_st;
#pragma unroll 1
      for (int c = 0; c < 4; c++) {   // dV[0:32], dV[32:64], dK[0:32], dK[32:64]
        uint32_t r[32];
        tmem_ld_32x32((c < 2 ? tdV : tdK) + lane_off + (c & 1) * 32, r);
        tmem_ld_wait();
        if (kj < a.T) {
          __nv_bfloat16 *dst = (__nv_bfloat16 *)(c < 2 ? a.dv : a.dk) + off + (c & 1) * 32;
#pragma unroll
          for (int q = 0; q < 4; q++) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = __uint_as_float(r[q * 8 + i]);
            Vec16<__nv_bfloat16> v;
            v.set(f);
            v.store(dst + q * 8);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_free);
    }
    if (lane == 0) bulk_wait<0>();   // this warp's last dQ boxes have landed
  }

  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
    if (threadIdx.x == 0 && a.err) atomicExch(a.err, 0xA8000000u | (uint32_t)(blockIdx.x & 0xFFFF));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// dQ[bh, query block qb] = sum over key blocks kb <= qb of the fp32 contributions the
// backward kernel left in the workspace, added in key-block order (the same order on every
// run), rounded to bf16 once.  Sixteen threads per query row (four floats each); the loads of
// four key blocks are in flight together.  HBM-bound: reads (qb + 1) * 32 KB, writes 16 KB per
// (bh, qb).
__global__ void __launch_bounds__(256) attn_tc_dq_reduce_kernel(const float *__restrict__ part, __nv_bfloat16 *dq,
                                                                int64_t q_sb, int64_t q_sh, int64_t q_st, int H, int T,
                                                                int n_qb) {
  const int n_pairs = n_qb * (n_qb + 1) / 2;
  const int bh = blockIdx.y, qb = n_qb - 1 - (int)(blockIdx.x >> 3);   // long sums first
  const int row = (int)(blockIdx.x & 7) * 16 + (int)(threadIdx.x >> 4), c4 = (int)(threadIdx.x & 15);
  const int qi = qb * 128 + row;
  grid_dependency_trigger();
  grid_dependency_wait();
  if (qi >= T) return;
  const float4 *src = reinterpret_cast<const float4 *>(part + (((int64_t)bh * n_pairs + qb * (qb + 1) / 2) * 128 + row) * 64) + c4;
  constexpr int64_t SLAB4 = 128 * 64 / 4;   // float4 per (qb, kb) slab
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  int kb = 0;
  for (; kb + 4 <= qb + 1; kb += 4) {
    const float4 v0 = __ldcs(src + (kb + 0) * SLAB4), v1 = __ldcs(src + (kb + 1) * SLAB4),
                 v2 = __ldcs(src + (kb + 2) * SLAB4), v3 = __ldcs(src + (kb + 3) * SLAB4);
    acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
    acc.x += v1.x; acc.y += v1.y; acc.z += v1.z; acc.w += v1.w;
    acc.x += v2.x; acc.y += v2.y; acc.z += v2.z; acc.w += v2.w;
    acc.x += v3.x; acc.y += v3.y; acc.z += v3.z; acc.w += v3.w;
  }
  for (; kb <= qb; kb++) {
    const float4 v = __ldcs(src + kb * SLAB4);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  const int b = bh / H, h = bh - b * H;
  __nv_bfloat16 *dst = dq + (int64_t)b * q_sb + (int64_t)h * q_sh + (int64_t)qi * q_st + c4 * 4;
  uint2 o;
  *reinterpret_cast<__nv_bfloat162 *>(&o.x) = __floats2bfloat162_rn(acc.x, acc.y);
  *reinterpret_cast<__nv_bfloat162 *>(&o.y) = __floats2bfloat162_rn(acc.z, acc.w);
  *reinterpret_cast<uint2 *>(dst) = o;
}

// ── forward, bounded scores (soft cap), persistent ─────────────────────────────────────
// With a soft cap the transformed score cap*tanh(s/cap) lies in [-cap, cap], so the softmax
// can use the constant cap as its reference maximum: exp2(c2*(tanh - 1)) never overflows and,
// for cap*log2(e) <= 50, never underflows either.  That removes the running maximum, the
// rescaling of O and every dependency between key blocks, and lets the tile be split over
// sixteen math warps (32 query rows x 32 key columns each, row sums combined once per query
// block).  tanh comes from the polynomial of the backward kernels, exp2 from the
// special-function unit.
//
// One CTA per SM walks (batch*head, query block) items, longest first, round-robin:
//   warp 0      TMA producer: Q (2 buffers), K tiles through a 3-stage ring (a K tile is free as
//               soon as its score product is done) and V tiles through a 4-stage ring; it
//               runs ahead into the next item while the current one is being computed
//   warp 1      MMA issuer: the score product of the tile two ahead in the CTA's tile stream
//               (across item boundaries) is issued as soon as the math warps have consumed
//               S of the current tile (two S buffers in TMEM), O += P(j) V(j) when P(j) is in
//               shared memory (two P buffers), so the tensor core works while the math warps
//               compute
//   warps 2-17  math warps
//   warps 18-21 epilogue warps (one per lane quadrant): combine the row sums, scale O, write
//               O and LSE while the other warps are already on the next item
// All barrier phases are running counters over items and tiles; every wait is bounded.
constexpr int AF2_THREADS = 64 + 32 * 16 + 128;
constexpr int AF2_KST = 3, AF2_VST = 4;
constexpr int AF2_Q = 0;                                   // 2 buffers
constexpr int AF2_K = 2 * AT_TILE;
constexpr int AF2_V = AF2_K + AF2_KST * AT_TILE;
constexpr int AF2_P = AF2_V + AF2_VST * AT_TILE;           // 2 buffers x 2 tiles (key halves)
constexpr int AF2_BAR = AF2_P + 4 * AT_TILE;
constexpr int AF2_LSUM = AF2_BAR + 256;                    // [4 items][4 column quarters][128 rows] floats
constexpr int AF2_DYN = AF2_LSUM + 8192 + 1024;
constexpr float AF2_MAX_C2 = 50.f;                         // largest cap*log2(e) this kernel accepts

// Constants of the bounded-score softmax with the polynomial tanh, folded so that the exponent
// comes straight from the raw score s:  c2*tanh(c1*s) - c2 = s*(b0 + u*(b1 + u*(b2 + u*b3))) - c2
// with u = s^2 and b_k = c2 * p_k * c1^(2k+1)  (p = 1, -1/3, 2/15, -17/315).
struct Fwd2Consts {
  float c1, c2;      // scale / cap, cap * log2(e)
  float b0, b1, b2, b3;
  float u_limit;     // largest s^2 the polynomial branch accepts (|c1*s| <= 0.35)
};
__device__ __forceinline__ Fwd2Consts fwd2_consts(float scale, float cap) {
  Fwd2Consts k;
  k.c1 = scale / cap;
  k.c2 = cap * 1.4426950408889634f;
  const float q = k.c1 * k.c1;
  k.b0 = k.c2 * k.c1;
  k.b1 = k.b0 * q * -0.3333333333f;
  k.b2 = k.b0 * q * q * 0.1333333333f;
  k.b3 = k.b0 * q * q * q * -0.0539682540f;
  k.u_limit = TANH_POLY_LIMIT2 / q;
  return k;
}

// P for 32 scores of one row (bounded-score softmax).  Returns the largest squared score seen
// (polynomial branch only); adds the row's probabilities to lsum.
template <bool DIAG, bool POLY>
__device__ __forceinline__ float fwd2_scores(uint32_t t_s, int row, int col0, const Fwd2Consts &k, uint64_t &lsum,
                                             uint32_t (&pk)[16]) {
  float big = 0.f;
  const uint64_t c1 = f2_pack(k.c1, k.c1), c2 = f2_pack(k.c2, k.c2), nm = f2_pack(-k.c2, -k.c2);
  const uint64_t b0 = f2_pack(k.b0, k.b0), b1 = f2_pack(k.b1, k.b1), b2 = f2_pack(k.b2, k.b2), b3 = f2_pack(k.b3, k.b3);
#pragma unroll
  for (int part = 0; part < 2; part++) {
    uint32_t r[16];
    tmem_ld_32x16(t_s + part * 16, r);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const uint64_t s = f2_pack(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
      uint64_t e;
      if (POLY) {
        const uint64_t u = f2_mul(s, s);
        float ua, ub;
        f2_unpack(u, ua, ub);
        big = fmax3(big, ua, ub);
        uint64_t t = f2_fma(u, b3, b2);
        t = f2_fma(t, u, b1);
        t = f2_fma(t, u, b0);
        e = f2_fma(s, t, nm);
      } else {
        float xa, xb;
        f2_unpack(f2_mul(s, c1), xa, xb);
        e = f2_fma(f2_pack(tanh_approx(xa), tanh_approx(xb)), c2, nm);
      }
      float ea, eb;
      f2_unpack(e, ea, eb);
      float pa = ex2_approx(ea), pb = ex2_approx(eb);
      if (DIAG) {
        const int c = col0 + part * 16 + i;
        if (c > row) pa = 0.f;
        if (c + 1 > row) pb = 0.f;
      }
      lsum = f2_add(lsum, f2_pack(pa, pb));
      pk[part * 8 + (i >> 1)] = bf16x2_pack(pa, pb);
    }
  }
  return big;
}

__global__ void __launch_bounds__(AF2_THREADS, 1)
attn_tc_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, AttnTcArgs a, int n_items, int BH) {
  extern __shared__ uint8_t at_smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)at_smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sb = smem_u32(smem);
  const uint32_t bar = sb + AF2_BAR;
  const uint32_t q_full0 = bar, q_empty0 = bar + 16, s_full0 = bar + 32, p_ready0 = bar + 48, p_free0 = bar + 64,
                 o_done = bar + 80, o_free = bar + 88, l_ready0 = bar + 96, k_full0 = bar + 128,
                 k_empty0 = k_full0 + 8 * AF2_KST, v_full0 = k_empty0 + 8 * AF2_KST, v_empty0 = v_full0 + 8 * AF2_VST;
  uint32_t *tmem_slot = (uint32_t *)(smem + AF2_BAR + 128 + 16 * (AF2_KST + AF2_VST));
  volatile uint32_t *abort_flag = (volatile uint32_t *)(tmem_slot + 1);
  float *lsm = reinterpret_cast<float *>(smem + AF2_LSUM);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qb = (a.T + 127) / 128;
  constexpr uint32_t TMEM_COLS = 512;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; i++) {
      mbar_init(q_full0 + 8 * i, 1);
      mbar_init(q_empty0 + 8 * i, 1);
      mbar_init(s_full0 + 8 * i, 1);
      mbar_init(p_ready0 + 8 * i, 16);
      mbar_init(p_free0 + 8 * i, 1);
    }
    mbar_init(o_done, 1);
    // The math warps can finish two more items while the epilogue warps are still on item n
    // (two S and two P buffers let them run two tiles past the tensor core, and a short item is
    // one tile), so the row sums and their barrier are kept per item in a ring of four.
    for (int i = 0; i < 4; i++) mbar_init(l_ready0 + 8 * i, 16);
    mbar_init(o_free, 4);
    for (int s = 0; s < AF2_KST; s++) {
      mbar_init(k_full0 + 8 * s, 1);
      mbar_init(k_empty0 + 8 * s, 1);
    }
    for (int s = 0; s < AF2_VST; s++) {
      mbar_init(v_full0 + 8 * s, 1);
      mbar_init(v_empty0 + 8 * s, 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  grid_dependency_trigger();
  grid_dependency_wait();  // set-up above is SM-local; global memory is touched from here on
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS0 = tmem_base, tO = tmem_base + 256;

  // item -> (batch*head, query block): the longest query blocks come first
  auto decode = [&](int item, int &bh, int &qb) {
    qb = n_qb - 1 - item / BH;
    bh = item - (item / BH) * BH;
  };

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
    }
    int t = 0, n = 0;
    bool ok = true;
    for (int item = snake_item(0); item < n_items && ok; item = snake_item(++n)) {
      int bh, qb;
      decode(item, bh, qb);
      const int b = bh / a.H, h = bh - b * a.H, nb = qb + 1;
      if (!mbar_wait(q_empty0 + 8 * (n & 1), ((n >> 1) & 1) ^ 1, abort_flag)) break;
      if (elect_one()) {
        mbar_expect_tx(q_full0 + 8 * (n & 1), AT_TILE);
        tma_load_4d(sb + AF2_Q + (n & 1) * AT_TILE, &tmap_q, q_full0 + 8 * (n & 1), 0, qb * 128, h, b);
      }
      __syncwarp();
      for (int j = 0; j < nb; j++, t++) {
        const int ks = t % AF2_KST, vs = t % AF2_VST;
        if (!mbar_wait(k_empty0 + 8 * ks, ((t / AF2_KST) & 1) ^ 1, abort_flag)) { ok = false; break; }
        if (elect_one()) {
          mbar_expect_tx(k_full0 + 8 * ks, AT_TILE);
          tma_load_4d(sb + AF2_K + ks * AT_TILE, &tmap_k, k_full0 + 8 * ks, 0, j * 128, h, b);
        }
        __syncwarp();
        if (!mbar_wait(v_empty0 + 8 * vs, ((t / AF2_VST) & 1) ^ 1, abort_flag)) { ok = false; break; }
        if (elect_one()) {
          mbar_expect_tx(v_full0 + 8 * vs, AT_TILE);
          tma_load_4d(sb + AF2_V + vs * AT_TILE, &tmap_v, v_full0 + 8 * vs, 0, j * 128, h, b);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false);
    constexpr uint32_t idesc_pv = make_idesc_bf16(128, 64, false, true);
    const uint64_t d_q = make_smem_desc(sb + AF2_Q, 16, 1024), d_k = make_smem_desc(sb + AF2_K, 16, 1024);
    const uint64_t d_p = make_smem_desc(sb + AF2_P, 16, 1024), d_v = make_smem_desc(sb + AF2_V, AT_TILE, 1024);
    // The score products run two tiles ahead of the P V products over the CTA's whole tile
    // stream, across item boundaries: `la_*` is the cursor of the next S to issue.
    int la_item = snake_item(0), la_j = 0, la_n = 0, la_t = 0, la_nb = 0;
    if (la_item < n_items) {
      int bh, qb;
      decode(la_item, bh, qb);
      la_nb = qb + 1;
    }
    auto issue_next_s = [&]() -> bool {   // S of the cursor's tile into buffer la_t & 1, then advance the cursor
      if (la_item >= n_items) return true;
      if (la_j == 0 && !mbar_wait(q_full0 + 8 * (la_n & 1), (la_n >> 1) & 1, abort_flag)) return false;
      const int st = la_t % AF2_KST;
      if (!mbar_wait(k_full0 + 8 * st, (la_t / AF2_KST) & 1, abort_flag)) return false;
      tc_fence_after();
      const uint64_t qd = d_q + (uint64_t)(((la_n & 1) * AT_TILE) >> 4), kd = d_k + (uint64_t)((st * AT_TILE) >> 4);
      const uint32_t ts = tS0 + (la_t & 1) * 128, done = s_full0 + 8 * (la_t & 1), k_freed = k_empty0 + 8 * st,
                     q_freed = q_empty0 + 8 * (la_n & 1);
      const bool last = la_j == la_nb - 1;
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < 4; kk++) mma_bf16_ss(ts, qd + kk * 2, kd + kk * 2, idesc_qk, kk > 0 ? 1u : 0u);
        mma_commit(k_freed);
        mma_commit(done);
        if (last) mma_commit(q_freed);  // Q is not needed after the item's last score product
      }
      __syncwarp();
      la_t++;
      if (++la_j == la_nb) {
        la_n++;
        la_item = snake_item(la_n);
        la_j = 0;
        if (la_item < n_items) {
          int bh, qb;
          decode(la_item, bh, qb);
          la_nb = qb + 1;
        }
      }
      return true;
    };
    bool ok = issue_next_s();
    if (ok) ok = issue_next_s();
    int t = 0, n = 0;
    for (int item = snake_item(0); item < n_items && ok; item = snake_item(++n)) {
      int bh, qb;
      decode(item, bh, qb);
      const int nb = qb + 1;
      for (int j = 0; j < nb && ok; j++) {
        const int tt = t + j, st = tt % AF2_VST;
        if (!mbar_wait(p_ready0 + 8 * (tt & 1), (tt >> 1) & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait(v_full0 + 8 * st, (tt / AF2_VST) & 1, abort_flag)) { ok = false; break; }
        // the epilogue warps must have read the previous item's O before it is overwritten
        if (j == 0 && n > 0 && !mbar_wait(o_free, (n - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint64_t pd = d_p + (uint64_t)(((tt & 1) * 2 * AT_TILE) >> 4);
        const uint64_t vd = d_v + (uint64_t)((st * AT_TILE) >> 4);
        const uint32_t first = j > 0 ? 1u : 0u, kv_freed = v_empty0 + 8 * st, p_freed = p_free0 + 8 * (tt & 1);
        const bool last = j == nb - 1;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; kk++)
            mma_bf16_ss(tO, pd + (uint64_t)(((kk >> 2) * AT_TILE + (kk & 3) * 32) >> 4), vd + kk * 128, idesc_pv,
                        kk > 0 ? 1u : first);
          mma_commit(kv_freed);
          mma_commit(p_freed);
          if (last) mma_commit(o_done);
        }
        __syncwarp();
        ok = issue_next_s();   // the S buffer of this tile is free: the math warps have consumed it
      }
      t += nb;
    }
  } else if (warp < 18) {
    const int quad = warp & 3, colq = (warp - 2) >> 2;
    const int col0 = colq * 32;
    const int row = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const Fwd2Consts kc = fwd2_consts(a.scale, a.cap);
    int t = 0, n = 0;
    bool ok = true;
    for (int item = snake_item(0); item < n_items && ok; item = snake_item(++n)) {
      int bh, qb;
      decode(item, bh, qb);
      const int nb = qb + 1;
      uint64_t lsum = 0;  // two fp32 zeros
      for (int j = 0; j < nb; j++) {
        const int tt = t + j, buf = tt & 1;
        if (!mbar_wait(s_full0 + 8 * buf, (tt >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t t_s = tS0 + buf * 128 + lane_off + col0;
        uint32_t pk[16];
        const bool diag = j == qb;
        const uint64_t l_before = lsum;
        const float big = diag ? fwd2_scores<true, true>(t_s, row, col0, kc, lsum, pk)
                               : fwd2_scores<false, true>(t_s, row, col0, kc, lsum, pk);
        if (__any_sync(0xffffffffu, !(big <= kc.u_limit))) {  // out of the polynomial's range (or NaN)
          lsum = l_before;
          if (diag) fwd2_scores<true, false>(t_s, row, col0, kc, lsum, pk);
          else fwd2_scores<false, false>(t_s, row, col0, kc, lsum, pk);
        }
        // the P buffer is free once O += P V of two tiles ago has read it
        if (tt >= 2 && !mbar_wait(p_free0 + 8 * buf, ((tt >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
        uint8_t *p_row = smem + AF2_P + buf * 2 * AT_TILE + (colq >> 1) * AT_TILE + row * 128;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const int off = (((colq & 1) * 4 + q) ^ (row & 7)) * 16;
          *reinterpret_cast<uint4 *>(p_row + off) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        }
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready0 + 8 * buf);
      }
      if (!ok) break;
      t += nb;
      // the row sums of the four column quarters go to the epilogue warps
      float la, lb;
      f2_unpack(lsum, la, lb);
      lsm[(n & 3) * 512 + colq * 128 + row] = la + lb;
      __syncwarp();
      if (lane == 0) mbar_arrive(l_ready0 + 8 * (n & 3));
    }
  } else {
    // epilogue warps: quadrant q finishes rows 32q .. 32q+31 of every item
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const float c2 = a.cap * 1.4426950408889634f;
    int n = 0;
    for (int item = snake_item(0); item < n_items; item = snake_item(++n)) {
      int bh, qb;
      decode(item, bh, qb);
      const int b = bh / a.H, h = bh - b * a.H;
      if (!mbar_wait(l_ready0 + 8 * (n & 3), (n >> 2) & 1, abort_flag)) break;
      const float *lp = lsm + (n & 3) * 512 + row;
      const float l = (lp[0] + lp[128]) + (lp[256] + lp[384]);
      if (!mbar_wait(o_done, n & 1, abort_flag)) break;
      tc_fence_after();
      const int qi = qb * 128 + row;
      const float inv = 1.f / l;
      __nv_bfloat16 *orow = (__nv_bfloat16 *)a.o + (int64_t)b * a.o_sb + (int64_t)h * a.o_sh + (int64_t)qi * a.o_st;
#pragma unroll 1
      for (int c = 0; c < 2; c++) {
        uint32_t r[32];
        tmem_ld_32x32(tO + lane_off + c * 32, r);
        tmem_ld_wait();
        if (qi < a.T) {
#pragma unroll
          for (int q = 0; q < 4; q++) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = __uint_as_float(r[q * 8 + i]) * inv;
            Vec16<__nv_bfloat16> v;
            v.set(f);
            v.store(orow + c * 32 + q * 8);
          }
        }
      }
      if (qi < a.T) a.lse[(int64_t)bh * a.T + qi] = (c2 + log2f(l)) * 0.6931471805599453f;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free);
    }
  }

  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
    if (threadIdx.x == 0 && a.err) atomicExch(a.err, 0xAA000000u | (uint32_t)(blockIdx.x & 0xFFFF));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ── host ────────────────────────────────────────────────────────────────────
struct Tmap4Key {
  uint64_t base, T, H, B, st, sh, sb;
  uint32_t rows;
  bool operator==(const Tmap4Key &o) const {
    return base == o.base && T == o.T && H == o.H && B == o.B && st == o.st && sh == o.sh && sb == o.sb && rows == o.rows;
  }
};
struct Tmap4Hash {
  size_t operator()(const Tmap4Key &k) const {
    uint64_t h = k.base * 0x9e3779b97f4a7c15ull ^ (k.T << 7) ^ (k.H << 23) ^ (k.B << 37) ^ (k.st * 31) ^ (k.sh * 131) ^
                 (k.sb * 0xff51afd7ed558ccdull) ^ k.rows;
    return (size_t)(h ^ (h >> 31));
  }
};
static std::unordered_map<Tmap4Key, CUtensorMap, Tmap4Hash> g_tmaps4;
static std::mutex g_tmap4_mu;

static int get_tmap4(CUtensorMap *out, const void *base, const alpha_attn_params_t *p, int64_t st, int64_t sh, int64_t sb,
                     uint32_t rows) {
  Tmap4Key key{(uint64_t)(uintptr_t)base, (uint64_t)p->T, (uint64_t)p->heads, (uint64_t)p->batch, (uint64_t)st,
               (uint64_t)sh, (uint64_t)sb, rows};
  std::lock_guard<std::mutex> lk(g_tmap4_mu);
  auto it = g_tmaps4.find(key);
  if (it != g_tmaps4.end()) {
    *out = it->second;
    return 0;
  }
  if (encode_tmap_4d_bf16(out, base, 64, p->T, p->heads, p->batch, st, sh, sb, rows)) return 1;
  if (g_tmaps4.size() > 4096) g_tmaps4.clear();
  g_tmaps4[key] = *out;
  return 0;
}

// The tensor-core path needs bf16 storage, head dim 64 and strides that TMA can describe.
bool attn_tc_supported(const alpha_attn_params_t *p, alpha_buf q, alpha_buf k, alpha_buf v) {
  if (p->dtype != ALPHA_BF16 || p->D != 64) return false;
  if ((q | k | v) & 15) return false;
  if (p->q_st % 8 || (p->heads > 1 && p->q_sh % 8) || (p->batch > 1 && p->q_sb % 8)) return false;
  if (p->o_st % 8 || p->o_sh % 8 || p->o_sb % 8) return false;
  if (p->batch * p->heads > 65535) return false;
  return true;
}

int attn_tc_fwd(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf o, alpha_buf lse, const alpha_attn_params_t *p) {
  if (p->batch * p->heads * p->T == 0) return 0;
  ProfScope prof(PROF_ATTN_FWD, 4.0 * p->batch * p->heads * (double)p->T * p->T * p->D);
  CUtensorMap tq, tk, tv;
  if (get_tmap4(&tq, ptr<void>(q), p, p->q_st, p->q_sh, p->q_sb, 128)) return 1;
  if (get_tmap4(&tk, ptr<void>(k), p, p->q_st, p->q_sh, p->q_sb, 128)) return 1;
  if (get_tmap4(&tv, ptr<void>(v), p, p->q_st, p->q_sh, p->q_sb, 128)) return 1;
  AttnTcArgs a;
  memset(&a, 0, sizeof(a));
  a.o = ptr<void>(o);
  a.lse = ptr<float>(lse);
  a.o_sb = p->o_sb; a.o_sh = p->o_sh; a.o_st = p->o_st;
  a.H = (int)p->heads; a.T = (int)p->T;
  a.scale = p->scale; a.cap = p->soft_cap;
  a.err = tc_error_word();
  static int attr = -1;
  if (attr != g_init_epoch) {
    ALPHA_CUDA(cudaFuncSetAttribute(attn_tc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AF_DYN));
    ALPHA_CUDA(cudaFuncSetAttribute(attn_tc_fwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AF2_DYN));
    attr = g_init_epoch;
  }
  if (p->soft_cap > 0.f && p->soft_cap * 1.4426950408889634f <= AF2_MAX_C2) {
    // bounded scores: the persistent kernel without a running maximum
    const int BH = (int)(p->batch * p->heads);
    const int n_items = (int)((p->T + 127) / 128) * BH;
    const int grid2 = n_items < g_sm_count ? n_items : g_sm_count;
    ALPHA_CUDA(launch_overlapped(OVL_ATTN_FWD, attn_tc_fwd2_kernel, dim3(grid2), dim3(AF2_THREADS), AF2_DYN, tq, tk, tv, a, n_items, BH));
    ALPHA_LAUNCHED();
    return 0;
  }
  dim3 grid((unsigned)((p->T + 127) / 128), (unsigned)(p->batch * p->heads));
  ALPHA_CUDA(launch_overlapped(OVL_ATTN_FWD, attn_tc_fwd_kernel, grid, dim3(AT_THREADS), AF_DYN, tq, tk, tv, a));
  ALPHA_LAUNCHED();
  return 0;
}

// `delta_in` != 0: the row-dots dO.O, [batch, heads, T] f32, already computed by the caller
// (alpha_gemm_nn_rowdot); `o` is then not read.
int attn_tc_bwd(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf o, alpha_buf d_o, alpha_buf lse, alpha_buf dq,
                alpha_buf dk, alpha_buf dv, const alpha_attn_params_t *p, alpha_buf delta_in) {
  if (p->batch * p->heads * p->T == 0) return 0;
  ProfScope prof(PROF_ATTN_BWD, 8.0 * p->batch * p->heads * (double)p->T * p->T * p->D);
  CUtensorMap tq, tk, tv, tdo;
  if (get_tmap4(&tq, ptr<void>(q), p, p->q_st, p->q_sh, p->q_sb, 128)) return 1;
  if (get_tmap4(&tk, ptr<void>(k), p, p->q_st, p->q_sh, p->q_sb, 128)) return 1;
  if (get_tmap4(&tv, ptr<void>(v), p, p->q_st, p->q_sh, p->q_sb, 128)) return 1;
  if (get_tmap4(&tdo, ptr<void>(d_o), p, p->o_st, p->o_sh, p->o_sb, 128)) return 1;
  const int64_t rows = p->batch * p->heads * p->T;
  void *delta = nullptr;
  if (delta_in) {
    delta = ptr<void>(delta_in);
  } else {
    if (pool_alloc((size_t)rows * sizeof(float), &delta)) return 1;
    ALPHA_CUDA(launch_overlapped(OVL_ATTN_BWD, attn_tc_delta_kernel, dim3(grid_for(rows, 32, 16)), dim3(256), 0,
                                 (const __nv_bfloat16 *)ptr<__nv_bfloat16>(o), (const __nv_bfloat16 *)ptr<__nv_bfloat16>(d_o),
                                 (float *)delta, p->o_sb, p->o_sh, p->o_st, (int)p->heads, (int)p->T, rows));
    g_launches++;
  }
  AttnBwdArgs a;
  memset(&a, 0, sizeof(a));
  a.dq = ptr<void>(dq); a.dk = ptr<void>(dk); a.dv = ptr<void>(dv);
  a.lse = ptr<float>(lse); a.delta = (const float *)delta;
  a.q_sb = p->q_sb; a.q_sh = p->q_sh; a.q_st = p->q_st;
  a.H = (int)p->heads; a.T = (int)p->T;
  a.scale = p->scale; a.cap = p->soft_cap;
  a.err = tc_error_word();
  static int attr = -1;
  if (attr != g_init_epoch) {
    ALPHA_CUDA(cudaFuncSetAttribute(attn_tc_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AK_DYN));
    attr = g_init_epoch;
  }
  const int BH = (int)(p->batch * p->heads);
  const int n_qb = (int)((p->T + 127) / 128);
  const int n_items = n_qb * BH;
  const int grid = n_items < g_sm_count ? n_items : g_sm_count;
  // One pass over the (query block, key block) tiles: the kernel that owns dK and dV of a key
  // block also multiplies each tile's dS by K; those dQ contributions (fp32, 32 KB per tile) go
  // to a workspace and a second, HBM-bound kernel adds them per query block in key-block order.
  void *part = nullptr;
  const size_t part_bytes = (size_t)BH * (n_qb * (n_qb + 1) / 2) * 128 * 64 * sizeof(float);
  if (pool_alloc(part_bytes, &part)) { if (!delta_in) pool_free(delta); return 1; }
  a.dq_part = (float *)part;
  CUtensorMap tpart;
  if (encode_tmap_2d_out(&tpart, part, ALPHA_F32, 64, (uint64_t)BH * (n_qb * (n_qb + 1) / 2) * 128, 64, 32)) {
    pool_free(part);
    if (!delta_in) pool_free(delta);
    return 1;
  }
  ALPHA_CUDA(launch_overlapped(OVL_ATTN_BWD, attn_tc_bwd_kernel, dim3(grid), dim3(ABP_THREADS), AK_DYN, tq, tk, tv, tdo, tpart, a, n_items, BH));
  g_launches++;
  ALPHA_CUDA(launch_overlapped(OVL_ATTN_BWD, attn_tc_dq_reduce_kernel, dim3((unsigned)(n_qb * 8), (unsigned)BH), dim3(256), 0,
                               (const float *)part, ptr<__nv_bfloat16>(dq), p->q_sb, p->q_sh, p->q_st, (int)p->heads,
                               (int)p->T, n_qb));
  pool_free(part);
  if (!delta_in) pool_free(delta);
  ALPHA_LAUNCHED();
  return 0;
}

}  // namespace alpha
