// bf16 GEMM on the 5th-generation tensor cores: TMA -> 128B-swizzled shared memory ->
// tcgen05.mma (fp32 accumulators in tensor memory) -> tcgen05.ld epilogue.
//
// Replaces the reference's three GEMM families for the train step — C = A*B, A*B^T, A^T*B
// (packages/helios/src/kernels/matmul.ts:17-30,574-587,1121-1136 and the cooperative-matrix
// variants in kernels/matmul-coop.ts), i.e. Backend.matmul / matmulTransposed /
// matmulTransposedA (packages/core/src/interfaces.ts:53,111-112) — and fuses what the
// reference runs as separate dispatches: GELU on the forward MLP GEMM
// (packages/autograd/src/ops.ts:426-487), the residual add, and GELU' on the dX GEMM.
//
// Shape of the kernel
//   * persistent: one CTA per SM walks output tiles (grouped order for L2 reuse);
//   * CTA tile 128 x BN (BN = 256 or 128), K step 64, 4-stage TMA ring;
//   * warp 0 = TMA producer, warp 1 = MMA issuer (one elected lane), warps 2-5 = epilogue
//     (one TMEM lane quadrant each);
//   * two accumulators in tensor memory (2 x BN columns) so the epilogue of tile i overlaps
//     the main loop of tile i+1;
//   * operands may be K-major or MN-major (the transposed layouts are read in place through
//     MN-major descriptors, nothing is transposed in memory);
//   * no cluster, no multicast: every CTA issues its own TMA loads.
//   * split-K for the weight-gradient shapes (few output tiles, K = tokens): partial
//     products go to an fp32 workspace and a second kernel adds them in split order.
// Algorithmic work: 2*M*N*K flop; bytes (M*K + N*K)*2 + M*N*e_out.
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "tc_common.cuh"

namespace alpha {

using namespace tc;

constexpr int GBM = 128, GBK = 64, GSTAGES = 4;
constexpr int GEMM_THREADS = 192;

struct GemmTcArgs {
  void *C;               // output (or the split-K workspace)
  const void *aux_in;    // ADD / GELU_BWD input
  void *aux_out;         // GELU pre-activation output
  int64_t ldc, ld_aux;
  int M, N, K;
  int tiles_m, tiles_n, splits, kb_per_split, kblocks;
  int out_f32;           // 1: C is fp32, 0: bf16
  int epilogue, accumulate;
  int tma_epi;           // 1: outputs (and epilogue operands) move through shared memory with TMA
  uint32_t *err;
};

// tanh-approximation GELU with the hardware tanh (MUFU): the epilogues run on bf16 data, whose
// resolution (2^-8) is far coarser than tanh.approx's error.
__device__ __forceinline__ float gelu_fast(float x) {
  const float c = 0.7978845608028654f;
  return 0.5f * x * (1.f + tc::tanh_approx(c * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_grad_fast(float x) {
  const float c = 0.7978845608028654f;
  const float t = tc::tanh_approx(c * (x + 0.044715f * x * x * x));
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * c * (1.f + 3.f * 0.044715f * x * x);
}

template <int BN>
struct GemmSmemLayout {
  static constexpr int A_BYTES = GBM * GBK * 2;
  static constexpr int B_BYTES = BN * GBK * 2;
  // epilogue staging: 4 warps x 2 buffers x (32 rows x 128 bytes), 128B-swizzled TMA boxes
  static constexpr int STAGE_OFF = GSTAGES * (A_BYTES + B_BYTES);
  static constexpr int STAGE_BYTES = 4 * 2 * 4096;
  static constexpr int BAR_OFF = STAGE_OFF + STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256;  // barriers + tmem base + abort flag
  static constexpr int DYN = TOTAL + 1024;     // slack to align the base to 1024 B
};

__device__ __forceinline__ void tile_coords(const GemmTcArgs &g, int tile, int &split, int &mt, int &nt) {
  const int per_split = g.tiles_m * g.tiles_n;
  split = tile / per_split;
  const int r = tile - split * per_split;
  constexpr int GROUP_M = 8;
  const int group = r / (GROUP_M * g.tiles_n);
  const int first_m = group * GROUP_M;
  const int gm = min(GROUP_M, g.tiles_m - first_m);
  const int in_group = r - group * GROUP_M * g.tiles_n;
  mt = first_m + in_group % gm;
  nt = in_group / gm;
}

template <typename OutT>
__device__ __forceinline__ void epilogue_store_chunk(const GemmTcArgs &g, const uint32_t (&r)[32], int64_t row,
                                                     int col0, bool row_ok) {
  if (!row_ok) return;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
  const bool full = col0 + 32 <= g.N;
  OutT *crow = (OutT *)g.C + row * g.ldc + col0;
  constexpr int V = Vec16<OutT>::N;
  const bool vec_c = full && aligned16(crow);
  if (g.epilogue != ALPHA_EPI_NONE) {
    // aux tensors share the output's element type
    if (g.epilogue == ALPHA_EPI_GELU) {
      OutT *arow = (OutT *)g.aux_out + row * g.ld_aux + col0;
      if (full && aligned16(arow)) {
#pragma unroll
        for (int c = 0; c < 32; c += V) {
          Vec16<OutT> t;
          t.set(&v[c]);
          t.store(arow + c);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; j++)
          if (col0 + j < g.N) arow[j] = from_f32<OutT>(v[j]);
      }
#pragma unroll
      for (int j = 0; j < 32; j++) v[j] = gelu_f(v[j]);
    } else {
      const OutT *arow = (const OutT *)g.aux_in + row * g.ld_aux + col0;
      float x[32];
      if (full && aligned16(arow)) {
#pragma unroll
        for (int c = 0; c < 32; c += V) {
          Vec16<OutT> t;
          t.load(arow + c);
          t.get(&x[c]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; j++) x[j] = (col0 + j < g.N) ? to_f32(arow[j]) : 0.f;
      }
      if (g.epilogue == ALPHA_EPI_ADD) {
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] += x[j];
      } else {
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] *= gelu_grad_f(x[j]);
      }
    }
  }
  if (g.accumulate) {
    if (vec_c) {
#pragma unroll
      for (int c = 0; c < 32; c += V) {
        Vec16<OutT> t;
        float x[V];
        t.load(crow + c);
        t.get(x);
#pragma unroll
        for (int j = 0; j < V; j++) v[c + j] += x[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j++)
        if (col0 + j < g.N) v[j] += to_f32(crow[j]);
    }
  }
  if (vec_c) {
#pragma unroll
    for (int c = 0; c < 32; c += V) {
      Vec16<OutT> t;
      t.set(&v[c]);
      t.store(crow + c);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; j++)
      if (col0 + j < g.N) crow[j] = from_f32<OutT>(v[j]);
  }
}

// Epilogue of one 128 x BN tile for one warp (32 accumulator rows) through shared memory.
// Direct register->global stores make every lane write its own row, 32 cache lines per
// instruction, and were measured to cost a third of the kernel on the K = 768 shapes; here
// each warp stages 32 rows x 128 bytes in a 128B-swizzled buffer (conflict-free 16-byte
// writes) and one lane hands the box to the TMA unit, which writes full lines and clips at
// the matrix edge.  Epilogue operands (residual, saved pre-activation) arrive the same way
// by a TMA load into the buffer the result will leave from.  Two buffers per warp: they
// alternate (plain / ADD / GELU') or hold the pre-activation and the activation (GELU).
template <typename OutT, int BN>
__device__ __forceinline__ bool epilogue_tile_tma(const GemmTcArgs &g, const CUtensorMap *tmap_c,
                                                  const CUtensorMap *tmap_aux, uint32_t t_row, int row0, int n0,
                                                  int lane, uint8_t *stage, uint32_t stage_u32, uint32_t aux_bar,
                                                  uint32_t &aux_phase, uint32_t &chunk_count,
                                                  volatile uint32_t *abort_flag) {
  constexpr int CH = 128 / (int)sizeof(OutT);  // columns per staged chunk (64 bf16 / 32 f32)
  constexpr int V = Vec16<OutT>::N;
  const bool gelu = g.epilogue == ALPHA_EPI_GELU;
  const bool has_in = g.epilogue == ALPHA_EPI_ADD || g.epilogue == ALPHA_EPI_GELU_BWD;
  const uint32_t sw = (uint32_t)(lane & 7);
  const uint64_t policy = l2_policy_evict_first();
#pragma unroll 1
  for (int c = 0; c < BN / CH; c++) {
    const int col0 = n0 + c * CH;
    if (col0 >= g.N) break;  // warp-uniform
    const int buf = gelu ? 1 : (int)(chunk_count & 1);
    chunk_count++;
    if (lane == 0) {  // the buffer(s) about to be written must have been read out by their last store
      if (gelu) bulk_wait_read<0>(); else bulk_wait_read<1>();
    }
    __syncwarp();
    uint8_t *bp = stage + buf * 4096 + lane * 128;
    const uint32_t bu = stage_u32 + buf * 4096;
    if (has_in && lane == 0) {
      mbar_expect_tx(aux_bar, 4096);
      tma_load_2d(bu, tmap_aux, aux_bar, col0, row0);
    }
    float v[CH];
#pragma unroll
    for (int k = 0; k < CH / 32; k++) {
      uint32_t r[32];
      tmem_ld_32x32(t_row + c * CH + k * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; i++) v[k * 32 + i] = __uint_as_float(r[i]);
    }
    if (has_in) {
      if (!mbar_wait(aux_bar, aux_phase, abort_flag)) return false;
      aux_phase ^= 1;
#pragma unroll
      for (int q = 0; q < 8; q++) {
        Vec16<OutT> t;
        float x[V];
        t.load(reinterpret_cast<const OutT *>(bp + ((q ^ sw) << 4)));
        t.get(x);
#pragma unroll
        for (int j = 0; j < V; j++)
          v[q * V + j] = g.epilogue == ALPHA_EPI_ADD ? v[q * V + j] + x[j] : v[q * V + j] * gelu_grad_fast(x[j]);
      }
    }
    if (gelu) {  // buffer 0 takes the pre-activation, buffer 1 the activation
      uint8_t *ap = stage + lane * 128;
#pragma unroll
      for (int q = 0; q < 8; q++) {
        Vec16<OutT> t;
        t.set(&v[q * V]);
        t.store(reinterpret_cast<OutT *>(ap + ((q ^ sw) << 4)));
      }
#pragma unroll
      for (int j = 0; j < CH; j++) v[j] = gelu_fast(v[j]);
    }
#pragma unroll
    for (int q = 0; q < 8; q++) {
      Vec16<OutT> t;
      t.set(&v[q * V]);
      t.store(reinterpret_cast<OutT *>(bp + ((q ^ sw) << 4)));
    }
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      if (gelu) tma_store_2d_hint(tmap_aux, stage_u32, col0, row0, policy);
      tma_store_2d_hint(tmap_c, bu, col0, row0, policy);
      bulk_commit();
    }
  }
  return true;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_aux, GemmTcArgs g) {
  using L = GemmSmemLayout<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t a_base = smem_base;
  const uint32_t b_base = smem_base + GSTAGES * L::A_BYTES;
  const uint32_t bar_base = smem_base + L::BAR_OFF;
  // barrier slots (8 bytes each): full[4], empty[4], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (GSTAGES + s); };
  auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * GSTAGES + s); };
  auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * GSTAGES + 2 + s); };
  auto aux_bar = [&](int q) { return bar_base + 8u * (2 * GSTAGES + 4 + q); };  // one per epilogue warp
  uint32_t *tmem_slot = (uint32_t *)(smem + L::BAR_OFF + 8 * (2 * GSTAGES + 8));
  volatile uint32_t *abort_flag = (volatile uint32_t *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GSTAGES; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int q = 0; q < 4; q++) mbar_init(aux_bar(q), 1);
    for (int s = 0; s < 2; s++) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), 4);
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
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = g.tiles_m * g.tiles_n * g.splits;

  if (warp == 0) {
    // ── TMA producer ───────────────────────────────────────────────────────
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int split, mt, nt;
        tile_coords(g, tile, split, mt, nt);
        const int m0 = mt * GBM, n0 = nt * BN;
        const int kb0 = split * g.kb_per_split;
        const int kb1 = min(g.kblocks, kb0 + g.kb_per_split);
        for (int kb = kb0; kb < kb1; kb++) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), L::A_BYTES + L::B_BYTES);
          const uint32_t a_dst = a_base + stage * L::A_BYTES;
          const uint32_t b_dst = b_base + stage * L::B_BYTES;
          const int k0 = kb * GBK;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < GBM / 64; i++) tma_load_2d(a_dst + i * 8192, &tmap_a, full_bar(stage), m0 + i * 64, k0);
          } else {
            tma_load_2d(a_dst, &tmap_a, full_bar(stage), k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; i++) tma_load_2d(b_dst + i * 8192, &tmap_b, full_bar(stage), n0 + i * 64, k0);
          } else {
            tma_load_2d(b_dst, &tmap_b, full_bar(stage), k0, n0);
          }
          if (++stage == GSTAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ── MMA issuer ─────────────────────────────────────────────────────────
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(GBM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, it++) {
        int split, mt, nt;
        tile_coords(g, tile, split, mt, nt);
        const int kb0 = split * g.kb_per_split;
        const int kb1 = min(g.kblocks, kb0 + g.kb_per_split);
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; kb++) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_s = a_base + stage * L::A_BYTES;
          const uint32_t b_s = b_base + stage * L::B_BYTES;
#pragma unroll
          for (int k = 0; k < GBK / 16; k++) {
            const uint64_t adesc = A_MN ? make_smem_desc(a_s + k * 2048, 8192, 1024)
                                        : make_smem_desc(a_s + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(b_s + k * 2048, 8192, 1024)
                                        : make_smem_desc(b_s + k * 32, 16, 1024);
            mma_bf16_ss(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          mma_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
          if (++stage == GSTAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) mma_commit(tfull_bar(acc));  // accumulator complete
      }
    }
  } else {
    // ── epilogue warps (2..5): TMEM -> registers -> global ─────────────────
    const int quad = warp & 3;  // the TMEM lane quadrant this warp may read
    int it = 0;
    bool ok = true;
    uint8_t *stage = smem + L::STAGE_OFF + quad * 8192;
    const uint32_t stage_u32 = smem_base + L::STAGE_OFF + quad * 8192;
    uint32_t aux_phase = 0, chunk_count = 0;
    if (g.tma_epi && lane == 0) {
      tma_prefetch_desc(&tmap_c);
      if (g.epilogue != ALPHA_EPI_NONE) tma_prefetch_desc(&tmap_aux);
    }
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, it++) {
      int split, mt, nt;
      tile_coords(g, tile, split, mt, nt);
      const int m0 = mt * GBM, n0 = nt * BN;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row_in_tile = quad * 32 + lane;
      const int64_t row = (int64_t)m0 + row_in_tile;
      const bool row_ok = row < g.M;
      const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(quad * 32) << 16);
      if (g.tma_epi) {
        const int row0 = m0 + quad * 32;
        if (row0 < g.M) {  // warp-uniform: a quadrant entirely below the matrix has nothing to store
          ok = g.out_f32 ? epilogue_tile_tma<float, BN>(g, &tmap_c, &tmap_aux, t_row, row0, n0, lane, stage, stage_u32,
                                                        aux_bar(quad), aux_phase, chunk_count, abort_flag)
                         : epilogue_tile_tma<__nv_bfloat16, BN>(g, &tmap_c, &tmap_aux, t_row, row0, n0, lane, stage,
                                                                stage_u32, aux_bar(quad), aux_phase, chunk_count,
                                                                abort_flag);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
        continue;
      }
      GemmTcArgs gl = g;
      if (g.splits > 1) gl.C = (float *)g.C + (int64_t)split * g.M * g.N;  // workspace slab, ldc = N
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        const int col0 = n0 + c * 32;
        if (col0 >= g.N) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        if (gl.out_f32)
          epilogue_store_chunk<float>(gl, r, row, col0, row_ok);
        else
          epilogue_store_chunk<__nv_bfloat16>(gl, r, row, col0, row_ok);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
    if (g.tma_epi && lane == 0) bulk_wait<0>();  // all stores have left shared memory and landed
  }

  // ── teardown ─────────────────────────────────────────────────────────────
  if (*abort_flag) {
    // A wait ran out: give copies in flight time to land before the block's shared
    // memory is released, then report.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
    if (threadIdx.x == 0 && g.err) atomicExch(g.err, 0x6E000000u | (uint32_t)(blockIdx.x & 0xFFFF));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// C (+)= sum_s ws[s]  — split order is fixed, so the result is reproducible.  ws holds
// `splits` dense [M, N] fp32 slabs; four columns per thread when the rows allow it.
template <typename OutT>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ ws, OutT *C, int64_t M, int64_t N,
                                                            int64_t ldc, int splits, int accumulate, int vec4) {
  const int64_t total = M * N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (vec4) {
    const int64_t n4 = total / 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
      float4 s = reinterpret_cast<const float4 *>(ws)[i];
      for (int k = 1; k < splits; k++) {
        const float4 t = reinterpret_cast<const float4 *>(ws + (int64_t)k * total)[i];
        s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
      }
      const int64_t e = i * 4, m = e / N, n = e - m * N;
      OutT *dst = C + m * ldc + n;
      float o[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
      for (int j = 0; j < 4; j++) dst[j] = from_f32<OutT>(accumulate ? to_f32(dst[j]) + o[j] : o[j]);
    }
    return;
  }
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    float s = 0.f;
    for (int k = 0; k < splits; k++) s += ws[(int64_t)k * total + i];
    const int64_t m = i / N, n = i - m * N;
    OutT *dst = C + m * ldc + n;
    *dst = from_f32<OutT>(accumulate ? to_f32(*dst) + s : s);
  }
}

// ── host ────────────────────────────────────────────────────────────────────
struct TmapKey {
  uint64_t base, inner, outer, ld;
  uint32_t box_inner, box_outer;
  bool operator==(const TmapKey &o) const {
    return base == o.base && inner == o.inner && outer == o.outer && ld == o.ld && box_inner == o.box_inner &&
           box_outer == o.box_outer;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey &k) const {
    uint64_t h = k.base * 0x9e3779b97f4a7c15ull;
    h ^= (k.inner + 0x7f4a7c15ull) * 0xff51afd7ed558ccdull;
    h ^= (k.outer << 17) ^ (k.ld << 31) ^ ((uint64_t)k.box_inner << 7) ^ ((uint64_t)k.box_outer << 3);
    return (size_t)(h ^ (h >> 29));
  }
};
static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmaps;
static std::mutex g_tmap_mu;

static int get_tmap(CUtensorMap *out, const void *base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                    uint32_t box_outer) {
  TmapKey key{(uint64_t)(uintptr_t)base, inner, outer, ld, box_inner, box_outer};
  std::lock_guard<std::mutex> lk(g_tmap_mu);
  auto it = g_tmaps.find(key);
  if (it != g_tmaps.end()) {
    *out = it->second;
    return 0;
  }
  if (encode_tmap_2d_bf16(out, base, inner, outer, ld, box_inner, box_outer)) return 1;
  if (g_tmaps.size() > 4096) g_tmaps.clear();
  g_tmaps[key] = *out;
  return 0;
}

static int get_tmap_out(CUtensorMap *out, const void *base, int dtype, uint64_t inner, uint64_t outer, uint64_t ld) {
  // key: box_inner carries the dtype (64 bf16 / 32 f32 columns), box_outer = 32 rows marks an output map
  TmapKey key{(uint64_t)(uintptr_t)base, inner, outer, ld, dtype == ALPHA_F32 ? 32u : 64u, 32u};
  std::lock_guard<std::mutex> lk(g_tmap_mu);
  auto it = g_tmaps.find(key);
  if (it != g_tmaps.end()) {
    *out = it->second;
    return 0;
  }
  if (encode_tmap_2d_out(out, base, dtype, inner, outer, ld, 32)) return 1;
  if (g_tmaps.size() > 4096) g_tmaps.clear();
  g_tmaps[key] = *out;
  return 0;
}

template <int BN, bool A_MN, bool B_MN>
static int launch_variant(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc_, const CUtensorMap &tx,
                          const GemmTcArgs &g, int grid) {
  using L = GemmSmemLayout<BN>;
  static bool attr = false;
  if (!attr) {
    ALPHA_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN));
    attr = true;
  }
  gemm_tc_kernel<BN, A_MN, B_MN><<<grid, GEMM_THREADS, L::DYN, g_stream>>>(ta, tb, tc_, tx, g);
  ALPHA_LAUNCHED();
  return 0;
}

int gemm_tc_launch(int layout, alpha_buf A, alpha_buf B, alpha_buf C, int64_t M, int64_t N, int64_t K, int64_t lda,
                   int64_t ldb, int64_t ldc, int out_dtype, int epilogue, alpha_buf aux, int64_t ld_aux,
                   int accumulate) {
  if (M == 0 || N == 0) return 0;
  ALPHA_CHECK(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "alpha_gemm: dimension exceeds int32");
  ALPHA_CHECK(out_dtype == ALPHA_F32 || out_dtype == ALPHA_BF16, "alpha_gemm: bad out dtype %d", out_dtype);
  if (K == 0) {
    // empty contraction: C = epi(0) is only meaningful for NONE
    ALPHA_CHECK(epilogue == ALPHA_EPI_NONE, "alpha_gemm: K == 0 with an epilogue");
    if (!accumulate)
      ALPHA_CUDA(cudaMemset2DAsync(ptr<void>(C), ldc * dtype_size(out_dtype), 0, N * dtype_size(out_dtype), M, g_stream));
    return 0;
  }
  ProfScope prof(PROF_GEMM_TC, 2.0 * (double)M * (double)N * (double)K);
  const bool a_mn = layout == ALPHA_GEMM_TN;
  const bool b_mn = layout != ALPHA_GEMM_NT;
  const int BN = N <= 128 ? 128 : 256;
  CUtensorMap ta, tb;
  // A: K-major [M,K] (inner K) or M-major [K,M] (inner M)
  if (a_mn) { if (get_tmap(&ta, ptr<void>(A), M, K, lda, 64, 64)) return 1; }
  else      { if (get_tmap(&ta, ptr<void>(A), K, M, lda, 64, GBM)) return 1; }
  if (b_mn) { if (get_tmap(&tb, ptr<void>(B), N, K, ldb, 64, 64)) return 1; }
  else      { if (get_tmap(&tb, ptr<void>(B), K, N, ldb, 64, BN)) return 1; }

  GemmTcArgs g;
  memset(&g, 0, sizeof(g));
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.tiles_m = (int)((M + GBM - 1) / GBM);
  g.tiles_n = (int)((N + BN - 1) / BN);
  g.kblocks = (int)((K + GBK - 1) / GBK);
  g.err = tc_error_word();
  const int tiles = g.tiles_m * g.tiles_n;
  int splits = 1;
  if (epilogue == ALPHA_EPI_NONE && tiles * 2 <= g_sm_count && g.kblocks >= 16) {
    splits = g_sm_count / tiles;
    if (splits > g.kblocks / 8) splits = g.kblocks / 8;
    if (splits < 1) splits = 1;
  }
  g.kb_per_split = (g.kblocks + splits - 1) / splits;
  splits = (g.kblocks + g.kb_per_split - 1) / g.kb_per_split;  // drop empty splits
  g.splits = splits;
  void *ws = nullptr;
  if (splits > 1) {
    if (pool_alloc((size_t)splits * M * N * sizeof(float), &ws)) return 1;
    g.C = ws; g.ldc = N; g.out_f32 = 1; g.epilogue = ALPHA_EPI_NONE; g.accumulate = 0;
  } else {
    g.C = ptr<void>(C); g.ldc = ldc; g.out_f32 = out_dtype == ALPHA_F32;
    g.epilogue = epilogue; g.accumulate = accumulate;
    g.aux_in = ptr<void>(aux); g.aux_out = ptr<void>(aux); g.ld_aux = ld_aux;
    if (epilogue != ALPHA_EPI_NONE) ALPHA_CHECK(aux != 0, "alpha_gemm: epilogue %d needs an aux buffer", epilogue);
  }
  // Outputs leave through shared memory + TMA stores when the layout allows a tensor map
  // (16-byte aligned base and rows) and nothing has to be read back from C.
  CUtensorMap tcm, txm;
  memset(&tcm, 0, sizeof(tcm));
  memset(&txm, 0, sizeof(txm));
  const size_t oes = dtype_size(out_dtype);
  g.tma_epi = 0;
  if (splits == 1 && !accumulate && (C & 15) == 0 && (ldc * oes) % 16 == 0 &&
      (epilogue == ALPHA_EPI_NONE || ((aux & 15) == 0 && (ld_aux * oes) % 16 == 0))) {
    if (get_tmap_out(&tcm, ptr<void>(C), out_dtype, N, M, ldc)) return 1;
    if (epilogue != ALPHA_EPI_NONE && get_tmap_out(&txm, ptr<void>(aux), out_dtype, N, M, ld_aux)) return 1;
    g.tma_epi = 1;
  }
  const int total = tiles * splits;
  const int grid = total < g_sm_count ? total : g_sm_count;
  int rc;
#define GEMM_VARIANT(BNV)                                                                               \
  (a_mn ? launch_variant<BNV, true, true>(ta, tb, tcm, txm, g, grid)                                    \
        : (b_mn ? launch_variant<BNV, false, true>(ta, tb, tcm, txm, g, grid)                           \
                : launch_variant<BNV, false, false>(ta, tb, tcm, txm, g, grid)))
  rc = BN == 256 ? GEMM_VARIANT(256) : GEMM_VARIANT(128);
#undef GEMM_VARIANT
  if (rc == 0 && splits > 1) {
    const int vec4 = (N % 4 == 0) ? 1 : 0;   // ws slabs are 512-byte aligned and dense
    const int rgrid = grid_for(M * N / (vec4 ? 4 : 1) + 1, 256, 8);
    if (out_dtype == ALPHA_F32)
      splitk_reduce_kernel<float><<<rgrid, 256, 0, g_stream>>>((const float *)ws, ptr<float>(C), M, N, ldc, splits,
                                                               accumulate, vec4);
    else
      splitk_reduce_kernel<__nv_bfloat16><<<rgrid, 256, 0, g_stream>>>((const float *)ws, ptr<__nv_bfloat16>(C), M, N,
                                                                       ldc, splits, accumulate, vec4);
    g_launches++;
  }
  if (ws) pool_free(ws);
  return rc;
}

int gemm_f32_launch(int layout, alpha_buf A, alpha_buf B, alpha_buf C, int64_t M, int64_t N, int64_t K, int64_t lda,
                    int64_t ldb, int64_t ldc, int epilogue, alpha_buf aux, int64_t ld_aux, int accumulate,
                    int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_c);

}  // namespace alpha

using namespace alpha;

extern "C" int alpha_gemm(int layout, alpha_buf A, alpha_buf B, alpha_buf C, int64_t M, int64_t N, int64_t K,
                          int64_t lda, int64_t ldb, int64_t ldc, int in_dtype, int out_dtype, int epilogue,
                          alpha_buf aux, int64_t ld_aux, int accumulate) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(layout >= ALPHA_GEMM_NT && layout <= ALPHA_GEMM_TN, "alpha_gemm: bad layout %d", layout);
  ALPHA_CHECK(epilogue >= ALPHA_EPI_NONE && epilogue <= ALPHA_EPI_GELU_BWD, "alpha_gemm: bad epilogue %d", epilogue);
  if (in_dtype == ALPHA_F32) {
    ALPHA_CHECK(out_dtype == ALPHA_F32, "alpha_gemm: fp32 inputs produce fp32 output");
    return gemm_f32_launch(layout, A, B, C, M, N, K, lda, ldb, ldc, epilogue, aux, ld_aux, accumulate, 1, 0, 0, 0);
  }
  ALPHA_CHECK(in_dtype == ALPHA_BF16, "alpha_gemm: unsupported input dtype %d", in_dtype);
  return gemm_tc_launch(layout, A, B, C, M, N, K, lda, ldb, ldc, out_dtype, epilogue, aux, ld_aux, accumulate);
}
