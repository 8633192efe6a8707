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
//   * pair form (the default for M > 128, N > 128): two CTAs of a cluster share a 256 x 256
//     tile through tcgen05 cta_group::2 — each loads its 128 rows of A and 128 of the 256
//     rows of B, so an SM fetches 32 KB per K step instead of 48 KB for the same tensor-core
//     work (the single-CTA form is bound by what one SM can pull from L2), 6-stage ring;
//   * single form: CTA tile 128 x BN (BN = 256 or 128), K step 64, 4-stage TMA ring;
//   * warp 0 = TMA producer, warp 1 = MMA issuer (one elected lane), warps 2-5 = epilogue
//     (one TMEM lane quadrant each);
//   * two accumulators in tensor memory (2 x BN columns) so the epilogue of tile i overlaps
//     the main loop of tile i+1;
//   * operands may be K-major or MN-major (the transposed layouts are read in place through
//     MN-major descriptors, nothing is transposed in memory);
//   * every CTA issues its own TMA loads (nothing is broadcast between CTAs);
//   * split-K for the weight-gradient shapes (few output tiles, K = tokens): partial
//     products go to an fp32 workspace and a second kernel adds them in split order.
// Algorithmic work: 2*M*N*K flop; bytes (M*K + N*K)*2 + M*N*e_out.
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "tc_common.cuh"

namespace alpha {

using namespace tc;

constexpr int GBM = 128, GBK = 64;
constexpr int ALPHA_EPI_ROWDOT = 4;   // internal epilogue code (alpha_gemm_nn_rowdot)
constexpr int GEMM_THREADS = 192;

struct GemmTcArgs {
  void *C;               // output (or the split-K workspace)
  const void *aux_in;    // ADD / GELU_BWD input
  void *aux_out;         // GELU pre-activation output
  int64_t ldc, ld_aux;
  int M, N, K;
  int tiles_m, tiles_n, splits, kb_per_split, kblocks;
  int m_pad;             // split-K: rows per workspace slab (tiles_m * tile rows), >= M
  // ALPHA_EPI_ROWDOT (internal): C = acc and, per row and 64-column group h (one attention head),
  // rowdot[(row / rd_T * rd_H + h) * rd_T + row % rd_T] = sum_j bf16(acc[row, 64h + j]) * aux[row, 64h + j]
  float *rowdot;
  int rd_T, rd_H;
  int out_f32;           // 1: C is fp32, 0: bf16
  int epilogue, accumulate;
  int tma_epi;           // 1: outputs (and epilogue operands) move through shared memory with TMA
  uint32_t *err;
};

// tanh-approximation GELU with the hardware tanh (MUFU): the epilogues run on bf16 data, whose
// resolution (2^-8) is far coarser than tanh.approx's error.  Two elements at a time with
// packed fp32 arithmetic: the epilogue warps are alone on their SM sub-partitions, so their
// instruction count is what limits the GELU epilogues.
__device__ __forceinline__ void gelu_fast2(float &a, float &b) {
  const float c = 0.7978845608028654f, c3 = c * 0.044715f;
  const uint64_t x = tc::f2_pack(a, b);
  const uint64_t x2 = tc::f2_mul(x, x);
  float i0, i1;
  tc::f2_unpack(tc::f2_mul(x, tc::f2_fma(x2, tc::f2_pack(c3, c3), tc::f2_pack(c, c))), i0, i1);
  const uint64_t t = tc::f2_pack(tc::tanh_approx(i0), tc::tanh_approx(i1));
  const uint64_t h = tc::f2_mul(x, tc::f2_pack(0.5f, 0.5f));
  tc::f2_unpack(tc::f2_fma(h, t, h), a, b);
}
// (ga, gb) *= gelu'(xa, xb)
__device__ __forceinline__ void gelu_grad_mul2(float &ga, float &gb, float xa, float xb) {
  const float c = 0.7978845608028654f, c3 = c * 0.044715f;
  const uint64_t half = tc::f2_pack(0.5f, 0.5f), one = tc::f2_pack(1.f, 1.f);
  const uint64_t x = tc::f2_pack(xa, xb);
  const uint64_t x2 = tc::f2_mul(x, x);
  float i0, i1;
  tc::f2_unpack(tc::f2_mul(x, tc::f2_fma(x2, tc::f2_pack(c3, c3), tc::f2_pack(c, c))), i0, i1);
  const uint64_t t = tc::f2_pack(tc::tanh_approx(i0), tc::tanh_approx(i1));
  const uint64_t q = tc::f2_fma(x2, tc::f2_pack(3.f * c3, 3.f * c3), tc::f2_pack(c, c));   // c (1 + 3 * 0.044715 x^2)
  const uint64_t sech2 = tc::f2_fma(tc::f2_mul(t, t), tc::f2_pack(-1.f, -1.f), one);      // 1 - t^2
  const uint64_t w = tc::f2_mul(tc::f2_mul(tc::f2_mul(x, half), sech2), q);               // 0.5 x (1 - t^2) c (...)
  const uint64_t d = tc::f2_add(tc::f2_fma(t, half, half), w);                            // 0.5 (1 + t) + w
  tc::f2_unpack(tc::f2_mul(tc::f2_pack(ga, gb), d), ga, gb);
}

// Per-CTA shared memory.  PAIR: the CTA holds 128 rows of A and BN/2 rows of B per stage.
// WIDE (pair form with the GELU epilogue, whose per-element work is several times that of a
// plain store): eight epilogue warps instead of four — two per TMEM lane quadrant, taking
// alternate column chunks — paid for with one pipeline stage.
template <int BN, bool PAIR, bool WIDE = false>
struct GemmSmemLayout {
  static constexpr int STAGES = PAIR ? (WIDE ? 5 : 6) : 4;
  static constexpr int EPI_WARPS = WIDE ? 8 : 4;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int A_BYTES = GBM * GBK * 2;
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;
  static constexpr int B_BYTES = B_ROWS * GBK * 2;
  // epilogue staging: 4 warps x 2 buffers x (32 rows x 128 bytes), 128B-swizzled TMA boxes
  static constexpr int STAGE_OFF = STAGES * (A_BYTES + B_BYTES);
  static constexpr int EPI_BUFS = 2;                       // 4 KB staging buffers per epilogue warp
  static constexpr int STAGE_BYTES = EPI_WARPS * EPI_BUFS * 4096;
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
template <typename OutT, int BN, bool WIDE>
__device__ __forceinline__ bool epilogue_tile_tma(const GemmTcArgs &g, const CUtensorMap *tmap_c,
                                                  const CUtensorMap *tmap_aux, uint32_t t_row, int row0, int n0,
                                                  int lane, uint8_t *stage, uint32_t stage_u32, uint32_t aux_bar,
                                                  uint32_t &aux_phase, uint32_t &chunk_count,
                                                  volatile uint32_t *abort_flag, int half) {
  constexpr int CH = 128 / (int)sizeof(OutT);  // columns per staged chunk (64 bf16 / 32 f32)
  constexpr int V = Vec16<OutT>::N;
  const bool gelu = g.epilogue == ALPHA_EPI_GELU;
  const bool rowdot = g.epilogue == ALPHA_EPI_ROWDOT;
  const bool has_in = g.epilogue == ALPHA_EPI_ADD || g.epilogue == ALPHA_EPI_GELU_BWD || rowdot;
  const uint32_t sw = (uint32_t)(lane & 7);
  const uint64_t policy = l2_policy_evict_first();
#pragma unroll 1
  for (int c = 0; c < BN / CH; c++) {
    const int col0 = n0 + c * CH;
    if (col0 >= g.N) break;  // warp-uniform
    if (WIDE && (c & 1) != half) continue;  // the quadrant's other warp takes this chunk
    // plain / ADD / GELU': the two buffers alternate.  GELU: buffer 0 takes the pre-activation,
    // buffer 1 the activation, so every chunk waits for the stores of its predecessor.
    const int pre_buf = 0;
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
      float dot = 0.f;   // ROWDOT: this lane's row of one head, (rounded) output times operand
#pragma unroll
      for (int q = 0; q < 8; q++) {
        Vec16<OutT> t;
        float x[V];
        t.load(reinterpret_cast<const OutT *>(bp + ((q ^ sw) << 4)));
        t.get(x);
        if (g.epilogue == ALPHA_EPI_ADD) {
#pragma unroll
          for (int j = 0; j < V; j++) v[q * V + j] += x[j];
        } else if (rowdot) {
#pragma unroll
          for (int j = 0; j < V; j++) dot = fmaf(to_f32(from_f32<OutT>(v[q * V + j])), x[j], dot);
        } else {
#pragma unroll
          for (int j = 0; j < V; j += 2) gelu_grad_mul2(v[q * V + j], v[q * V + j + 1], x[j], x[j + 1]);
        }
      }
      if (rowdot) {
        const int row = row0 + lane;
        if (row < g.M) {
          const int b = row / g.rd_T, tpos = row - b * g.rd_T;
          g.rowdot[((int64_t)b * g.rd_H + col0 / CH) * g.rd_T + tpos] = dot;
        }
      }
    }
    if (gelu) {  // buffer 0 takes the pre-activation, buffer 1 the activation
      uint8_t *ap = stage + pre_buf * 4096 + lane * 128;
#pragma unroll
      for (int q = 0; q < 8; q++) {
        Vec16<OutT> t;
        t.set(&v[q * V]);
        t.store(reinterpret_cast<OutT *>(ap + ((q ^ sw) << 4)));
      }
#pragma unroll
      for (int j = 0; j < CH; j += 2) gelu_fast2(v[j], v[j + 1]);
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
      if (gelu) tma_store_2d_hint(tmap_aux, stage_u32 + pre_buf * 4096, col0, row0, policy);
      tma_store_2d_hint(tmap_c, bu, col0, row0, policy);
      bulk_commit();
    }
  }
  return true;
}

// One GEMM of a launch: its operand and output maps and its arguments.
struct GemmProblem {
  const CUtensorMap *a, *b, *c, *aux;
  const GemmTcArgs *g;
};

// GROUP2: the launch carries a second, independent GEMM of the same layout and K (p1).  The tile
// walkers take p0's tiles first and p1's after them, so that two GEMMs which alone would each
// fill half of the device (and would have to split K to fill it) run side by side, unsplit.
template <int BN, bool A_MN, bool B_MN, bool PAIR, bool WIDE, bool GROUP2 = false>
__device__ __forceinline__ void gemm_tc_body(const GemmProblem &p0, const GemmProblem &p1) {
  using L = GemmSmemLayout<BN, PAIR, WIDE>;
  const GemmTcArgs &g = *p0.g;
  const int tiles_p0 = g.tiles_m * g.tiles_n * g.splits;
  // the problem a tile index belongs to and the index inside that problem
  auto problem_of = [&](int tile, int &local) -> const GemmProblem & {
    if (GROUP2 && tile >= tiles_p0) {
      local = tile - tiles_p0;
      return p1;
    }
    local = tile;
    return p0;
  };
  constexpr int STAGES = L::STAGES;
  constexpr int TILE_M = PAIR ? 2 * GBM : GBM;  // rows of C per tile walker (CTA or CTA pair)
  extern __shared__ uint8_t smem_raw[];
  // the pair's MMA addresses both CTAs' operands by one offset, so the aligned bases must
  // sit at the same offset in both CTAs: the dynamic window starts at the same address in
  // every CTA of a launch, hence so does its 1024-byte round-up
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t a_base = smem_base;
  const uint32_t b_base = smem_base + STAGES * L::A_BYTES;
  const uint32_t bar_base = smem_base + L::BAR_OFF;
  // barrier slots (8 bytes each): full[S], empty[S], tmem_full[2], tmem_empty[2], aux[4]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 + s); };
  auto aux_bar = [&](int q) { return bar_base + 8u * (2 * STAGES + 4 + q); };  // one per epilogue warp
  uint32_t *tmem_slot = (uint32_t *)(smem + L::BAR_OFF + 8 * (2 * STAGES + 4 + L::EPI_WARPS));
  volatile uint32_t *abort_flag = (volatile uint32_t *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // 0 = the pair's leader
  const int walker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int n_walkers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int q = 0; q < L::EPI_WARPS; q++) mbar_init(aux_bar(q), 1);
    for (int s = 0; s < 2; s++) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), (PAIR ? 2 : 1) * L::EPI_WARPS);  // the leader's collects both CTAs' epilogue warps
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
  if (PAIR) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  // everything above touched only this SM; global memory is first read or written below
  grid_dependency_trigger();
  grid_dependency_wait();
  const uint32_t tmem_base = *tmem_slot;
  // The pair's MMA writes both CTAs' tensor memory at one address, so both allocations must
  // start at the same column; each CTA takes all 512 columns of its SM, which puts them at 0.
  if (PAIR && (tmem_base & 0xFFFFu) != 0 && threadIdx.x == 0 && g.err) atomicExch(g.err, 0x6F000000u);

  const int total_tiles = tiles_p0 + (GROUP2 ? p1.g->tiles_m * p1.g->tiles_n * p1.g->splits : 0);

  if (warp == 0) {
    // ── TMA producer (each CTA loads its own share); the warp runs the loop, one lane issues ──
    {
      if (elect_one()) {
        tma_prefetch_desc(p0.a);
        tma_prefetch_desc(p0.b);
        if (GROUP2) {
          tma_prefetch_desc(p1.a);
          tma_prefetch_desc(p1.b);
        }
      }
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = walker; tile < total_tiles && ok; tile += n_walkers) {
        int split, mt, nt, local;
        const GemmProblem &pr = problem_of(tile, local);
        const GemmTcArgs &g = *pr.g;
        const CUtensorMap &tmap_a = *pr.a, &tmap_b = *pr.b;
        tile_coords(g, local, split, mt, nt);
        const int m0 = mt * TILE_M + (int)rank * GBM;
        const int n0 = nt * BN + (PAIR ? (int)rank * L::B_ROWS : 0);
        const int kb0 = split * g.kb_per_split;
        const int kb1 = min(g.kblocks, kb0 + g.kb_per_split);
        for (int kb = kb0; kb < kb1; kb++) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t fb = PAIR ? map_to_cta(full_bar(stage), 0) : full_bar(stage);
          const uint32_t a_dst = a_base + stage * L::A_BYTES;
          const uint32_t b_dst = b_base + stage * L::B_BYTES;
          const int k0 = kb * GBK;
          if (elect_one()) {
            // the leader's barrier counts the bytes of both CTAs
            if (!PAIR || rank == 0) mbar_expect_tx(full_bar(stage), (PAIR ? 2 : 1) * (L::A_BYTES + L::B_BYTES));
            auto load = [&](uint32_t dst, const CUtensorMap *map, int x, int y) {
              if (PAIR) tma_load_2d_pair(dst, map, fb, x, y); else tma_load_2d(dst, map, fb, x, y);
            };
            if (A_MN) {
#pragma unroll
              for (int i = 0; i < GBM / 64; i++) load(a_dst + i * 8192, &tmap_a, m0 + i * 64, k0);
            } else {
              load(a_dst, &tmap_a, k0, m0);
            }
            if (B_MN) {
#pragma unroll
              for (int i = 0; i < L::B_ROWS / 64; i++) load(b_dst + i * 8192, &tmap_b, n0 + i * 64, k0);
            } else {
              load(b_dst, &tmap_b, k0, n0);
            }
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ── MMA issuer (the leader's, for a pair): warp-uniform loop, one lane issues ─────────
    if (rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TILE_M, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = walker; tile < total_tiles && ok; tile += n_walkers, it++) {
        int split, mt, nt, local;
        const GemmTcArgs &g = *problem_of(tile, local).g;
        tile_coords(g, local, split, mt, nt);
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
          uint64_t adesc[GBK / 16], bdesc[GBK / 16];
#pragma unroll
          for (int k = 0; k < GBK / 16; k++) {
            adesc[k] = A_MN ? make_smem_desc(a_s + k * 2048, 8192, 1024) : make_smem_desc(a_s + k * 32, 16, 1024);
            bdesc[k] = B_MN ? make_smem_desc(b_s + k * 2048, 8192, 1024) : make_smem_desc(b_s + k * 32, 16, 1024);
          }
          const uint32_t first = kb > kb0 ? 1u : 0u;
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < GBK / 16; k++) {
              if (PAIR) mma_bf16_ss_pair(d_tmem, adesc[k], bdesc[k], idesc, k > 0 ? 1u : first);
              else mma_bf16_ss(d_tmem, adesc[k], bdesc[k], idesc, k > 0 ? 1u : first);
            }
            // frees the stage (in both CTAs) once these MMAs have read it
            if (PAIR) mma_commit_pair(empty_bar(stage)); else mma_commit(empty_bar(stage));
            if (kb == kb1 - 1) {  // accumulator complete
              if (PAIR) mma_commit_pair(tfull_bar(acc)); else mma_commit(tfull_bar(acc));
            }
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    // ── epilogue warps (2..5): TMEM -> registers -> global ─────────────────
    const int quad = warp & 3;  // the TMEM lane quadrant this warp may read
    const int ew = warp - 2, half = ew >> 2;  // epilogue warp index; which of the quadrant's two warps (WIDE)
    int it = 0;
    bool ok = true;
    uint8_t *stage = smem + L::STAGE_OFF + ew * (L::EPI_BUFS * 4096);
    const uint32_t stage_u32 = smem_base + L::STAGE_OFF + ew * (L::EPI_BUFS * 4096);
    uint32_t aux_phase = 0, chunk_count = 0;
    if (g.tma_epi && lane == 0) {
      tma_prefetch_desc(p0.c);
      if (g.epilogue != ALPHA_EPI_NONE) tma_prefetch_desc(p0.aux);
    }
    if (GROUP2 && p1.g->tma_epi && lane == 0) {
      tma_prefetch_desc(p1.c);
      if (p1.g->epilogue != ALPHA_EPI_NONE) tma_prefetch_desc(p1.aux);
    }
    auto release_acc = [&](int acc) {  // this warp has read its accumulator rows
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR && rank != 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
        else mbar_arrive(tempty_bar(acc));
      }
    };
    for (int tile = walker; tile < total_tiles && ok; tile += n_walkers, it++) {
      int split, mt, nt, local;
      const GemmProblem &pr = problem_of(tile, local);
      const GemmTcArgs &g = *pr.g;
      const CUtensorMap &tmap_c = *pr.c, &tmap_aux = *pr.aux;
      tile_coords(g, local, split, mt, nt);
      const int m0 = mt * TILE_M + (int)rank * GBM, n0 = nt * BN;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row_in_tile = quad * 32 + lane;
      const int64_t row = (int64_t)m0 + row_in_tile;
      const bool row_ok = row < g.M;
      const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(quad * 32) << 16);
      if (g.tma_epi) {
        const int row0 = m0 + quad * 32 + split * g.m_pad;  // split-K: slab `split` of the workspace
        if (m0 + quad * 32 < g.M) {  // warp-uniform: a quadrant entirely below the matrix has nothing to store
          ok = g.out_f32 ? epilogue_tile_tma<float, BN, WIDE>(g, &tmap_c, &tmap_aux, t_row, row0, n0, lane, stage,
                                                              stage_u32, aux_bar(ew), aux_phase, chunk_count,
                                                              abort_flag, half)
                         : epilogue_tile_tma<__nv_bfloat16, BN, WIDE>(g, &tmap_c, &tmap_aux, t_row, row0, n0, lane, stage,
                                                                      stage_u32, aux_bar(ew), aux_phase, chunk_count,
                                                                      abort_flag, half);
        }
        release_acc(acc);
        continue;
      }
      GemmTcArgs gl = g;
      if (g.splits > 1) gl.C = (float *)g.C + (int64_t)split * g.m_pad * g.N;  // workspace slab, ldc = N
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        const int col0 = n0 + c * 32;
        if (col0 >= g.N) break;  // warp-uniform
        if (WIDE && (c & 1) != half) continue;
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        if (gl.out_f32)
          epilogue_store_chunk<float>(gl, r, row, col0, row_ok);
        else
          epilogue_store_chunk<__nv_bfloat16>(gl, r, row, col0, row_ok);
      }
      release_acc(acc);
    }
    if ((g.tma_epi || (GROUP2 && p1.g->tma_epi)) && lane == 0) bulk_wait<0>();  // all stores have left shared memory and landed
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
  // neither CTA of a pair may leave while the other can still signal its barriers or its
  // tensor memory is still being written by the leader's MMAs
  if (PAIR) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_aux, GemmTcArgs g) {
  const GemmProblem p{&tmap_a, &tmap_b, &tmap_c, &tmap_aux, &g};
  gemm_tc_body<BN, A_MN, B_MN, false, false>(p, p);
}

// Pair form: clusters of two CTAs, one 256 x 256 tile per pair and step.
template <bool A_MN, bool B_MN, bool WIDE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GemmSmemLayout<256, true, WIDE>::THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_aux,
                    GemmTcArgs g) {
  const GemmProblem p{&tmap_a, &tmap_b, &tmap_c, &tmap_aux, &g};
  gemm_tc_body<256, A_MN, B_MN, true, WIDE>(p, p);
}

// Pair form carrying two GEMMs (see GROUP2 above).
struct GemmTmaps {
  CUtensorMap a, b, c, aux;
};
template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GemmSmemLayout<256, true, false>::THREADS, 1)
gemm_tc_pair_group2_kernel(const __grid_constant__ GemmTmaps m0, const __grid_constant__ GemmTmaps m1,
                           const __grid_constant__ GemmTcArgs g0, const __grid_constant__ GemmTcArgs g1) {
  const GemmProblem p0{&m0.a, &m0.b, &m0.c, &m0.aux, &g0}, p1{&m1.a, &m1.b, &m1.c, &m1.aux, &g1};
  gemm_tc_body<256, A_MN, B_MN, true, false, true>(p0, p1);
}

// C (+)= sum_s ws[s]  — split order is fixed, so the result is reproducible.  ws holds
// `splits` dense [m_pad, N] fp32 slabs (`slab` elements apart; only the first M rows of each are
// read); four columns per thread when the rows allow it.
template <typename OutT>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ ws, OutT *C, int64_t M, int64_t N,
                                                            int64_t ldc, int splits, int accumulate, int vec4,
                                                            int64_t slab) {
  const int64_t total = M * N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  grid_dependency_trigger();
  grid_dependency_wait();  // the slabs come from the GEMM launched just before
  if (vec4) {
    const int64_t n4 = total / 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
      float4 s = reinterpret_cast<const float4 *>(ws)[i];
      for (int k = 1; k < splits; k++) {
        const float4 t = reinterpret_cast<const float4 *>(ws + (int64_t)k * slab)[i];
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
    for (int k = 0; k < splits; k++) s += ws[(int64_t)k * slab + i];
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
  using L = GemmSmemLayout<BN, false>;
  static int attr = -1;
  if (attr != g_init_epoch) {
    ALPHA_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN));
    attr = g_init_epoch;
  }
  ALPHA_CUDA(launch_overlapped(OVL_GEMM, gemm_tc_kernel<BN, A_MN, B_MN>, dim3(grid), dim3(GEMM_THREADS), L::DYN, ta, tb, tc_, tx, g));
  ALPHA_LAUNCHED();
  return 0;
}

// Pair form.  `pairs` = tile walkers wanted; the grid is capped at the number of two-CTA
// clusters the device can hold at once (asked from the occupancy API on first use).
template <bool A_MN, bool B_MN, bool WIDE = false>
static int launch_pair_variant(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc_,
                               const CUtensorMap &tx, const GemmTcArgs &g, int pairs) {
  using L = GemmSmemLayout<256, true, WIDE>;
  static int max_pairs = 0, epoch = -1;
  if (epoch != g_init_epoch) {   // function attributes and cluster capacity belong to the device
    epoch = g_init_epoch;
    ALPHA_CUDA(cudaFuncSetAttribute(gemm_tc_pair_kernel<A_MN, B_MN, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN));
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * (g_sm_count / 2));
    cfg.blockDim = dim3(L::THREADS);
    cfg.dynamicSmemBytes = L::DYN;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<A_MN, B_MN, WIDE>, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = g_sm_count / 2;
    }
    max_pairs = n < g_sm_count / 2 ? n : g_sm_count / 2;
  }
  const int n = pairs < max_pairs ? pairs : max_pairs;
  ALPHA_CUDA(launch_overlapped(OVL_GEMM, gemm_tc_pair_kernel<A_MN, B_MN, WIDE>, dim3(2 * n), dim3(L::THREADS), L::DYN, ta, tb,
                               tc_, tx, g));
  ALPHA_LAUNCHED();
  return 0;
}

int gemm_tc_launch(int layout, alpha_buf A, alpha_buf B, alpha_buf C, int64_t M, int64_t N, int64_t K, int64_t lda,
                   int64_t ldb, int64_t ldc, int out_dtype, int epilogue, alpha_buf aux, int64_t ld_aux,
                   int accumulate, float *rowdot = nullptr, int rd_T = 0, int rd_H = 0) {
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
  const bool pair = BN == 256 && M > GBM;  // two CTAs per 256 x 256 tile
  const int tile_m = pair ? 2 * GBM : GBM;
  CUtensorMap ta, tb;
  // A: K-major [M,K] (inner K) or M-major [K,M] (inner M)
  if (a_mn) { if (get_tmap(&ta, ptr<void>(A), M, K, lda, 64, 64)) return 1; }
  else      { if (get_tmap(&ta, ptr<void>(A), K, M, lda, 64, GBM)) return 1; }
  if (b_mn) { if (get_tmap(&tb, ptr<void>(B), N, K, ldb, 64, 64)) return 1; }
  else      { if (get_tmap(&tb, ptr<void>(B), K, N, ldb, 64, pair ? BN / 2 : BN)) return 1; }

  GemmTcArgs g;
  memset(&g, 0, sizeof(g));
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.tiles_m = (int)((M + tile_m - 1) / tile_m);
  g.tiles_n = (int)((N + BN - 1) / BN);
  g.kblocks = (int)((K + GBK - 1) / GBK);
  g.err = tc_error_word();
  const int tiles = g.tiles_m * g.tiles_n;
  // Split-K when the output has too few tiles to fill the device: pick the split count that
  // minimises (waves of tiles) x (K steps per tile + per-tile overhead) + the cost of adding
  // the fp32 partial slabs, all in units of one K step of one tile walker (~0.5 us).
  const int slots = pair ? g_sm_count / 2 : g_sm_count;
  int splits = 1;
  if (epilogue == ALPHA_EPI_NONE && tiles < slots && g.kblocks >= 16) {
    const int max_s = g.kblocks / 8 < 32 ? g.kblocks / 8 : 32;
    double best = 1e30;
    for (int sp = 1; sp <= max_s; sp++) {
      const int waves = (tiles * sp + slots - 1) / slots;
      const int kb = (g.kblocks + sp - 1) / sp;
      double t = (double)waves * (kb + 3);
      if (sp > 1) t += (double)(sp + 1) * (double)M * (double)N * 4.0 / 5.0e12 / 0.5e-6;
      if (t < best) { best = t; splits = sp; }
    }
  }
  g.kb_per_split = (g.kblocks + splits - 1) / splits;
  splits = (g.kblocks + g.kb_per_split - 1) / g.kb_per_split;  // drop empty splits
  g.splits = splits;
  // C += A*B with nothing else in the epilogue is the residual-add epilogue with C as its own
  // addend: the old tile arrives by TMA in the staging buffer the new one leaves from, instead
  // of every lane reading and writing its own row.
  const size_t oes0 = dtype_size(out_dtype);
  if (splits == 1 && accumulate && epilogue == ALPHA_EPI_NONE && (C & 15) == 0 && (ldc * oes0) % 16 == 0) {
    epilogue = ALPHA_EPI_ADD;
    aux = C;
    ld_aux = ldc;
    accumulate = 0;
  }
  void *ws = nullptr;
  g.m_pad = g.tiles_m * tile_m;
  if (splits > 1) {
    // one slab per split, padded to whole tiles so that a tile's rows below the matrix land in
    // the slab's own padding (TMA clips at the tensor's edge, not at a slab's)
    if (pool_alloc((size_t)splits * g.m_pad * N * sizeof(float), &ws)) return 1;
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
  if (epilogue == ALPHA_EPI_ROWDOT) {
    ALPHA_CHECK(g.tma_epi && out_dtype == ALPHA_BF16 && K > 0,
                "alpha_gemm_nn_rowdot: needs bf16 output and 16-byte aligned output and operand rows");
    g.rowdot = rowdot; g.rd_T = rd_T; g.rd_H = rd_H;
  }
  if (splits > 1 && N % 4 == 0) {
    // the partial products leave through shared memory and TMA stores as well (full lines
    // instead of one row per lane); measured on the 3072 x 768 x 16384 weight gradient:
    // 0.0688 -> 0.0631 ms
    if (get_tmap_out(&tcm, ws, ALPHA_F32, N, (uint64_t)splits * g.m_pad, N)) { pool_free(ws); return 1; }
    g.tma_epi = 1;
  }
  const int total = tiles * splits;
  const int grid = total < g_sm_count ? total : g_sm_count;
  int rc;
  if (pair) {
    rc = a_mn ? launch_pair_variant<true, true>(ta, tb, tcm, txm, g, total)
              : (b_mn ? launch_pair_variant<false, true>(ta, tb, tcm, txm, g, total)
                      : ((g.tma_epi && g.epilogue == ALPHA_EPI_GELU)
                             ? launch_pair_variant<false, false, true>(ta, tb, tcm, txm, g, total)
                             : launch_pair_variant<false, false>(ta, tb, tcm, txm, g, total)));
  } else {
#define GEMM_VARIANT(BNV)                                                                               \
  (a_mn ? launch_variant<BNV, true, true>(ta, tb, tcm, txm, g, grid)                                    \
        : (b_mn ? launch_variant<BNV, false, true>(ta, tb, tcm, txm, g, grid)                           \
                : launch_variant<BNV, false, false>(ta, tb, tcm, txm, g, grid)))
  rc = BN == 256 ? GEMM_VARIANT(256) : GEMM_VARIANT(128);
#undef GEMM_VARIANT
  }
  if (rc == 0 && splits > 1) {
    const int vec4 = (N % 4 == 0) ? 1 : 0;   // ws slabs are 512-byte aligned and dense
    const int rgrid = grid_for(M * N / (vec4 ? 4 : 1) + 1, 256, 8);
    cudaError_t e;
    if (out_dtype == ALPHA_F32)
      e = launch_overlapped(OVL_SPLITK, splitk_reduce_kernel<float>, dim3(rgrid), dim3(256), 0, (const float *)ws, ptr<float>(C), M,
                            N, ldc, splits, accumulate, vec4, (int64_t)g.m_pad * N);
    else
      e = launch_overlapped(OVL_SPLITK, splitk_reduce_kernel<__nv_bfloat16>, dim3(rgrid), dim3(256), 0, (const float *)ws,
                            ptr<__nv_bfloat16>(C), M, N, ldc, splits, accumulate, vec4, (int64_t)g.m_pad * N);
    if (e != cudaSuccess) rc = set_error("split-K reduce launch -> %s", cudaGetErrorString(e));
    g_launches++;
  }
  if (ws) pool_free(ws);
  return rc;
}

int gemm_f32_launch(int layout, alpha_buf A, alpha_buf B, alpha_buf C, int64_t M, int64_t N, int64_t K, int64_t lda,
                    int64_t ldb, int64_t ldc, int epilogue, alpha_buf aux, int64_t ld_aux, int accumulate,
                    int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_c);

// Two weight gradients in one launch: C_i (+)= A_i^T B_i with A_i [K, M_i], B_i [K, N_i] bf16 and
// C_i fp32, i = 0, 1, both over the same K.  Alone, each of the step's MLP weight gradients
// (3072 x 768 and 768 x 3072 over K = 16384) has 36 tiles for 74 CTA pairs and has to split K
// in two and add the halves in a second kernel; side by side their 72 tiles fill the device
// unsplit: one launch instead of four and no partial products.  Returns -1 (nothing launched)
// when the pair does not qualify; the caller then runs the two GEMMs on their own.
struct TnProblem {
  alpha_buf A, B, C;
  int64_t M, N, lda, ldb, ldc;
  int accumulate;
};
// `splits` > 1: the problem's K is cut into that many parts whose partial products go to fp32
// slabs in *ws (allocated here, freed by the caller after the reduce kernel is enqueued).
static int prepare_tn_problem(const TnProblem &q, int64_t K, int splits, GemmTcArgs &g, GemmTmaps &m, void **ws) {
  memset(&g, 0, sizeof(g));
  memset(&m, 0, sizeof(m));
  *ws = nullptr;
  const int tile_m = 2 * GBM, BN = 256;
  g.M = (int)q.M; g.N = (int)q.N; g.K = (int)K;
  g.tiles_m = (int)((q.M + tile_m - 1) / tile_m);
  g.tiles_n = (int)((q.N + BN - 1) / BN);
  g.kblocks = (int)((K + GBK - 1) / GBK);
  g.kb_per_split = (g.kblocks + splits - 1) / splits;
  g.splits = (g.kblocks + g.kb_per_split - 1) / g.kb_per_split;
  g.m_pad = g.tiles_m * tile_m;
  g.err = tc_error_word();
  g.out_f32 = 1; g.tma_epi = 1; g.accumulate = 0;
  if (get_tmap(&m.a, ptr<void>(q.A), q.M, K, q.lda, 64, 64)) return 1;
  if (get_tmap(&m.b, ptr<void>(q.B), q.N, K, q.ldb, 64, 64)) return 1;
  if (g.splits > 1) {
    if (pool_alloc((size_t)g.splits * g.m_pad * q.N * sizeof(float), ws)) return 1;
    g.C = *ws; g.ldc = q.N; g.epilogue = ALPHA_EPI_NONE;
    if (get_tmap_out(&m.c, *ws, ALPHA_F32, q.N, (uint64_t)g.splits * g.m_pad, q.N)) return 1;
  } else {
    g.C = ptr<void>(q.C); g.ldc = q.ldc;
    // C += A^T B is the residual-add epilogue with C as its own addend
    g.epilogue = q.accumulate ? ALPHA_EPI_ADD : ALPHA_EPI_NONE;
    g.aux_in = ptr<void>(q.C); g.aux_out = ptr<void>(q.C); g.ld_aux = q.ldc;
    if (get_tmap_out(&m.c, ptr<void>(q.C), ALPHA_F32, q.N, q.M, q.ldc)) return 1;
  }
  m.aux = m.c;
  return 0;
}
static bool tn_problem_qualifies(const TnProblem &q, int64_t K) {
  return q.M > GBM && q.N > 128 && K >= GBK && q.M < (1ll << 31) && q.N < (1ll << 31) && K < (1ll << 31) &&
         (q.A & 15) == 0 && (q.B & 15) == 0 && (q.C & 15) == 0 && (q.lda * 2) % 16 == 0 && (q.ldb * 2) % 16 == 0 &&
         (q.ldc * 4) % 16 == 0;
}
static int gemm_tn_pair_launch(const TnProblem &q0, const TnProblem &q1, int64_t K) {
  if (!tn_problem_qualifies(q0, K) || !tn_problem_qualifies(q1, K)) return -1;
  const int64_t t0 = ((q0.M + 255) / 256) * ((q0.N + 255) / 256), t1 = ((q1.M + 255) / 256) * ((q1.N + 255) / 256);
  const int slots = g_sm_count / 2;
  // worth it when each would split K on its own and together they still fit one wave
  if (t0 + t1 > slots || 2 * t0 > slots + t0 / 2 || 2 * t1 > slots + t1 / 2) return -1;
  // a pair that fills less than half of the device splits K as well (both problems alike),
  // which still halves the launches and lets the two share every wave
  const int kblocks = (int)((K + GBK - 1) / GBK);
  int splits = (int)(slots / (t0 + t1));
  if (splits > kblocks / 16) splits = kblocks / 16;
  if (splits < 1 || q0.N % 4 != 0 || q1.N % 4 != 0) splits = 1;
  GemmTcArgs g0, g1;
  GemmTmaps m0, m1;
  void *ws0 = nullptr, *ws1 = nullptr;
  if (prepare_tn_problem(q0, K, splits, g0, m0, &ws0) || prepare_tn_problem(q1, K, splits, g1, m1, &ws1)) {
    if (ws0) pool_free(ws0);
    if (ws1) pool_free(ws1);
    return 1;
  }
  ProfScope prof(PROF_GEMM_TC, 2.0 * (double)K * ((double)q0.M * (double)q0.N + (double)q1.M * (double)q1.N));
  using L = GemmSmemLayout<256, true, false>;
  static int max_pairs = 0, epoch = -1;
  if (epoch != g_init_epoch) {
    epoch = g_init_epoch;
    ALPHA_CUDA(cudaFuncSetAttribute(gemm_tc_pair_group2_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN));
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * (g_sm_count / 2));
    cfg.blockDim = dim3(L::THREADS);
    cfg.dynamicSmemBytes = L::DYN;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_group2_kernel<true, true>, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = g_sm_count / 2;
    }
    max_pairs = n < g_sm_count / 2 ? n : g_sm_count / 2;
  }
  const int total = (int)(t0 * g0.splits + t1 * g1.splits);
  const int n = total < max_pairs ? total : max_pairs;
  cudaError_t e = launch_overlapped(OVL_GEMM, gemm_tc_pair_group2_kernel<true, true>, dim3(2 * n), dim3(L::THREADS), L::DYN, m0,
                                    m1, g0, g1);
  int rc = 0;
  if (e != cudaSuccess) rc = set_error("alpha_gemm_tn_pair: launch -> %s", cudaGetErrorString(e));
  else g_launches++;
  const TnProblem *qs[2] = {&q0, &q1};
  const GemmTcArgs *gs[2] = {&g0, &g1};
  void *wss[2] = {ws0, ws1};
  for (int i = 0; i < 2 && rc == 0; i++) {
    if (gs[i]->splits <= 1) continue;
    const int rgrid = grid_for(qs[i]->M * qs[i]->N / 4 + 1, 256, 8);
    e = launch_overlapped(OVL_SPLITK, splitk_reduce_kernel<float>, dim3(rgrid), dim3(256), 0, (const float *)wss[i],
                          ptr<float>(qs[i]->C), qs[i]->M, qs[i]->N, qs[i]->ldc, gs[i]->splits, qs[i]->accumulate, 1,
                          (int64_t)gs[i]->m_pad * qs[i]->N);
    if (e != cudaSuccess) rc = set_error("alpha_gemm_tn_pair: reduce launch -> %s", cudaGetErrorString(e));
    else g_launches++;
  }
  if (ws0) pool_free(ws0);
  if (ws1) pool_free(ws1);
  return rc;
}

}  // namespace alpha

using namespace alpha;

extern "C" int alpha_gemm_tn_pair(alpha_buf A0, alpha_buf B0, alpha_buf C0, int64_t M0, int64_t N0, int64_t lda0,
                                  int64_t ldb0, int64_t ldc0, int accumulate0, alpha_buf A1, alpha_buf B1, alpha_buf C1,
                                  int64_t M1, int64_t N1, int64_t lda1, int64_t ldb1, int64_t ldc1, int accumulate1,
                                  int64_t K) {
  ALPHA_REQUIRE_INIT();
  const TnProblem q0{A0, B0, C0, M0, N0, lda0, ldb0, ldc0, accumulate0}, q1{A1, B1, C1, M1, N1, lda1, ldb1, ldc1, accumulate1};
  const int rc = gemm_tn_pair_launch(q0, q1, K);
  if (rc >= 0) return rc;
  // not a pair that gains from sharing a launch: one GEMM each
  if (gemm_tc_launch(ALPHA_GEMM_TN, A0, B0, C0, M0, N0, K, lda0, ldb0, ldc0, ALPHA_F32, ALPHA_EPI_NONE, 0, 0, accumulate0))
    return 1;
  return gemm_tc_launch(ALPHA_GEMM_TN, A1, B1, C1, M1, N1, K, lda1, ldb1, ldc1, ALPHA_F32, ALPHA_EPI_NONE, 0, 0, accumulate1);
}


// dO = G W with the row-dot of attention's backward in the epilogue: besides C = A B (NN,
// bf16, N = heads * 64) it writes delta[b, h, t] = sum_d C[b*T + t, 64h + d] * O[b*T + t, 64h + d]
// (C as rounded to bf16), which alpha_flash_attn_bwd_delta then takes instead of computing it
// from O and dO in a pass of its own.
extern "C" int alpha_gemm_nn_rowdot(alpha_buf A, alpha_buf B, alpha_buf C, int64_t M, int64_t N, int64_t K, int64_t lda,
                                    int64_t ldb, int64_t ldc, alpha_buf O, int64_t ld_o, alpha_buf delta, int64_t T,
                                    int64_t heads) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(heads > 0 && N == heads * 64, "alpha_gemm_nn_rowdot: N = %lld is not heads * 64", (long long)N);
  ALPHA_CHECK(T > 0 && M % T == 0, "alpha_gemm_nn_rowdot: M = %lld is not a multiple of T = %lld", (long long)M, (long long)T);
  ALPHA_CHECK(O != 0 && delta != 0, "alpha_gemm_nn_rowdot: null operand");
  return gemm_tc_launch(ALPHA_GEMM_NN, A, B, C, M, N, K, lda, ldb, ldc, ALPHA_BF16, ALPHA_EPI_ROWDOT, O, ld_o, 0,
                        ptr<float>(delta), (int)T, (int)heads);
}

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
