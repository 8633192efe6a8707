// fp32 GEMM on the FMA pipes: the full-precision mode used by the fp32 parity
// configurations (the reference accumulates each dot product in a double and rounds once,
// packages/tensor/src/cpu_ref.ts:246-254; bf16 tensor-core products cannot meet a 1e-4
// parameter tolerance, fp32 FMA accumulation does).  Arbitrary element strides cover the
// three layouts of the Backend interface — A*B, A*B^T (matmulTransposed) and A^T*B
// (matmulTransposedA), packages/core/src/interfaces.ts:53,111-112 — and batched matmul
// with broadcastable batch strides for the unfused attention branch
// (packages/model/src/gpt.ts:256-279).
//
// 64x64x16 shared-memory tiles, 256 threads, 4x4 outputs per thread.
#include "common.cuh"

namespace alpha {

struct GemmF32Args {
  const float *A, *B;
  float *C;
  const float *aux_in;  // ADD: residual; GELU_BWD: saved pre-activation
  float *aux_out;       // GELU: receives the pre-activation
  int64_t M, N, K;
  int64_t sam, sak, sbk, sbn, ldc, ld_aux;
  int64_t batch_a, batch_b, batch_c;
  int epilogue, accumulate;
};

constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256) gemm_f32_kernel(GemmF32Args g) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN;
  const float *A = g.A + (int64_t)blockIdx.z * g.batch_a;
  const float *B = g.B + (int64_t)blockIdx.z * g.batch_b;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  // Loader mapping: prefer the contiguous direction of each operand for coalescing.
  const bool a_k_contig = g.sak == 1;
  const bool b_n_contig = g.sbn == 1;
  for (int64_t k0 = 0; k0 < g.K; k0 += TK) {
#pragma unroll
    for (int it = 0; it < (TM * TK) / 256; it++) {
      const int e = tid + it * 256;
      int mm, kk;
      if (a_k_contig) { kk = e % TK; mm = e / TK; } else { mm = e % TM; kk = e / TM; }
      const int64_t m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < g.M && k < g.K) ? A[m * g.sam + k * g.sak] : 0.f;
    }
#pragma unroll
    for (int it = 0; it < (TN * TK) / 256; it++) {
      const int e = tid + it * 256;
      int nn, kk;
      if (b_n_contig) { nn = e % TN; kk = e / TN; } else { kk = e % TK; nn = e / TK; }
      const int64_t n = n0 + nn, k = k0 + kk;
      Bs[kk][nn] = (n < g.N && k < g.K) ? B[k * g.sbk + n * g.sbn] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk++) {
      const float4 a4 = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w};
      const float b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

  float *C = g.C + (int64_t)blockIdx.z * g.batch_c;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int64_t n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      float v = acc[i][j];
      switch (g.epilogue) {
        case ALPHA_EPI_GELU:
          g.aux_out[m * g.ld_aux + n] = v;
          v = gelu_f(v);
          break;
        case ALPHA_EPI_ADD:
          v += g.aux_in[m * g.ld_aux + n];
          break;
        case ALPHA_EPI_GELU_BWD:
          v *= gelu_grad_f(g.aux_in[m * g.ld_aux + n]);
          break;
        default:
          break;
      }
      float *dst = C + m * g.ldc + n;
      *dst = g.accumulate ? *dst + v : v;
    }
  }
}

int gemm_f32_launch(int layout, alpha_buf A, alpha_buf B, alpha_buf C, int64_t M, int64_t N, int64_t K, int64_t lda,
                    int64_t ldb, int64_t ldc, int epilogue, alpha_buf aux, int64_t ld_aux, int accumulate,
                    int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_c) {
  if (M == 0 || N == 0 || batch == 0) return 0;
  ProfScope prof(PROF_GEMM_F32, 2.0 * (double)M * (double)N * (double)K * (double)batch);
  GemmF32Args g;
  g.A = ptr<float>(A);
  g.B = ptr<float>(B);
  g.C = ptr<float>(C);
  g.aux_in = ptr<float>(aux);
  g.aux_out = ptr<float>(aux);
  g.M = M; g.N = N; g.K = K;
  g.ldc = ldc; g.ld_aux = ld_aux;
  g.batch_a = stride_a; g.batch_b = stride_b; g.batch_c = stride_c;
  g.epilogue = epilogue; g.accumulate = accumulate;
  switch (layout) {
    case ALPHA_GEMM_NT: g.sam = lda; g.sak = 1; g.sbk = 1; g.sbn = ldb; break;   // B stored [N,K]
    case ALPHA_GEMM_NN: g.sam = lda; g.sak = 1; g.sbk = ldb; g.sbn = 1; break;   // B stored [K,N]
    case ALPHA_GEMM_TN: g.sam = 1; g.sak = lda; g.sbk = ldb; g.sbn = 1; break;   // A stored [K,M]
    default: return set_error("alpha_gemm: bad layout %d", layout);
  }
  ALPHA_CHECK(batch <= 65535, "alpha_gemm: batch %lld > 65535", (long long)batch);
  ALPHA_CHECK((M + TM - 1) / TM <= 65535, "alpha_gemm: M too large for the fp32 kernel");
  dim3 grid((unsigned)((N + TN - 1) / TN), (unsigned)((M + TM - 1) / TM), (unsigned)batch);
  gemm_f32_kernel<<<grid, 256, 0, g_stream>>>(g);
  ALPHA_LAUNCHED();
  return 0;
}

}  // namespace alpha

using namespace alpha;

extern "C" int alpha_gemm_batched_f32(int layout, alpha_buf A, alpha_buf B, alpha_buf C, int64_t M, int64_t N,
                                      int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t batch,
                                      int64_t stride_a, int64_t stride_b, int64_t stride_c) {
  ALPHA_REQUIRE_INIT();
  return gemm_f32_launch(layout, A, B, C, M, N, K, lda, ldb, ldc, ALPHA_EPI_NONE, 0, 0, 0, batch, stride_a, stride_b,
                         stride_c);
}
