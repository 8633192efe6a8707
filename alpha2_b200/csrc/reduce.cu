// Reductions: axis sums, row softmax / log-softmax, the multi-tensor sum of squares that
// feeds the global gradient norm, and the non-finite check.
//
// Reference semantics: packages/tensor/src/cpu_ref.ts:260-333 (sum/mean), :439-541
// (softmax/logSoftmax with max subtraction); packages/train/src/trainer.ts:1314-1375 (the
// gradient norm is sqrt(sum over tensors of sum(g^2)) * |gradScale|; the reference issues
// one reduction per tensor plus a tree of scalar adds, ~100 launches — here it is one
// launch over a pointer table plus one finishing launch, deterministic: fixed block
// partition, fixed-order final add).
#include <vector>

#include "common.cuh"

namespace alpha {

// a viewed [outer, dim, inner] -> out [outer, inner]; one thread per output when inner > 1
// (coalesced across inner), one block per output row when inner == 1.
template <typename T>
__global__ void __launch_bounds__(256) sum_axis_strided(const T *a, T *out, int64_t outer, int64_t dim, int64_t inner,
                                                        float scale) {
  const int64_t total = outer * inner;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t o = i / inner, in = i - o * inner;
    const T *p = a + o * dim * inner + in;
    float s = 0.f;
    for (int64_t d = 0; d < dim; d++) s += to_f32(p[d * inner]);
    out[i] = from_f32<T>(s * scale);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) sum_axis_rows(const T *a, T *out, int64_t outer, int64_t dim, float scale) {
  __shared__ float red[32];
  for (int64_t o = blockIdx.x; o < outer; o += gridDim.x) {
    const T *p = a + o * dim;
    float s = 0.f;
    for (int64_t d = threadIdx.x; d < dim; d += blockDim.x) s += to_f32(p[d]);
    s = block_sum(s, red);
    if (threadIdx.x == 0) out[o] = from_f32<T>(s * scale);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) softmax_rows(const T *a, T *out, int64_t rows, int64_t cols, int log_mode) {
  __shared__ float red[32];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T *p = a + r * cols;
    float mx = -INFINITY;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) mx = fmaxf(mx, to_f32(p[c]));
    mx = block_max(mx, red);
    float s = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += expf(to_f32(p[c]) - mx);
    s = block_sum(s, red);
    if (log_mode) {
      const float lse = mx + logf(s);
      for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) out[r * cols + c] = from_f32<T>(to_f32(p[c]) - lse);
    } else {
      const float inv = 1.f / s;
      for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
        out[r * cols + c] = from_f32<T>(expf(to_f32(p[c]) - mx) * inv);
    }
  }
}

// ── multi-tensor sum of squares ─────────────────────────────────────────────
// The tensors are cut into chunks of SUMSQ_CHUNK elements; block b reduces chunk b of the
// table and writes partial[b]; a single block then adds the partials in index order.
constexpr int64_t SUMSQ_CHUNK = 1 << 16;

struct SumsqChunk {
  const void *base;
  int32_t count;
  int32_t dtype;
};

__global__ void __launch_bounds__(256) sumsq_chunks_kernel(const SumsqChunk *__restrict__ chunks,
                                                           float *__restrict__ partial, int mode) {
  __shared__ float red[32];
  const SumsqChunk ch = chunks[blockIdx.x];
  float s = 0.f;
  if (ch.dtype == ALPHA_F32) {
    const float *p = (const float *)ch.base;
    const int n4 = aligned16(p) ? ch.count / 4 : 0;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 v = reinterpret_cast<const float4 *>(p)[i];
      if (mode == 0) s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      else s += (float)(!isfinite(v.x)) + (float)(!isfinite(v.y)) + (float)(!isfinite(v.z)) + (float)(!isfinite(v.w));
    }
    for (int i = n4 * 4 + threadIdx.x; i < ch.count; i += blockDim.x)
      s += mode == 0 ? p[i] * p[i] : (float)(!isfinite(p[i]));
  } else {
    const __nv_bfloat16 *p = (const __nv_bfloat16 *)ch.base;
    const int n8 = aligned16(p) ? ch.count / 8 : 0;
    for (int i = threadIdx.x; i < n8; i += blockDim.x) {
      Vec16<__nv_bfloat16> v;
      v.load(p + i * 8);
      float f[8];
      v.get(f);
#pragma unroll
      for (int j = 0; j < 8; j++) s += mode == 0 ? f[j] * f[j] : (float)(!isfinite(f[j]));
    }
    for (int i = n8 * 8 + threadIdx.x; i < ch.count; i += blockDim.x) {
      const float f = to_f32(p[i]);
      s += mode == 0 ? f * f : (float)(!isfinite(f));
    }
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__global__ void __launch_bounds__(1024) sum_partials_kernel(const float *__restrict__ partial, int n,
                                                            float *__restrict__ out) {
  // fixed order: thread t adds partial[t], partial[t+1024], ... then a fixed-shape tree
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = s;
}

static int reduce_table(const alpha_buf *tensors, const int64_t *counts, const int32_t *dtypes, int n_tensors,
                        alpha_buf out_scalar, int mode) {
  std::vector<SumsqChunk> table;
  for (int t = 0; t < n_tensors; t++) {
    const size_t es = dtype_size(dtypes[t]);
    if (dtypes[t] != ALPHA_F32 && dtypes[t] != ALPHA_BF16) return set_error("sumsq: unsupported dtype %d", dtypes[t]);
    for (int64_t off = 0; off < counts[t]; off += SUMSQ_CHUNK) {
      const int64_t c = counts[t] - off < SUMSQ_CHUNK ? counts[t] - off : SUMSQ_CHUNK;
      table.push_back({(const void *)(uintptr_t)(tensors[t] + off * es), (int32_t)c, dtypes[t]});
    }
  }
  if (table.empty()) {
    ALPHA_CUDA(cudaMemsetAsync(ptr<void>(out_scalar), 0, 4, g_stream));
    return 0;
  }
  const void *dev_table = nullptr;
  if (table_upload(table.data(), table.size() * sizeof(SumsqChunk), &dev_table)) return 1;
  void *scratch = nullptr;
  if (pool_alloc(table.size() * sizeof(float), &scratch)) return 1;
  float *partial = (float *)scratch;
  sumsq_chunks_kernel<<<(unsigned)table.size(), 256, 0, g_stream>>>((const SumsqChunk *)dev_table, partial, mode);
  g_launches++;
  sum_partials_kernel<<<1, 1024, 0, g_stream>>>(partial, (int)table.size(), ptr<float>(out_scalar));
  pool_free(scratch);
  ALPHA_LAUNCHED();
  return 0;
}

}  // namespace alpha

using namespace alpha;

extern "C" {

int alpha_sum_axis(alpha_buf a, alpha_buf out, int64_t outer, int64_t dim, int64_t inner, float scale, int dtype) {
  ALPHA_REQUIRE_INIT();
  if (outer * inner == 0) return 0;
#define SUM_AXIS(T)                                                                                          \
  if (inner == 1)                                                                                            \
    sum_axis_rows<T><<<grid_for(outer, 1, 8), 256, 0, g_stream>>>(ptr<T>(a), ptr<T>(out), outer, dim, scale); \
  else                                                                                                       \
    sum_axis_strided<T><<<grid_for(outer * inner, 256, 8), 256, 0, g_stream>>>(ptr<T>(a), ptr<T>(out), outer, dim, inner, scale);
  if (dtype == ALPHA_F32) { SUM_AXIS(float) }
  else if (dtype == ALPHA_BF16) { SUM_AXIS(__nv_bfloat16) }
  else return set_error("alpha_sum_axis: unsupported dtype %d", dtype);
#undef SUM_AXIS
  ALPHA_LAUNCHED();
  return 0;
}

int alpha_softmax(alpha_buf a, alpha_buf out, int64_t rows, int64_t cols, int log_mode, int dtype) {
  ALPHA_REQUIRE_INIT();
  if (rows * cols == 0) return 0;
  const int grid = grid_for(rows, 1, 8);
  if (dtype == ALPHA_F32)
    softmax_rows<float><<<grid, 256, 0, g_stream>>>(ptr<float>(a), ptr<float>(out), rows, cols, log_mode);
  else if (dtype == ALPHA_BF16)
    softmax_rows<__nv_bfloat16><<<grid, 256, 0, g_stream>>>(ptr<__nv_bfloat16>(a), ptr<__nv_bfloat16>(out), rows, cols,
                                                            log_mode);
  else
    return set_error("alpha_softmax: unsupported dtype %d", dtype);
  ALPHA_LAUNCHED();
  return 0;
}

int alpha_sumsq_multi(const alpha_buf *tensors, const int64_t *counts, const int32_t *dtypes, int n_tensors,
                      alpha_buf out_scalar) {
  ALPHA_REQUIRE_INIT();
  double n = 0;
  for (int t = 0; t < n_tensors; t++) n += (double)counts[t];
  ProfScope prof(PROF_ELEMENTWISE, n);
  return reduce_table(tensors, counts, dtypes, n_tensors, out_scalar, 0);
}

int alpha_check_finite(alpha_buf a, int64_t n, int dtype, alpha_buf out_scalar) {
  ALPHA_REQUIRE_INIT();
  const int32_t dt = dtype;
  return reduce_table(&a, &n, &dt, 1, out_scalar, 1);
}

}  // extern "C"
