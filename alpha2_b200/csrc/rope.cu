// Rotary position embedding on the q/k slices of the fused QKV activation.
// No reference counterpart (the reference has learned positions only,
// packages/model/src/gpt.ts:362-379); asked for by the 350M configuration.
// Rotate-half convention: for head dim D and pair index i < D/2,
//   out[i]       = x[i]*cos(t*w_i) - x[i+D/2]*sin(t*w_i)
//   out[i+D/2]   = x[i+D/2]*cos(t*w_i) + x[i]*sin(t*w_i),   w_i = theta^(-2i/D).
// The backward is the transposed rotation (sin negated).  HBM-bound: one read and one
// write per element.  The vectorised kernel reads cos/sin from a [T, D/2] table built once
// per (T, D, theta) on the host in double precision (it stays in L2) and moves 16 bytes per
// access; alpha_rope_qkv rotates q and k and copies v in the same pass, so a fused
// [rows, 3E] activation is produced out of place with one read and one write of each row.
// Odd layouts fall back to the scalar kernel, which computes its angles with sincosf.
#include <cmath>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace alpha {

template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const T *x, T *out, int64_t rows, int T_len, int heads, int D,
                                                   int64_t ld_x, int64_t ld_out, float log_theta, float sign) {
  const int half = D / 2;
  const int64_t total = rows * heads * half;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int i = (int)(e % half);
    const int64_t rh = e / half;
    const int h = (int)(rh % heads);
    const int64_t r = rh / heads;
    const int t = (int)(r % T_len);
    const float w = expf(-log_theta * (2.f * i) / D);
    float sn, cs;
    sincosf(t * w, &sn, &cs);
    sn *= sign;
    const int64_t src = r * ld_x + (int64_t)h * D + i, dst = r * ld_out + (int64_t)h * D + i;
    const float a = to_f32(x[src]), b = to_f32(x[src + half]);
    out[dst] = from_f32<T>(a * cs - b * sn);
    out[dst + half] = from_f32<T>(b * cs + a * sn);
  }
}

// One thread per pair of 16-byte chunks (x[i..i+V) and x[i+D/2..i+D/2+V)) of a rotated head, or
// per 16-byte chunk of the copied tail [rot_cols, copy_cols) of the row.
template <typename T>
__global__ void __launch_bounds__(256) rope_vec_kernel(const T *x, T *out, int64_t rows,
                                                       int T_len, int heads, int D, int64_t ld_x, int64_t ld_out,
                                                       int copy_cols, const float2 *__restrict__ table, float sign) {
  constexpr int V = Vec16<T>::N;
  const int half = D / 2, upr_rot = heads * (half / V), rot_cols = heads * D;
  const int upr = upr_rot + (copy_cols - rot_cols) / V;
  const int64_t total = rows * upr;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t r = e / upr;
    const int u = (int)(e - r * upr);
    if (u >= upr_rot) {
      const int c = rot_cols + (u - upr_rot) * V;
      Vec16<T> t;
      t.load(x + r * ld_x + c);
      t.store(out + r * ld_out + c);
      continue;
    }
    const int h = u / (half / V), i = (u % (half / V)) * V;
    const int t_pos = (int)(r % T_len);
    const T *src = x + r * ld_x + (int64_t)h * D + i;
    T *dst = out + r * ld_out + (int64_t)h * D + i;
    Vec16<T> va, vb;
    va.load(src);
    vb.load(src + half);
    float a[V], b[V], oa[V], ob[V];
    va.get(a);
    vb.get(b);
    const float4 *cs = reinterpret_cast<const float4 *>(table + (int64_t)t_pos * half + i);
#pragma unroll
    for (int j = 0; j < V; j += 2) {
      const float4 t2 = cs[j / 2];  // {cos_j, sin_j, cos_j+1, sin_j+1}
      const float s0 = t2.y * sign, s1 = t2.w * sign;
      oa[j] = a[j] * t2.x - b[j] * s0;
      ob[j] = b[j] * t2.x + a[j] * s0;
      oa[j + 1] = a[j + 1] * t2.z - b[j + 1] * s1;
      ob[j + 1] = b[j + 1] * t2.z + a[j + 1] * s1;
    }
    va.set(oa);
    vb.set(ob);
    va.store(dst);
    vb.store(dst + half);
  }
}

// cos/sin tables, one per (T, D, theta), kept on the device until shutdown.
struct RopeTable {
  int64_t T, D;
  float theta;
  float2 *dev;
};
static std::vector<RopeTable> g_rope_tables;
static std::mutex g_rope_mu;

void rope_tables_clear() {
  std::lock_guard<std::mutex> lk(g_rope_mu);
  for (auto &t : g_rope_tables) cudaFree(t.dev);
  g_rope_tables.clear();
}

static int rope_table(int64_t T, int64_t D, float theta, const float2 **out) {
  std::lock_guard<std::mutex> lk(g_rope_mu);
  for (auto &t : g_rope_tables)
    if (t.T == T && t.D == D && t.theta == theta) {
      *out = t.dev;
      return 0;
    }
  const int64_t half = D / 2;
  std::vector<float2> host((size_t)(T * half));
  for (int64_t i = 0; i < half; i++) {
    const double w = std::exp(-std::log((double)theta) * (2.0 * (double)i) / (double)D);
    for (int64_t t = 0; t < T; t++) {
      const double ang = (double)t * w;
      host[(size_t)(t * half + i)] = make_float2((float)std::cos(ang), (float)std::sin(ang));
    }
  }
  float2 *dev = nullptr;
  ALPHA_CUDA(cudaMalloc(&dev, host.size() * sizeof(float2)));
  // pageable source: the copy has left the host buffer when the call returns
  cudaError_t e = cudaMemcpyAsync(dev, host.data(), host.size() * sizeof(float2), cudaMemcpyHostToDevice, g_stream);
  if (e != cudaSuccess) {
    cudaFree(dev);
    return set_error("rope table upload: %s", cudaGetErrorString(e));
  }
  g_rope_tables.push_back({T, D, theta, dev});
  *out = dev;
  return 0;
}

// x and out: [rows, *] with row strides ld_x / ld_out; columns [0, heads*D) are rotated and
// [heads*D, copy_cols) copied (copy_cols == heads*D: nothing copied).
static int rope_launch(alpha_buf x, alpha_buf out, int64_t batch, int64_t T, int64_t heads, int64_t D, int64_t ld_x,
                       int64_t ld_out, int64_t copy_cols, float theta, int inverse, int dtype, const char *who) {
  ALPHA_CHECK(D % 2 == 0, "%s: odd head dim", who);
  ALPHA_CHECK(dtype == ALPHA_F32 || dtype == ALPHA_BF16, "%s: unsupported dtype %d", who, dtype);
  const int64_t rows = batch * T, total = rows * heads * (D / 2);
  if (rows == 0 || (total == 0 && copy_cols == 0)) return 0;
  const float sign = inverse ? -1.f : 1.f;
  const int64_t es = (int64_t)dtype_size(dtype), V = 16 / es, half = D / 2;
  ProfScope prof(PROF_ELEMENTWISE, 2.0 * rows * copy_cols);
  const bool vec = half % V == 0 && (x & 15) == 0 && (out & 15) == 0 && (ld_x * es) % 16 == 0 &&
                   (ld_out * es) % 16 == 0 && (copy_cols - heads * D) % V == 0 && heads * D < (1ll << 30) &&
                   copy_cols < (1ll << 30);
  if (vec) {
    const float2 *table = nullptr;
    if (rope_table(T, D, theta, &table)) return 1;
    const int64_t units = rows * (heads * (half / V) + (copy_cols - heads * D) / V);
    if (dtype == ALPHA_F32)
      rope_vec_kernel<float><<<grid_for(units, 256, 8), 256, 0, g_stream>>>(
          ptr<float>(x), ptr<float>(out), rows, (int)T, (int)heads, (int)D, ld_x, ld_out, (int)copy_cols, table, sign);
    else
      rope_vec_kernel<__nv_bfloat16><<<grid_for(units, 256, 8), 256, 0, g_stream>>>(
          ptr<__nv_bfloat16>(x), ptr<__nv_bfloat16>(out), rows, (int)T, (int)heads, (int)D, ld_x, ld_out,
          (int)copy_cols, table, sign);
    ALPHA_LAUNCHED();
    return 0;
  }
  const float lt = logf(theta);
  if (total > 0) {
    if (dtype == ALPHA_F32)
      rope_kernel<float><<<grid_for(total, 256, 16), 256, 0, g_stream>>>(ptr<float>(x), ptr<float>(out), rows, (int)T,
                                                                         (int)heads, (int)D, ld_x, ld_out, lt, sign);
    else
      rope_kernel<__nv_bfloat16><<<grid_for(total, 256, 16), 256, 0, g_stream>>>(
          ptr<__nv_bfloat16>(x), ptr<__nv_bfloat16>(out), rows, (int)T, (int)heads, (int)D, ld_x, ld_out, lt, sign);
    ALPHA_LAUNCHED();
  }
  if (copy_cols > heads * D && x != out)  // the tail columns, row by row
    ALPHA_CUDA(cudaMemcpy2DAsync(ptr<char>(out) + heads * D * es, (size_t)(ld_out * es),
                                 ptr<char>(x) + heads * D * es, (size_t)(ld_x * es),
                                 (size_t)((copy_cols - heads * D) * es), (size_t)rows, cudaMemcpyDeviceToDevice,
                                 g_stream));
  return 0;
}

}  // namespace alpha

using namespace alpha;

extern "C" {

int alpha_rope(alpha_buf x, alpha_buf out, int64_t batch, int64_t T, int64_t heads, int64_t D, int64_t ld, float theta,
               int inverse, int dtype) {
  ALPHA_REQUIRE_INIT();
  return rope_launch(x, out, batch, T, heads, D, ld, ld, heads * D, theta, inverse, dtype, "alpha_rope");
}

int alpha_rope_qkv(alpha_buf qkv, alpha_buf out, int64_t batch, int64_t T, int64_t heads, int64_t D, float theta,
                   int inverse, int dtype) {
  ALPHA_REQUIRE_INIT();
  const int64_t E = heads * D;
  // q and k are 2*heads rotated heads side by side; v is the copied tail
  return rope_launch(qkv, out, batch, T, 2 * heads, D, 3 * E, 3 * E, 3 * E, theta, inverse, dtype, "alpha_rope_qkv");
}

}  // extern "C"
