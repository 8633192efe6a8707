// Rotary position embedding on the q/k slices of the fused QKV activation.
// No reference counterpart (the reference has learned positions only,
// packages/model/src/gpt.ts:362-379); asked for by the 350M configuration.
// Rotate-half convention: for head dim D and pair index i < D/2,
//   out[i]       = x[i]*cos(t*w_i) - x[i+D/2]*sin(t*w_i)
//   out[i+D/2]   = x[i+D/2]*cos(t*w_i) + x[i]*sin(t*w_i),   w_i = theta^(-2i/D).
// The backward is the transposed rotation (sin negated).  HBM-bound: one read and one
// write per element; angles are computed in fp32 with sincosf (t <= 2048 here).
#include "common.cuh"

namespace alpha {

template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const T *x, T *out, int64_t rows, int T_len, int heads, int D,
                                                   int64_t ld, float log_theta, float sign) {
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
    const int64_t base = r * ld + (int64_t)h * D + i;
    const float a = to_f32(x[base]), b = to_f32(x[base + half]);
    out[base] = from_f32<T>(a * cs - b * sn);
    out[base + half] = from_f32<T>(b * cs + a * sn);
  }
}

}  // namespace alpha

using namespace alpha;

extern "C" int alpha_rope(alpha_buf x, alpha_buf out, int64_t batch, int64_t T, int64_t heads, int64_t D, int64_t ld,
                          float theta, int inverse, int dtype) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(D % 2 == 0, "alpha_rope: odd head dim");
  const int64_t rows = batch * T, total = rows * heads * (D / 2);
  if (total == 0) return 0;
  const float lt = logf(theta), sign = inverse ? -1.f : 1.f;
  if (dtype == ALPHA_F32)
    rope_kernel<float><<<grid_for(total, 256, 16), 256, 0, g_stream>>>(ptr<float>(x), ptr<float>(out), rows, (int)T,
                                                                       (int)heads, (int)D, ld, lt, sign);
  else if (dtype == ALPHA_BF16)
    rope_kernel<__nv_bfloat16><<<grid_for(total, 256, 16), 256, 0, g_stream>>>(
        ptr<__nv_bfloat16>(x), ptr<__nv_bfloat16>(out), rows, (int)T, (int)heads, (int)D, ld, lt, sign);
  else
    return set_error("alpha_rope: unsupported dtype %d", dtype);
  ALPHA_LAUNCHED();
  return 0;
}
