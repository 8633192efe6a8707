// Fused AdamW, single tensor and multi-tensor.  HBM-bound: per parameter it reads p, g, m, v
// and writes p, m, v (+ a bf16 shadow of p): 28 bytes with bf16 gradients, 30 with f32
// gradients and a shadow, 28 with f32 gradients and no shadow.
//
// Reference semantics: packages/train/src/optimizers.ts:84-92
//   g = grad*gradScale; if wd > 0: p -= lr*wd*p; m = b1*m + (1-b1)*g; v = b2*v + (1-b2)*g*g;
//   p -= lr*(m/bc1)/(sqrt(v/bc2)+eps)
// with bc1 = 1-b1^t, bc2 = 1-b2^t (:107-115).  The reference launches one kernel per tensor
// (~100 per step, packages/helios/src/backend.ts:5374-5434); the multi-tensor entry makes
// it one launch over a chunk table.  The clip coefficient can be taken from a device
// scalar (sum of squared gradients) so that nothing is read back between the norm and the
// update (packages/train/src/trainer.ts:1650-1656 computes it on the host).
#include <string.h>

#include <vector>

#include "common.cuh"

namespace alpha {

struct AdamHyper {
  float lr, beta1, beta2, eps, bc1, bc2, grad_scale, max_norm;
  const float *clip_sumsq;
};

// Gradient scale with the clip coefficient folded in.  `*skip` is set when the norm is not
// finite: the caller must then leave p, m, v and the shadow exactly as they are (the
// reference does not call the optimizer at all for such a step, trainer.ts:1495-1527,1750;
// scaling the gradient by zero would not do, 0 * Inf is NaN and decay would still apply).
__device__ __forceinline__ float effective_scale(const AdamHyper &h, bool *skip) {
  float gs = h.grad_scale;
  *skip = false;
  if (h.clip_sumsq) {
    const float gnorm = sqrtf(h.clip_sumsq[0]) * fabsf(h.grad_scale);
    if (h.max_norm > 0.f && gnorm > h.max_norm) gs *= h.max_norm / gnorm;
    if (!isfinite(gnorm)) *skip = true;
  }
  return gs;
}

__device__ __forceinline__ void adam_one(float &p, float g, float &m, float &v, const AdamHyper &h, float gs,
                                         float wd) {
  g *= gs;
  if (wd > 0.f) p -= h.lr * wd * p;
  m = h.beta1 * m + (1.f - h.beta1) * g;
  v = h.beta2 * v + (1.f - h.beta2) * g * g;
  const float mhat = m / h.bc1, vhat = v / h.bc2;
  p -= h.lr * mhat / (sqrtf(vhat) + h.eps);
}

template <typename G>
__device__ __forceinline__ void adam_span(float *p, const G *g, float *m, float *v, __nv_bfloat16 *shadow, int64_t n,
                                          const AdamHyper &h, float gs, float wd, int64_t tid, int64_t nthreads) {
  const bool vec = aligned16(p) && aligned16(m) && aligned16(v) &&
                   ((reinterpret_cast<uintptr_t>(g) & (sizeof(G) * 4 - 1)) == 0) &&
                   (!shadow || (reinterpret_cast<uintptr_t>(shadow) & 7) == 0);
  const int64_t n4 = vec ? n / 4 : 0;
  for (int64_t i = tid; i < n4; i += nthreads) {
    float4 pv = reinterpret_cast<float4 *>(p)[i];
    float4 mv = reinterpret_cast<float4 *>(m)[i];
    float4 vv = reinterpret_cast<float4 *>(v)[i];
    float gv[4];
    if (sizeof(G) == 4) {
      const float4 t = reinterpret_cast<const float4 *>(g)[i];
      gv[0] = t.x; gv[1] = t.y; gv[2] = t.z; gv[3] = t.w;
    } else {
      const uint2 t = reinterpret_cast<const uint2 *>(g)[i];
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&t.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&t.y));
      gv[0] = a.x; gv[1] = a.y; gv[2] = b.x; gv[3] = b.y;
    }
    adam_one(pv.x, gv[0], mv.x, vv.x, h, gs, wd);
    adam_one(pv.y, gv[1], mv.y, vv.y, h, gs, wd);
    adam_one(pv.z, gv[2], mv.z, vv.z, h, gs, wd);
    adam_one(pv.w, gv[3], mv.w, vv.w, h, gs, wd);
    reinterpret_cast<float4 *>(p)[i] = pv;
    reinterpret_cast<float4 *>(m)[i] = mv;
    reinterpret_cast<float4 *>(v)[i] = vv;
    if (shadow) {
      uint2 o;
      *reinterpret_cast<__nv_bfloat162 *>(&o.x) = __floats2bfloat162_rn(pv.x, pv.y);
      *reinterpret_cast<__nv_bfloat162 *>(&o.y) = __floats2bfloat162_rn(pv.z, pv.w);
      reinterpret_cast<uint2 *>(shadow)[i] = o;
    }
  }
  for (int64_t i = n4 * 4 + tid; i < n; i += nthreads) {
    float pv = p[i], mv = m[i], vv = v[i];
    adam_one(pv, to_f32(g[i]), mv, vv, h, gs, wd);
    p[i] = pv; m[i] = mv; v[i] = vv;
    if (shadow) shadow[i] = __float2bfloat16_rn(pv);
  }
}

constexpr int64_t ADAM_CHUNK = 1 << 16;

struct AdamChunk {
  float *p, *m, *v;
  const void *g;
  __nv_bfloat16 *shadow;
  int32_t n;
  int32_t grad_dtype;
  float wd;
  float pad_;
};

__global__ void __launch_bounds__(256) adamw_chunks_kernel(const AdamChunk *__restrict__ chunks, AdamHyper h) {
  const AdamChunk c = chunks[blockIdx.x];
  bool skip;
  const float gs = effective_scale(h, &skip);
  if (skip) return;
  if (c.grad_dtype == ALPHA_F32)
    adam_span<float>(c.p, (const float *)c.g, c.m, c.v, c.shadow, c.n, h, gs, c.wd, threadIdx.x, blockDim.x);
  else
    adam_span<__nv_bfloat16>(c.p, (const __nv_bfloat16 *)c.g, c.m, c.v, c.shadow, c.n, h, gs, c.wd, threadIdx.x,
                             blockDim.x);
}

}  // namespace alpha

using namespace alpha;

extern "C" {

int alpha_adamw_multi(const alpha_adamw_tensor_t *tensors, int n_tensors, float lr, float beta1, float beta2,
                      float eps, float bc1, float bc2, float grad_scale, alpha_buf clip_sumsq, float max_norm) {
  ALPHA_REQUIRE_INIT();
  std::vector<AdamChunk> table;
  for (int t = 0; t < n_tensors; t++) {
    const alpha_adamw_tensor_t &T = tensors[t];
    ALPHA_CHECK(T.grad_dtype == ALPHA_F32 || T.grad_dtype == ALPHA_BF16, "alpha_adamw: unsupported grad dtype %d",
                T.grad_dtype);
    const size_t gs = dtype_size(T.grad_dtype);
    for (int64_t off = 0; off < T.n; off += ADAM_CHUNK) {
      AdamChunk c;
      memset(&c, 0, sizeof(c));  // the table is hashed by content: no stray padding bytes
      c.p = ptr<float>(T.p) + off;
      c.m = ptr<float>(T.m) + off;
      c.v = ptr<float>(T.v) + off;
      c.g = (const void *)(uintptr_t)(T.g + off * gs);
      c.shadow = T.p_shadow ? ptr<__nv_bfloat16>(T.p_shadow) + off : nullptr;
      c.n = (int32_t)(T.n - off < ADAM_CHUNK ? T.n - off : ADAM_CHUNK);
      c.grad_dtype = T.grad_dtype;
      c.wd = T.weight_decay;
      c.pad_ = 0.f;
      table.push_back(c);
    }
  }
  if (table.empty()) return 0;
  double prof_bytes = 0;
  for (int t = 0; t < n_tensors; t++)
    prof_bytes += (double)tensors[t].n * (24.0 + dtype_size(tensors[t].grad_dtype) + (tensors[t].p_shadow ? 2.0 : 0.0));
  ProfScope prof(PROF_ADAMW, prof_bytes);
  const void *dev_table = nullptr;
  if (table_upload(table.data(), table.size() * sizeof(AdamChunk), &dev_table)) return 1;
  AdamHyper h{lr, beta1, beta2, eps, bc1, bc2, grad_scale, max_norm, clip_sumsq ? ptr<float>(clip_sumsq) : nullptr};
  adamw_chunks_kernel<<<(unsigned)table.size(), 256, 0, g_stream>>>((const AdamChunk *)dev_table, h);
  ALPHA_LAUNCHED();
  return 0;
}

int alpha_adamw(alpha_buf p, alpha_buf g, alpha_buf m, alpha_buf v, int64_t n, float lr, float beta1, float beta2,
                float eps, float weight_decay, float bc1, float bc2, float grad_scale, int grad_dtype,
                alpha_buf p_shadow) {
  alpha_adamw_tensor_t t{p, g, m, v, p_shadow, n, weight_decay, grad_dtype};
  return alpha_adamw_multi(&t, 1, lr, beta1, beta2, eps, bc1, bc2, grad_scale, 0, 0.f);
}

}  // extern "C"
