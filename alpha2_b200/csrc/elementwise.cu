// Element-wise, cast, broadcast and layout kernels.  All are HBM-bound: 16-byte vector
// loads/stores on the contiguous paths, grid-stride loops sized to the SM count.
//
// Reference semantics: packages/tensor/src/cpu_ref.ts:151-165 (binary), :337-362 (unary),
// :422-437 (gelu/relu/silu), :567-656 (transpose/slice/scatterSlice), :884-915 (masks);
// backward formulas packages/autograd/src/ops.ts:287-419; dropout hash ops.ts:74-81.
#include <string.h>

#include "common.cuh"

namespace alpha {

__device__ __forceinline__ float apply_binary(int op, float a, float b) {
  switch (op) {
    case ALPHA_ADD: return a + b;
    case ALPHA_SUB: return a - b;
    case ALPHA_MUL: return a * b;
    default: return a / b;
  }
}

__device__ __forceinline__ float softcap_f(float x, float cap) {
  // tanh(x/cap)*cap (ops.ts:329-340; the reference clamps 2x/cap to +-80 before exp, which
  // leaves tanh unchanged to fp32 precision)
  return tanhf(x / cap) * cap;
}

__device__ __forceinline__ float apply_unary(int op, float x, float p0, float p1) {
  switch (op) {
    case ALPHA_NEG: return -x;
    case ALPHA_EXP: return expf(x);
    case ALPHA_LOG: return logf(x);
    case ALPHA_SQRT: return sqrtf(x);
    case ALPHA_RELU: return x > 0.f ? x : 0.f;
    case ALPHA_SILU: return x / (1.f + expf(-x));
    case ALPHA_GELU: return gelu_f(x);
    case ALPHA_SCALE: return x * p0;
    case ALPHA_CLAMP: return fmaxf(p0, fminf(p1, x));
    case ALPHA_POW: return powf(x, p0);
    default: return softcap_f(x, p0);
  }
}

__device__ __forceinline__ float apply_unary_bwd(int op, float x, float g, float p0, float p1) {
  switch (op) {
    case ALPHA_RELU: return x > 0.f ? g : 0.f;
    case ALPHA_SILU: {
      const float s = 1.f / (1.f + expf(-x));
      return g * (s * (1.f + x * (1.f - s)));
    }
    case ALPHA_GELU: return g * gelu_grad_f(x);
    case ALPHA_CLAMP: return (x > p0 && x < p1) ? g : 0.f;
    default: {  // SOFTCAP: d/dx tanh(x/cap)*cap = 1 - tanh^2(x/cap)
      const float t = tanhf(x / p0);
      return g * (1.f - t * t);
    }
  }
}

// Generic driver: Op::apply(i-th elements of up to three inputs) -> up to two outputs.
template <typename T, typename Op>
__global__ void __launch_bounds__(256) ew_kernel(Op op, int64_t n) {
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = op.vec_ok ? n / V : 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) op.vec(i * V);
  for (int64_t i = nvec * V + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) op.one(i);
}

template <typename T> struct OpFill {
  T *out; float v; bool vec_ok;
  __device__ void vec(int64_t i) const {
    float f[Vec16<T>::N];
#pragma unroll
    for (int j = 0; j < Vec16<T>::N; j++) f[j] = v;
    Vec16<T> o; o.set(f); o.store(out + i);
  }
  __device__ void one(int64_t i) const { out[i] = from_f32<T>(v); }
};

template <typename T> struct OpBinary {
  const T *a, *b; T *out; int op; bool vec_ok;
  __device__ void vec(int64_t i) const {
    constexpr int V = Vec16<T>::N;
    Vec16<T> va, vb, vo; float fa[V], fb[V];
    va.load(a + i); vb.load(b + i); va.get(fa); vb.get(fb);
#pragma unroll
    for (int j = 0; j < V; j++) fa[j] = apply_binary(op, fa[j], fb[j]);
    vo.set(fa); vo.store(out + i);
  }
  __device__ void one(int64_t i) const { out[i] = from_f32<T>(apply_binary(op, to_f32(a[i]), to_f32(b[i]))); }
};

template <typename T> struct OpUnary {
  const T *a; T *out; int op; float p0, p1; bool vec_ok;
  __device__ void vec(int64_t i) const {
    constexpr int V = Vec16<T>::N;
    Vec16<T> va, vo; float fa[V];
    va.load(a + i); va.get(fa);
#pragma unroll
    for (int j = 0; j < V; j++) fa[j] = apply_unary(op, fa[j], p0, p1);
    vo.set(fa); vo.store(out + i);
  }
  __device__ void one(int64_t i) const { out[i] = from_f32<T>(apply_unary(op, to_f32(a[i]), p0, p1)); }
};

template <typename T> struct OpUnaryBwd {
  const T *x, *g; T *out; int op; float p0, p1; bool vec_ok;
  __device__ void vec(int64_t i) const {
    constexpr int V = Vec16<T>::N;
    Vec16<T> vx, vg, vo; float fx[V], fg[V];
    vx.load(x + i); vg.load(g + i); vx.get(fx); vg.get(fg);
#pragma unroll
    for (int j = 0; j < V; j++) fx[j] = apply_unary_bwd(op, fx[j], fg[j], p0, p1);
    vo.set(fx); vo.store(out + i);
  }
  __device__ void one(int64_t i) const {
    out[i] = from_f32<T>(apply_unary_bwd(op, to_f32(x[i]), to_f32(g[i]), p0, p1));
  }
};

template <typename T> struct OpSiluMul {
  const T *a, *b; T *out; bool vec_ok;
  __device__ static float f(float x, float y) { return x / (1.f + expf(-x)) * y; }
  __device__ void vec(int64_t i) const {
    constexpr int V = Vec16<T>::N;
    Vec16<T> va, vb, vo; float fa[V], fb[V];
    va.load(a + i); vb.load(b + i); va.get(fa); vb.get(fb);
#pragma unroll
    for (int j = 0; j < V; j++) fa[j] = f(fa[j], fb[j]);
    vo.set(fa); vo.store(out + i);
  }
  __device__ void one(int64_t i) const { out[i] = from_f32<T>(f(to_f32(a[i]), to_f32(b[i]))); }
};

// da = g*b*silu'(a), db = g*silu(a)  (ops.ts:364-399)
template <typename T> struct OpSiluMulBwd {
  const T *a, *b, *g; T *da, *db; bool vec_ok;
  __device__ static void f(float x, float y, float gg, float &oa, float &ob) {
    const float s = 1.f / (1.f + expf(-x));
    oa = gg * y * (s * (1.f + x * (1.f - s)));
    ob = gg * (x * s);
  }
  __device__ void vec(int64_t i) const {
    constexpr int V = Vec16<T>::N;
    Vec16<T> va, vb, vg, oa, ob; float fa[V], fb[V], fg[V];
    va.load(a + i); vb.load(b + i); vg.load(g + i); va.get(fa); vb.get(fb); vg.get(fg);
#pragma unroll
    for (int j = 0; j < V; j++) { float x, y; f(fa[j], fb[j], fg[j], x, y); fa[j] = x; fb[j] = y; }
    oa.set(fa); ob.set(fb); oa.store(da + i); ob.store(db + i);
  }
  __device__ void one(int64_t i) const {
    float x, y; f(to_f32(a[i]), to_f32(b[i]), to_f32(g[i]), x, y);
    da[i] = from_f32<T>(x); db[i] = from_f32<T>(y);
  }
};

template <typename T> struct OpScaleInplace {
  T *a; float s; bool vec_ok;
  __device__ void vec(int64_t i) const {
    constexpr int V = Vec16<T>::N;
    Vec16<T> va; float fa[V];
    va.load(a + i); va.get(fa);
#pragma unroll
    for (int j = 0; j < V; j++) fa[j] *= s;
    va.set(fa); va.store(a + i);
  }
  __device__ void one(int64_t i) const { a[i] = from_f32<T>(to_f32(a[i]) * s); }
};

template <typename T> struct OpResidualDropoutAdd {
  const T *r, *p, *m; T *out; bool vec_ok;
  __device__ void vec(int64_t i) const {
    constexpr int V = Vec16<T>::N;
    Vec16<T> vr, vp, vm, vo; float fr[V], fp[V], fm[V];
    vr.load(r + i); vp.load(p + i); vm.load(m + i); vr.get(fr); vp.get(fp); vm.get(fm);
#pragma unroll
    for (int j = 0; j < V; j++) fr[j] = fr[j] + fp[j] * fm[j];
    vo.set(fr); vo.store(out + i);
  }
  __device__ void one(int64_t i) const { out[i] = from_f32<T>(to_f32(r[i]) + to_f32(p[i]) * to_f32(m[i])); }
};

template <typename T, typename Op>
static int launch_ew(Op op, int64_t n) {
  if (n <= 0) return 0;
  ProfScope prof(PROF_ELEMENTWISE, (double)n);
  const int block = 256;
  const int grid = grid_for((n + Vec16<T>::N - 1) / Vec16<T>::N, block, 16);
  ew_kernel<T, Op><<<grid, block, 0, g_stream>>>(op, n);
  ALPHA_LAUNCHED();
  return 0;
}

static inline bool al16(alpha_buf b) { return (b & 15) == 0; }

// a (Ta) += b (Tb); covers f32 += f32, f32 += bf16 (gradient accumulation), bf16 += bf16.
template <typename Ta, typename Tb>
__global__ void __launch_bounds__(256) add_inplace_kernel(Ta *a, const Tb *b, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    a[i] = from_f32<Ta>(to_f32(a[i]) + to_f32(b[i]));
}

template <typename Ts, typename Td>
__global__ void __launch_bounds__(256) cast_kernel(const Ts *s, Td *d, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t n4 = n / 4;
  const bool vec = aligned16(s) && aligned16(d) || (sizeof(Ts) == 2 && (((uintptr_t)s & 7) == 0) && aligned16(d)) ||
                   (sizeof(Td) == 2 && aligned16(s) && (((uintptr_t)d & 7) == 0));
  if (vec) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
      float f[4];
#pragma unroll
      for (int j = 0; j < 4; j++) f[j] = to_f32(s[i * 4 + j]);
#pragma unroll
      for (int j = 0; j < 4; j++) d[i * 4 + j] = from_f32<Td>(f[j]);
    }
    for (int64_t i = n4 * 4 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
      d[i] = from_f32<Td>(to_f32(s[i]));
  } else {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
      d[i] = from_f32<Td>(to_f32(s[i]));
  }
}

struct Shape6 {
  int64_t shape[6], sa[6], sb[6];
  int ndim;
};

template <typename T, bool BINARY>
__global__ void __launch_bounds__(256) bcast_kernel(const T *a, const T *b, T *out, Shape6 s, int64_t n, int op) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t rem = i, ia = 0, ib = 0;
    for (int d = s.ndim - 1; d >= 0; d--) {
      const int64_t c = rem % s.shape[d];
      rem /= s.shape[d];
      ia += c * s.sa[d];
      if (BINARY) ib += c * s.sb[d];
    }
    out[i] = BINARY ? from_f32<T>(apply_binary(op, to_f32(a[ia]), to_f32(b[ib]))) : a[ia];
  }
}

// out[..., j(d1), ..., i(d0), ...] = a[..., i, ..., j, ...]; s.sa holds, per output
// dimension, the input stride to walk (a pure stride permutation).
template <typename T>
__global__ void __launch_bounds__(256) permute_kernel(const T *a, T *out, Shape6 s, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t rem = i, ia = 0;
    for (int d = s.ndim - 1; d >= 0; d--) {
      const int64_t c = rem % s.shape[d];
      rem /= s.shape[d];
      ia += c * s.sa[d];
    }
    out[i] = a[ia];
  }
}

// [batch, R, C] -> [batch, C, R] through a padded 32x32 shared tile (coalesced both ways).
template <typename T>
__global__ void __launch_bounds__(256) transpose_tile_kernel(const T *a, T *out, int64_t R, int64_t C) {
  __shared__ T tile[32][33];
  const int64_t base = (int64_t)blockIdx.z * R * C;
  const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int64_t r = r0 + j, c = c0 + threadIdx.x;
    if (r < R && c < C) tile[j][threadIdx.x] = a[base + r * C + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int64_t c = c0 + j, r = r0 + threadIdx.x;
    if (r < R && c < C) out[base + c * R + r] = tile[threadIdx.x][j];
  }
}

// mode 0: out[r, 0:w] = a[r, c0:c0+w];  mode 1: out[r, :] = zeros except out[r, c0:c0+w] = g[r, :]
template <typename T>
__global__ void __launch_bounds__(256) cols_kernel(const T *src, T *dst, int64_t rows, int64_t cols, int64_t c0,
                                                   int64_t w, int mode) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t n = mode == 0 ? rows * w : rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    if (mode == 0) {
      const int64_t r = i / w, c = i - r * w;
      dst[i] = src[r * cols + c0 + c];
    } else {
      const int64_t r = i / cols, c = i - r * cols;
      dst[i] = (c >= c0 && c < c0 + w) ? src[r * w + (c - c0)] : from_f32<T>(0.f);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) slice_qkv_kernel(const T *a, T *q, T *k, T *v, int64_t rows, int64_t d) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t n = rows * 3 * d;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t r = i / (3 * d), c = i - r * 3 * d;
    const int which = (int)(c / d);
    const int64_t cc = c - which * d;
    T *dst = which == 0 ? q : (which == 1 ? k : v);
    dst[r * d + cc] = a[i];
  }
}

__global__ void __launch_bounds__(256) causal_mask_kernel(float *out, int64_t size) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < size * size; i += stride) {
    const int64_t r = i / size, c = i - r * size;
    out[i] = c > r ? -INFINITY : 0.f;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) masked_fill_kernel(const T *a, const float *mask, T *out, int64_t n,
                                                          int64_t mask_n, float value) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = mask[i % mask_n] != 0.f ? from_f32<T>(value) : a[i];
}

// ops.ts:74-81 — splitmix32-style hash of (seed, counter, index); keep where hash > p.
template <typename T>
__global__ void __launch_bounds__(256) dropout_mask_kernel(T *out, int64_t n, int32_t seed, int32_t counter, float p) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const float keep = 1.f / (1.f - p);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    // JavaScript evaluates seed + counter*2654435761 + index*2246822519 in doubles and then
    // truncates to int32; for the magnitudes that occur the low 32 bits equal this sum.
    uint32_t h = (uint32_t)seed + (uint32_t)counter * 2654435761u + (uint32_t)i * 2246822519u;
    h = (h ^ (h >> 16)) * 0x85ebca6bu;
    h = (h ^ (h >> 13)) * 0xc2b2ae35u;
    h = h ^ (h >> 16);
    const float u = (float)((double)h / 4294967296.0);
    out[i] = from_f32<T>(u > p ? keep : 0.f);
  }
}

}  // namespace alpha

using namespace alpha;

#define DISPATCH_FLOAT(dt, ...)                                   \
  if ((dt) == ALPHA_F32) { using T = float; __VA_ARGS__; }         \
  else if ((dt) == ALPHA_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
  else return set_error("%s: unsupported dtype %d", __func__, (int)(dt));

extern "C" {

int alpha_fill(alpha_buf dst, int64_t n, float value, int dtype) {
  ALPHA_REQUIRE_INIT();
  if (dtype == ALPHA_I32) {
    // integer fill: route through the f32 kernel on the bit pattern of the int value
    const int32_t iv = (int32_t)value;
    float bits;
    memcpy(&bits, &iv, 4);
    return launch_ew<float>(OpFill<float>{ptr<float>(dst), bits, al16(dst)}, n);
  }
  DISPATCH_FLOAT(dtype, return launch_ew<T>(OpFill<T>{ptr<T>(dst), value, al16(dst)}, n));
}

int alpha_binary(int op, alpha_buf a, alpha_buf b, alpha_buf out, int64_t n, int dtype) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(op >= ALPHA_ADD && op <= ALPHA_DIV, "alpha_binary: bad op %d", op);
  DISPATCH_FLOAT(dtype, return launch_ew<T>(
      OpBinary<T>{ptr<T>(a), ptr<T>(b), ptr<T>(out), op, al16(a) && al16(b) && al16(out)}, n));
}

static int fill_shape6(Shape6 &s, int ndim, const int64_t *shape, const int64_t *sa, const int64_t *sb,
                       int64_t *n_out) {
  if (ndim < 0 || ndim > 6) return set_error("broadcast: ndim %d > 6", ndim);
  s.ndim = ndim;
  int64_t n = 1;
  for (int d = 0; d < ndim; d++) {
    s.shape[d] = shape[d];
    s.sa[d] = sa ? sa[d] : 0;
    s.sb[d] = sb ? sb[d] : 0;
    n *= shape[d];
  }
  *n_out = n;
  return 0;
}

int alpha_binary_bcast(int op, alpha_buf a, alpha_buf b, alpha_buf out, int ndim, const int64_t *out_shape,
                       const int64_t *a_strides, const int64_t *b_strides, int dtype) {
  ALPHA_REQUIRE_INIT();
  Shape6 s;
  int64_t n;
  if (fill_shape6(s, ndim, out_shape, a_strides, b_strides, &n)) return 1;
  if (n == 0) return 0;
  DISPATCH_FLOAT(dtype, {
    bcast_kernel<T, true><<<grid_for(n, 256), 256, 0, g_stream>>>(ptr<T>(a), ptr<T>(b), ptr<T>(out), s, n, op);
    ALPHA_LAUNCHED();
    return 0;
  });
}

int alpha_broadcast(alpha_buf a, alpha_buf out, int ndim, const int64_t *out_shape, const int64_t *a_strides,
                    int dtype) {
  ALPHA_REQUIRE_INIT();
  Shape6 s;
  int64_t n;
  if (fill_shape6(s, ndim, out_shape, a_strides, nullptr, &n)) return 1;
  if (n == 0) return 0;
  DISPATCH_FLOAT(dtype, {
    bcast_kernel<T, false><<<grid_for(n, 256), 256, 0, g_stream>>>(ptr<T>(a), nullptr, ptr<T>(out), s, n, 0);
    ALPHA_LAUNCHED();
    return 0;
  });
}

int alpha_unary(int op, alpha_buf a, alpha_buf out, int64_t n, float p0, float p1, int dtype) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(op >= ALPHA_NEG && op <= ALPHA_SOFTCAP, "alpha_unary: bad op %d", op);
  DISPATCH_FLOAT(dtype, return launch_ew<T>(OpUnary<T>{ptr<T>(a), ptr<T>(out), op, p0, p1, al16(a) && al16(out)}, n));
}

int alpha_unary_bwd(int op, alpha_buf x, alpha_buf g, alpha_buf out, int64_t n, float p0, float p1, int dtype) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(op == ALPHA_RELU || op == ALPHA_SILU || op == ALPHA_GELU || op == ALPHA_CLAMP || op == ALPHA_SOFTCAP,
              "alpha_unary_bwd: op %d has no backward entry", op);
  DISPATCH_FLOAT(dtype, return launch_ew<T>(
      OpUnaryBwd<T>{ptr<T>(x), ptr<T>(g), ptr<T>(out), op, p0, p1, al16(x) && al16(g) && al16(out)}, n));
}

int alpha_add_inplace(alpha_buf a, alpha_buf b, int64_t n, int a_dtype, int b_dtype) {
  ALPHA_REQUIRE_INIT();
  if (n <= 0) return 0;
  if (a_dtype == b_dtype) {
    DISPATCH_FLOAT(a_dtype, return launch_ew<T>(
        OpBinary<T>{ptr<T>(a), ptr<T>(b), ptr<T>(a), ALPHA_ADD, al16(a) && al16(b)}, n));
  }
  ALPHA_CHECK(a_dtype == ALPHA_F32 && b_dtype == ALPHA_BF16, "alpha_add_inplace: only f32 += bf16 mixes dtypes");
  ProfScope prof(PROF_ELEMENTWISE, (double)n);
  add_inplace_kernel<float, __nv_bfloat16><<<grid_for(n, 256, 16), 256, 0, g_stream>>>(ptr<float>(a),
                                                                                         ptr<__nv_bfloat16>(b), n);
  ALPHA_LAUNCHED();
  return 0;
}

int alpha_scale_inplace(alpha_buf a, float s, int64_t n, int dtype) {
  ALPHA_REQUIRE_INIT();
  DISPATCH_FLOAT(dtype, return launch_ew<T>(OpScaleInplace<T>{ptr<T>(a), s, al16(a)}, n));
}

int alpha_cast(alpha_buf src, int sdt, alpha_buf dst, int ddt, int64_t n) {
  ALPHA_REQUIRE_INIT();
  if (n <= 0) return 0;
  ProfScope prof(PROF_ELEMENTWISE, (double)n);
  const int grid = grid_for((n + 3) / 4, 256, 16);
  if (sdt == ALPHA_F32 && ddt == ALPHA_BF16)
    cast_kernel<float, __nv_bfloat16><<<grid, 256, 0, g_stream>>>(ptr<float>(src), ptr<__nv_bfloat16>(dst), n);
  else if (sdt == ALPHA_BF16 && ddt == ALPHA_F32)
    cast_kernel<__nv_bfloat16, float><<<grid, 256, 0, g_stream>>>(ptr<__nv_bfloat16>(src), ptr<float>(dst), n);
  else if (sdt == ddt)
    return alpha_d2d(dst, src, (size_t)n * dtype_size(sdt));
  else
    return set_error("alpha_cast: unsupported %d -> %d", sdt, ddt);
  ALPHA_LAUNCHED();
  return 0;
}

int alpha_silu_mul_fwd(alpha_buf a, alpha_buf b, alpha_buf out, int64_t n, int dtype) {
  ALPHA_REQUIRE_INIT();
  DISPATCH_FLOAT(dtype, return launch_ew<T>(
      OpSiluMul<T>{ptr<T>(a), ptr<T>(b), ptr<T>(out), al16(a) && al16(b) && al16(out)}, n));
}

int alpha_silu_mul_bwd(alpha_buf a, alpha_buf b, alpha_buf g, alpha_buf da, alpha_buf db, int64_t n, int dtype) {
  ALPHA_REQUIRE_INIT();
  DISPATCH_FLOAT(dtype, return launch_ew<T>(
      OpSiluMulBwd<T>{ptr<T>(a), ptr<T>(b), ptr<T>(g), ptr<T>(da), ptr<T>(db),
                      al16(a) && al16(b) && al16(g) && al16(da) && al16(db)}, n));
}

int alpha_transpose(alpha_buf a, alpha_buf out, int ndim, const int64_t *shape, int d0, int d1, int dtype) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(ndim >= 1 && ndim <= 6, "alpha_transpose: ndim %d not in [1,6]", ndim);
  if (d0 < 0) d0 += ndim;
  if (d1 < 0) d1 += ndim;
  ALPHA_CHECK(d0 >= 0 && d0 < ndim && d1 >= 0 && d1 < ndim, "alpha_transpose: bad dims");
  int64_t in_strides[6], n = 1;
  for (int d = ndim - 1; d >= 0; d--) {
    in_strides[d] = n;
    n *= shape[d];
  }
  if (n == 0) return 0;
  if (d0 == d1) return alpha_d2d(out, a, (size_t)n * dtype_size(dtype));
  const int lo = d0 < d1 ? d0 : d1, hi = d0 < d1 ? d1 : d0;
  // Swapping the last two dimensions: tiled transpose, batch = product of the leading ones.
  if (hi == ndim - 1 && lo == ndim - 2) {
    const int64_t R = shape[lo], C = shape[hi], batch = n / (R * C);
    if (batch <= 65535 && (R + 31) / 32 <= 65535) {
      dim3 grid((unsigned)((C + 31) / 32), (unsigned)((R + 31) / 32), (unsigned)batch), block(32, 8);
      DISPATCH_FLOAT(dtype, {
        transpose_tile_kernel<T><<<grid, block, 0, g_stream>>>(ptr<T>(a), ptr<T>(out), R, C);
        ALPHA_LAUNCHED();
        return 0;
      });
    }
  }
  Shape6 s;
  s.ndim = ndim;
  for (int d = 0; d < ndim; d++) {
    const int src = d == d0 ? d1 : (d == d1 ? d0 : d);
    s.shape[d] = shape[src];
    s.sa[d] = in_strides[src];
    s.sb[d] = 0;
  }
  DISPATCH_FLOAT(dtype, {
    permute_kernel<T><<<grid_for(n, 256, 16), 256, 0, g_stream>>>(ptr<T>(a), ptr<T>(out), s, n);
    ALPHA_LAUNCHED();
    return 0;
  });
}

int alpha_slice_cols(alpha_buf a, alpha_buf out, int64_t rows, int64_t cols, int64_t c0, int64_t c1, int dtype) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(0 <= c0 && c0 <= c1 && c1 <= cols, "alpha_slice_cols: bad range [%lld,%lld) of %lld", (long long)c0,
              (long long)c1, (long long)cols);
  const int64_t n = rows * (c1 - c0);
  if (n == 0) return 0;
  DISPATCH_FLOAT(dtype, {
    cols_kernel<T><<<grid_for(n, 256, 16), 256, 0, g_stream>>>(ptr<T>(a), ptr<T>(out), rows, cols, c0, c1 - c0, 0);
    ALPHA_LAUNCHED();
    return 0;
  });
}

int alpha_scatter_cols(alpha_buf g, alpha_buf out, int64_t rows, int64_t cols, int64_t c0, int64_t c1, int dtype) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(0 <= c0 && c0 <= c1 && c1 <= cols, "alpha_scatter_cols: bad range");
  const int64_t n = rows * cols;
  if (n == 0) return 0;
  DISPATCH_FLOAT(dtype, {
    cols_kernel<T><<<grid_for(n, 256, 16), 256, 0, g_stream>>>(ptr<T>(g), ptr<T>(out), rows, cols, c0, c1 - c0, 1);
    ALPHA_LAUNCHED();
    return 0;
  });
}

int alpha_slice_qkv(alpha_buf a, alpha_buf q, alpha_buf k, alpha_buf v, int64_t rows, int64_t d, int dtype) {
  ALPHA_REQUIRE_INIT();
  const int64_t n = rows * 3 * d;
  if (n == 0) return 0;
  DISPATCH_FLOAT(dtype, {
    slice_qkv_kernel<T><<<grid_for(n, 256, 16), 256, 0, g_stream>>>(ptr<T>(a), ptr<T>(q), ptr<T>(k), ptr<T>(v), rows, d);
    ALPHA_LAUNCHED();
    return 0;
  });
}

int alpha_causal_mask(alpha_buf out, int64_t size) {
  ALPHA_REQUIRE_INIT();
  if (size == 0) return 0;
  causal_mask_kernel<<<grid_for(size * size, 256), 256, 0, g_stream>>>(ptr<float>(out), size);
  ALPHA_LAUNCHED();
  return 0;
}

int alpha_masked_fill(alpha_buf a, alpha_buf mask, alpha_buf out, int64_t n, int64_t mask_n, float value, int dtype) {
  ALPHA_REQUIRE_INIT();
  if (n == 0) return 0;
  ALPHA_CHECK(mask_n > 0, "alpha_masked_fill: empty mask");
  DISPATCH_FLOAT(dtype, {
    masked_fill_kernel<T><<<grid_for(n, 256, 16), 256, 0, g_stream>>>(ptr<T>(a), ptr<float>(mask), ptr<T>(out), n,
                                                                      mask_n, value);
    ALPHA_LAUNCHED();
    return 0;
  });
}

int alpha_dropout_mask(alpha_buf out, int64_t n, int32_t seed, int32_t counter, float p, int dtype) {
  ALPHA_REQUIRE_INIT();
  if (n == 0) return 0;
  DISPATCH_FLOAT(dtype, {
    dropout_mask_kernel<T><<<grid_for(n, 256, 16), 256, 0, g_stream>>>(ptr<T>(out), n, seed, counter, p);
    ALPHA_LAUNCHED();
    return 0;
  });
}

int alpha_residual_dropout_add(alpha_buf residual, alpha_buf projected, alpha_buf mask, alpha_buf out, int64_t n,
                               int dtype) {
  ALPHA_REQUIRE_INIT();
  DISPATCH_FLOAT(dtype, return launch_ew<T>(
      OpResidualDropoutAdd<T>{ptr<T>(residual), ptr<T>(projected), ptr<T>(mask), ptr<T>(out),
                              al16(residual) && al16(projected) && al16(mask) && al16(out)}, n));
}

}  // extern "C"
