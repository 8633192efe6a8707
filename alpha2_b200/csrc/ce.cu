// Softmax cross-entropy: forward, backward, and the fused forward+backward used by the
// train step.  HBM-bound on the [N, V] logits.
//
// Reference semantics: packages/tensor/src/cpu_ref.ts:543-563 (loss = mean_i(lse_i -
// logit_i[target_i])) and packages/autograd/src/ops.ts:702-729 (grad = (softmax - onehot) *
// g / N).  The reference's GPU path reads the summed loss back to divide by N and reads the
// upstream scalar on the host (packages/helios/src/backend.ts:2704,4511-4515); here both
// stay on the device.
//
// One block per row.  The row is staged once in shared memory with 16-byte loads (V*e
// bytes: 100 KB for V=50257 in bf16), so the fused kernel reads each logit from HBM once
// and writes each gradient once: algorithmic bytes per row = V*e read + V*e written.
// Row losses go to a scratch vector and are averaged by one block in index order.
#include "tc_common.cuh"

namespace alpha {

constexpr int CE_THREADS = 512;

// mode bit 0: write the row loss; bit 1: write dlogits.
template <typename T, bool STAGE>
__global__ void __launch_bounds__(CE_THREADS) ce_rows_kernel(const T *__restrict__ logits,
                                                             const int32_t *__restrict__ targets, T *dlogits,
                                                             float *__restrict__ row_loss,
                                                             const float *__restrict__ grad_out_dev, float grad_scale,
                                                             int64_t N, int V, int64_t ld, int mode) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float red[32];
  T *row_s = reinterpret_cast<T *>(smem_raw);
  constexpr int VEC = Vec16<T>::N;
  const float gs = (grad_out_dev ? grad_out_dev[0] : 1.f) * grad_scale / (float)N;
  for (int64_t r = blockIdx.x; r < N; r += gridDim.x) {
    const T *row = logits + r * ld;
    const int nvec = V / VEC;
    float mx = -INFINITY;
    if (STAGE) {
      for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
        Vec16<T> v;
        v.load(row + i * VEC);
        v.store(row_s + i * VEC);
        float f[VEC];
        v.get(f);
#pragma unroll
        for (int j = 0; j < VEC; j++) mx = fmaxf(mx, f[j]);
      }
      for (int c = nvec * VEC + threadIdx.x; c < V; c += CE_THREADS) {
        const T t = row[c];
        row_s[c] = t;
        mx = fmaxf(mx, to_f32(t));
      }
    } else {
      for (int c = threadIdx.x; c < V; c += CE_THREADS) mx = fmaxf(mx, to_f32(row[c]));
    }
    mx = block_max(mx, red);  // also orders the shared-memory row before it is re-read
    const T *src = STAGE ? row_s : row;
    float s = 0.f;
    if (STAGE) {
      for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
        Vec16<T> v;
        v.load(src + i * VEC);
        float f[VEC];
        v.get(f);
#pragma unroll
        for (int j = 0; j < VEC; j++) s += __expf(f[j] - mx);
      }
      for (int c = nvec * VEC + threadIdx.x; c < V; c += CE_THREADS) s += __expf(to_f32(src[c]) - mx);
    } else {
      for (int c = threadIdx.x; c < V; c += CE_THREADS) s += expf(to_f32(src[c]) - mx);
    }
    s = block_sum(s, red);
    const int tgt = targets[r];
    if ((mode & 1) && threadIdx.x == 0) {
      const float lt = (tgt >= 0 && tgt < V) ? to_f32(src[tgt]) : 0.f;
      row_loss[r] = (mx + logf(s)) - lt;
    }
    if (mode & 2) {
      // dlogits may alias logits: the target logit above must be read before anyone writes
      if (!STAGE) __syncthreads();
      const float inv = 1.f / s;
      T *drow = dlogits + r * ld;
      if (STAGE) {
        for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
          Vec16<T> v;
          v.load(src + i * VEC);
          float f[VEC];
          v.get(f);
#pragma unroll
          for (int j = 0; j < VEC; j++) {
            const float p = __expf(f[j] - mx) * inv;
            f[j] = (p - ((i * VEC + j) == tgt ? 1.f : 0.f)) * gs;
          }
          v.set(f);
          v.store(drow + i * VEC);
        }
        for (int c = nvec * VEC + threadIdx.x; c < V; c += CE_THREADS) {
          const float p = __expf(to_f32(src[c]) - mx) * inv;
          drow[c] = from_f32<T>((p - (c == tgt ? 1.f : 0.f)) * gs);
        }
      } else {
        for (int c = threadIdx.x; c < V; c += CE_THREADS) {
          const float p = expf(to_f32(src[c]) - mx) * inv;
          drow[c] = from_f32<T>((p - (c == tgt ? 1.f : 0.f)) * gs);
        }
      }
    }
    __syncthreads();  // the staged row is overwritten by the next iteration
  }
}

// bf16 rows staged in shared memory, lean arithmetic (the generic staged kernel above spends
// ~28 thread instructions per logit and is bound by instruction issue, not by HBM):
//   pass 1  global -> shared with 16-byte copies, row maximum (3-input max on unpacked pairs)
//   pass 2  sum of exp2(x*log2e - max*log2e): one packed FMA per pair + one exp2 per element
//   pass 3  the same exponentials times (grad scale / sum), packed, rounded to bf16, stored;
//           the thread that owns the target's 16-byte vector subtracts the one-hot term
// exp2 is evaluated twice per logit (passes 2 and 3) rather than kept, so the shared copy
// stays read-only and the probabilities are rounded once.
__device__ __forceinline__ void bf16x8_to_pairs(const uint4 &v, uint64_t (&p)[4]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int q = 0; q < 4; q++) p[q] = tc::bf16x2_to_f2(w[q]);
}

__global__ void __launch_bounds__(CE_THREADS, 2)
ce_rows_bf16_kernel(const __nv_bfloat16 *__restrict__ logits, const int32_t *__restrict__ targets,
                    __nv_bfloat16 *dlogits, float *__restrict__ row_loss, const float *__restrict__ grad_out_dev,
                    float grad_scale, int64_t N, int V, int64_t ld, int mode) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float red[32];
  uint4 *row_s = reinterpret_cast<uint4 *>(smem_raw);
  const __nv_bfloat16 *row_e = reinterpret_cast<const __nv_bfloat16 *>(smem_raw);
  const float LOG2E = 1.4426950408889634f;
  const float gs = (grad_out_dev ? grad_out_dev[0] : 1.f) * grad_scale / (float)N;
  const int nvec = V / 8;
  for (int64_t r = blockIdx.x; r < N; r += gridDim.x) {
    const __nv_bfloat16 *row = logits + r * ld;
    const uint4 *row_v = reinterpret_cast<const uint4 *>(row);
    const int tgt = targets[r];
    // the target's logit is read before dlogits (which may alias logits) is written
    float lt = 0.f;
    if (threadIdx.x == 0 && tgt >= 0 && tgt < V) lt = __bfloat162float(row[tgt]);
    // the row maximum is taken on packed bf16 pairs (one instruction per two logits; exact:
    // the maximum of bf16 values is one of them) and widened once at the end
    __nv_bfloat162 mx2 = __float2bfloat162_rn(-INFINITY);
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
      const uint4 v = row_v[i];
      row_s[i] = v;
      mx2 = __hmax2(mx2, __hmax2(__hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&v.x),
                                         *reinterpret_cast<const __nv_bfloat162 *>(&v.y)),
                                 __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&v.z),
                                         *reinterpret_cast<const __nv_bfloat162 *>(&v.w))));
    }
    float mx = fmaxf(__low2float(mx2), __high2float(mx2));
    for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) {
      const __nv_bfloat16 t = row[c];
      reinterpret_cast<__nv_bfloat16 *>(smem_raw)[c] = t;
      mx = fmaxf(mx, __bfloat162float(t));
    }
    mx = block_max(mx, red);  // also orders the shared-memory row before it is re-read
    const float nmx2 = -mx * LOG2E;
    const uint64_t l2 = tc::f2_pack(LOG2E, LOG2E), nm = tc::f2_pack(nmx2, nmx2);
    uint64_t s2 = tc::f2_pack(0.f, 0.f);
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
      uint64_t p[4];
      bf16x8_to_pairs(row_s[i], p);
#pragma unroll
      for (int q = 0; q < 4; q++) {
        float a, b;
        tc::f2_unpack(tc::f2_fma(p[q], l2, nm), a, b);
        s2 = tc::f2_add(s2, tc::f2_pack(tc::ex2_approx(a), tc::ex2_approx(b)));
      }
    }
    float sa, sb;
    tc::f2_unpack(s2, sa, sb);
    float s = sa + sb;
    for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS)
      s += tc::ex2_approx(fmaf(__bfloat162float(row_e[c]), LOG2E, nmx2));
    s = block_sum(s, red);
    if ((mode & 1) && threadIdx.x == 0) row_loss[r] = (mx + logf(s)) - lt;
    if (mode & 2) {
      const float k = gs / s;
      const uint64_t k2 = tc::f2_pack(k, k);
      uint4 *drow = reinterpret_cast<uint4 *>(dlogits + r * ld);
      const int tvec = (tgt >= 0 && tgt < V) ? tgt >> 3 : -1;
      for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
        uint64_t p[4];
        bf16x8_to_pairs(row_s[i], p);
        float o[8];
#pragma unroll
        for (int q = 0; q < 4; q++) {
          float a, b;
          tc::f2_unpack(tc::f2_fma(p[q], l2, nm), a, b);
          tc::f2_unpack(tc::f2_mul(tc::f2_pack(tc::ex2_approx(a), tc::ex2_approx(b)), k2), o[2 * q], o[2 * q + 1]);
        }
        if (i == tvec) o[tgt & 7] -= gs;
        uint4 w;
        w.x = tc::bf16x2_pack(o[0], o[1]);
        w.y = tc::bf16x2_pack(o[2], o[3]);
        w.z = tc::bf16x2_pack(o[4], o[5]);
        w.w = tc::bf16x2_pack(o[6], o[7]);
        drow[i] = w;
      }
      __nv_bfloat16 *dtail = dlogits + r * ld;
      for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) {
        const float pr = tc::ex2_approx(fmaf(__bfloat162float(row_e[c]), LOG2E, nmx2)) * k;
        dtail[c] = __float2bfloat16(pr - (c == tgt ? gs : 0.f));
      }
    }
    __syncthreads();  // the staged row is overwritten by the next iteration
  }
}

__global__ void __launch_bounds__(1024) ce_mean_kernel(const float *__restrict__ row_loss, int64_t N,
                                                       float *__restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < N; i += blockDim.x) s += row_loss[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = s / (float)N;
}

template <typename T>
static int ce_launch(alpha_buf logits, alpha_buf targets, alpha_buf dlogits, alpha_buf loss_mean, alpha_buf grad_out,
                     float grad_scale, int64_t N, int64_t V, int64_t ld, int mode) {
  if (N == 0 || V == 0) {
    if ((mode & 1) && loss_mean) ALPHA_CUDA(cudaMemsetAsync(ptr<void>(loss_mean), 0, 4, g_stream));
    return 0;
  }
  ALPHA_CHECK(V < (1ll << 31), "cross entropy: V too large");
  ProfScope prof(PROF_CE, (double)N * V * sizeof(T) * ((mode & 2) ? 2.0 : 1.0));
  void *row_loss = nullptr;
  if (mode & 1)
    if (pool_alloc((size_t)N * sizeof(float), &row_loss)) return 1;
  constexpr int VEC = Vec16<T>::N;
  const size_t row_bytes = ((size_t)V * sizeof(T) + 15) & ~size_t(15);
  // The fp32 path (parity mode) keeps full-precision expf; the staged path uses the fast
  // exponential (2 ulp), which is far inside bf16 resolution.
  const bool stage = sizeof(T) == 2 && row_bytes <= 200 * 1024 && ld % VEC == 0 && (logits & 15) == 0 &&
                     (!(mode & 2) || (dlogits & 15) == 0);
  const int grid = grid_for(N, 1, stage ? 2 : 4);
  if (stage) {
    static int attr_set = -1;
    if (attr_set != g_init_epoch) {
      ALPHA_CUDA(cudaFuncSetAttribute(ce_rows_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      attr_set = g_init_epoch;
    }
    if constexpr (sizeof(T) == 2) {
      static int attr2_set = -1;
      if (attr2_set != g_init_epoch) {
        ALPHA_CUDA(cudaFuncSetAttribute(ce_rows_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr2_set = g_init_epoch;
      }
      ce_rows_bf16_kernel<<<grid, CE_THREADS, row_bytes, g_stream>>>(
          ptr<__nv_bfloat16>(logits), ptr<int32_t>(targets), ptr<__nv_bfloat16>(dlogits), (float *)row_loss,
          grad_out ? ptr<float>(grad_out) : nullptr, grad_scale, N, (int)V, ld, mode);
    } else {
      ce_rows_kernel<T, true><<<grid, CE_THREADS, row_bytes, g_stream>>>(
          ptr<T>(logits), ptr<int32_t>(targets), ptr<T>(dlogits), (float *)row_loss,
          grad_out ? ptr<float>(grad_out) : nullptr, grad_scale, N, (int)V, ld, mode);
    }
  } else {
    ce_rows_kernel<T, false><<<grid, CE_THREADS, 0, g_stream>>>(
        ptr<T>(logits), ptr<int32_t>(targets), ptr<T>(dlogits), (float *)row_loss,
        grad_out ? ptr<float>(grad_out) : nullptr, grad_scale, N, (int)V, ld, mode);
  }
  if (mode & 1) {
    g_launches++;
    ce_mean_kernel<<<1, 1024, 0, g_stream>>>((const float *)row_loss, N, ptr<float>(loss_mean));
    pool_free(row_loss);
  }
  ALPHA_LAUNCHED();
  return 0;
}

}  // namespace alpha

using namespace alpha;

extern "C" {

int alpha_cross_entropy_fwd(alpha_buf logits, alpha_buf targets, alpha_buf loss_mean, int64_t N, int64_t V, int64_t ld,
                            int dtype) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(ld >= V, "alpha_cross_entropy_fwd: ld < V");
  if (dtype == ALPHA_F32) return ce_launch<float>(logits, targets, 0, loss_mean, 0, 1.f, N, V, ld, 1);
  if (dtype == ALPHA_BF16) return ce_launch<__nv_bfloat16>(logits, targets, 0, loss_mean, 0, 1.f, N, V, ld, 1);
  return set_error("alpha_cross_entropy_fwd: unsupported dtype %d", dtype);
}

int alpha_cross_entropy_bwd(alpha_buf logits, alpha_buf targets, alpha_buf grad_out_scalar, alpha_buf dlogits,
                            int64_t N, int64_t V, int64_t ld, int dtype) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(ld >= V, "alpha_cross_entropy_bwd: ld < V");
  if (dtype == ALPHA_F32) return ce_launch<float>(logits, targets, dlogits, 0, grad_out_scalar, 1.f, N, V, ld, 2);
  if (dtype == ALPHA_BF16)
    return ce_launch<__nv_bfloat16>(logits, targets, dlogits, 0, grad_out_scalar, 1.f, N, V, ld, 2);
  return set_error("alpha_cross_entropy_bwd: unsupported dtype %d", dtype);
}

int alpha_softmax_ce_fwd_bwd(alpha_buf logits, alpha_buf targets, alpha_buf dlogits, alpha_buf loss_mean, int64_t N,
                             int64_t V, int64_t ld, float grad_scale, int dtype) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(ld >= V, "alpha_softmax_ce_fwd_bwd: ld < V");
  if (dtype == ALPHA_F32) return ce_launch<float>(logits, targets, dlogits, loss_mean, 0, grad_scale, N, V, ld, 3);
  if (dtype == ALPHA_BF16)
    return ce_launch<__nv_bfloat16>(logits, targets, dlogits, loss_mean, 0, grad_scale, N, V, ld, 3);
  return set_error("alpha_softmax_ce_fwd_bwd: unsupported dtype %d", dtype);
}

}  // extern "C"

// ── cross-entropy forward without any allocation ─────────────────────────────
// For hosts that fix their device-memory budget at start-up and must not reach the CUDA
// allocator afterwards: an evaluation hook running beside a trainer that has already
// claimed the rest of HBM (a late cudaMalloc may fail there), or a latency-bound loop that
// forbids driver allocation calls once warm because cudaMalloc/cudaFree synchronise the
// device.  The per-row losses, which alpha_cross_entropy_fwd keeps in pool memory, live
// here in a fixed device array that is part of the library image: every GPU that loads the
// library carries these 256 KiB until the process exits.
namespace alpha {

constexpr int64_t CE_NOALLOC_MAX_ROWS = 65536;
static __device__ __align__(256) float g_ce_noalloc_row_loss[CE_NOALLOC_MAX_ROWS];

// In host code the array's name is only a handle for the runtime, not an address a kernel
// can use; the device address is looked up once per device, with that device current.
constexpr int CE_NOALLOC_MAX_DEVICES = 64;
static float *g_ce_noalloc_dev_ptr[CE_NOALLOC_MAX_DEVICES] = {nullptr};

static int ce_noalloc_scratch(float **out) {
  int dev = -1;
  ALPHA_CUDA(cudaGetDevice(&dev));
  // The launch goes to the library's stream, which lives on the device alpha_init chose.  A
  // host thread that never selected that device has device 0 current; resolving the symbol
  // there would quietly create a context (and load this library's image) on a GPU the
  // caller never asked for — an allocation this entry point promises not to make.
  ALPHA_CHECK(dev == g_device,
              "alpha_cross_entropy_fwd_noalloc: the calling thread's current device is %d but the library runs on "
              "device %d; call cudaSetDevice(%d) (or alpha_init) in this thread first",
              dev, g_device, g_device);
  ALPHA_CHECK(dev >= 0 && dev < CE_NOALLOC_MAX_DEVICES, "alpha_cross_entropy_fwd_noalloc: device ordinal %d out of range",
              dev);
  if (g_ce_noalloc_dev_ptr[dev] == nullptr) {
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_ce_noalloc_row_loss);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return set_error("alpha_cross_entropy_fwd_noalloc: cudaGetSymbolAddress -> %s", cudaGetErrorString(e));
    }
    g_ce_noalloc_dev_ptr[dev] = static_cast<float *>(p);
  }
  *out = g_ce_noalloc_dev_ptr[dev];
  return 0;
}

template <typename T>
static int ce_noalloc_launch(alpha_buf logits, alpha_buf targets, alpha_buf loss_mean, float *row_loss, int64_t N,
                             int64_t V, int64_t ld) {
  // Same row kernel as alpha_cross_entropy_fwd (loss only, rows re-read from L2 instead of
  // staged in shared memory), then the same fixed-order mean.  Rows [0, N) of the array are
  // written before they are read and nothing beyond N is read, so stale contents left by an
  // earlier call do not matter and nothing has to be cleared.
  ce_rows_kernel<T, false><<<grid_for(N, 1, 4), CE_THREADS, 0, g_stream>>>(
      ptr<T>(logits), ptr<int32_t>(targets), nullptr, row_loss, nullptr, 1.f, N, (int)V, ld, 1);
  g_launches++;
  ce_mean_kernel<<<1, 1024, 0, g_stream>>>(row_loss, N, ptr<float>(loss_mean));
  ALPHA_LAUNCHED();
  return 0;
}

}  // namespace alpha

extern "C" int alpha_cross_entropy_fwd_noalloc(alpha_buf logits, alpha_buf targets, alpha_buf loss_mean, int64_t N,
                                               int64_t V, int64_t ld, int dtype) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(ld >= V, "alpha_cross_entropy_fwd_noalloc: ld < V");
  ALPHA_CHECK(N >= 0 && V >= 0 && V < (1ll << 31), "alpha_cross_entropy_fwd_noalloc: bad sizes");
  ALPHA_CHECK(N <= CE_NOALLOC_MAX_ROWS,
              "alpha_cross_entropy_fwd_noalloc: N = %lld rows exceeds the fixed scratch of %lld rows; "
              "use alpha_cross_entropy_fwd or split the batch",
              (long long)N, (long long)CE_NOALLOC_MAX_ROWS);
  ALPHA_CHECK(dtype == ALPHA_F32 || dtype == ALPHA_BF16, "alpha_cross_entropy_fwd_noalloc: unsupported dtype %d", dtype);
  if (N == 0 || V == 0) {
    ALPHA_CUDA(cudaMemsetAsync(ptr<void>(loss_mean), 0, 4, g_stream));
    return 0;
  }
  float *row_loss = nullptr;
  if (ce_noalloc_scratch(&row_loss)) return 1;  // first call on a device: resolves the array's address
  if (dtype == ALPHA_F32) return ce_noalloc_launch<float>(logits, targets, loss_mean, row_loss, N, V, ld);
  return ce_noalloc_launch<__nv_bfloat16>(logits, targets, loss_mean, row_loss, N, V, ld);
}
