// Shared helpers of libalpha_cuda.so: error convention, the compute stream, launch
// accounting, storage-type loads/stores and warp/block reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/alpha_cuda.h"

namespace alpha {

// ── global state (runtime.cu) ───────────────────────────────────────────────
extern cudaStream_t g_stream;
extern int g_device;
extern int g_sm_count;
extern bool g_inited;
// Counts alpha_init calls.  Per-device set-up that a launch site does on first use (function
// attributes, device scratch) is remembered as "done in epoch N", so that it is repeated
// after alpha_shutdown + alpha_init, which may select another GPU.
extern int g_init_epoch;
extern unsigned long long g_launches;

int set_error(const char *fmt, ...);
// Scratch from the caching pool (runtime.cu); returned with pool_free.
int pool_alloc(size_t bytes, void **out);
void rope_tables_clear();  // rope.cu: frees the cos/sin tables (shutdown)
namespace tc { void tc_error_word_free(); }  // tc_host.cu: frees the bounded-wait error word (shutdown)
int pool_free(void *p);
// Device-resident copy of a small host table (pointer/size tables of the multi-tensor
// kernels).  Tables are cached by content, so a training loop that passes the same
// tensors every step uploads its table once and never synchronises the host afterwards.
int table_upload(const void *host, size_t bytes, const void **dev);

// Per-kernel-family timing (alpha_profile_*): when enabled, the launch sites of the heavy
// kernels bracket themselves with CUDA events on the compute stream.
enum ProfCat { PROF_GEMM_TC = 0, PROF_GEMM_F32 = 1, PROF_ATTN_FWD = 2, PROF_ATTN_BWD = 3, PROF_CE = 4,
               PROF_ADAMW = 5, PROF_NORM = 6, PROF_EMBED = 7, PROF_ELEMENTWISE = 8, PROF_NCAT = 9 };
extern bool g_profiling;
void prof_begin(int cat, double work);
void prof_end(int cat);
void range_begin(int cat);  // NVTX range named after the kernel family (no-op without a tool attached)
void range_end();
struct ProfScope {
  int cat;
  bool on;
  ProfScope(int c, double work) : cat(c), on(g_profiling) {
    range_begin(c);
    if (on) prof_begin(c, work);
  }
  ~ProfScope() {
    if (on) prof_end(cat);
    range_end();
  }
};

#define ALPHA_REQUIRE_INIT()                                                 \
  do {                                                                         \
    if (!alpha::g_inited) return alpha::set_error("%s: alpha_init was not called", __func__); \
  } while (0)

#define ALPHA_CHECK(cond, ...)                                \
  do {                                                        \
    if (!(cond)) return alpha::set_error(__VA_ARGS__);        \
  } while (0)

#define ALPHA_CUDA(call)                                                                    \
  do {                                                                                      \
    cudaError_t e_ = (call);                                                                \
    if (e_ != cudaSuccess)                                                                  \
      return alpha::set_error("%s:%d %s -> %s", __FILE__, __LINE__, #call, cudaGetErrorString(e_)); \
  } while (0)

// Counts one launch and reports a launch-configuration error, if any.
#define ALPHA_LAUNCHED()                                                                    \
  do {                                                                                      \
    alpha::g_launches++;                                                                    \
    cudaError_t e_ = cudaPeekAtLastError();                                                 \
    if (e_ != cudaSuccess) {                                                                \
      cudaGetLastError();                                                                   \
      return alpha::set_error("%s:%d kernel launch -> %s", __FILE__, __LINE__, cudaGetErrorString(e_)); \
    }                                                                                       \
  } while (0)

// Launch that may overlap the tail of its predecessor in the stream (programmatic dependent
// launch): the kernel's blocks can become resident and run their set-up (barriers, tensor
// memory, shared-memory tables) while the previous kernel drains.  Such a kernel executes
// grid_dependency_wait() before its first access to global memory, which returns once the
// previous kernel has finished and its writes are visible, and grid_dependency_trigger()
// as early as it likes to give its own successor the same head start.
extern int g_overlap_launches;  // bit mask of kernel families (OVL_*) launched this way
// Number of coming launches to serialise fully: a collective that has just been queued on the
// side stream needs one ordinary kernel boundary, with idle SMs, to get its blocks resident.
extern int g_overlap_hold;
enum { OVL_GEMM = 1, OVL_SPLITK = 2, OVL_ATTN_FWD = 4, OVL_ATTN_BWD = 8, OVL_NORM_FWD = 16, OVL_NORM_BWD = 32 };
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(int family, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     Args &&...args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = g_stream;
  cudaLaunchAttribute at;
  memset(&at, 0, sizeof(at));
  at.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at.val.programmaticStreamSerializationAllowed = ((g_overlap_launches & family) && g_overlap_hold == 0) ? 1 : 0;
  if (g_overlap_hold > 0) g_overlap_hold--;
  cfg.attrs = &at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

template <typename T>
__host__ __device__ inline T *ptr(alpha_buf b) {
  return reinterpret_cast<T *>(static_cast<uintptr_t>(b));
}

inline size_t dtype_size(int dt) { return dt == ALPHA_BF16 ? 2 : 4; }

inline int grid_for(int64_t work_items, int per_block, int max_blocks_per_sm = 8) {
  int64_t b = (work_items + per_block - 1) / per_block;
  int64_t cap = (int64_t)g_sm_count * max_blocks_per_sm;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

// ── storage-type conversion ─────────────────────────────────────────────────
__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

// 16-byte vector of storage elements: 4 floats or 8 bf16.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ void load(const float *p) { raw = *reinterpret_cast<const float4 *>(p); }
  __device__ __forceinline__ void store(float *p) const { *reinterpret_cast<float4 *>(p) = raw; }
  __device__ __forceinline__ void get(float *f) const { f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w; }
  __device__ __forceinline__ void set(const float *f) { raw = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ void load(const __nv_bfloat16 *p) { raw = *reinterpret_cast<const uint4 *>(p); }
  __device__ __forceinline__ void store(__nv_bfloat16 *p) const { *reinterpret_cast<uint4 *>(p) = raw; }
  __device__ __forceinline__ void get(float *f) const {
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ __forceinline__ void set(const float *f) {
    __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  }
};

__device__ __forceinline__ bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ── reductions ──────────────────────────────────────────────────────────────
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; every thread gets the result. `red` is >= 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float *red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float *red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

// Activation math shared by the elementwise kernels and the GEMM epilogues.
// GELU: tanh approximation (packages/tensor/src/cpu_ref.ts:422-427) and its derivative
// (packages/autograd/src/ops.ts:404-418).
__device__ __forceinline__ float gelu_f(float x) {
  const float c = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanhf(c * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float c = 0.7978845608028654f;
  const float t = tanhf(c * (x + 0.044715f * x * x * x));
  const float sech2 = 1.f - t * t;
  const float d_inner = c * (1.f + 3.f * 0.044715f * x * x);
  return 0.5f * (1.f + t) + 0.5f * x * sech2 * d_inner;
}

}  // namespace alpha
