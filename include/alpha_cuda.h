/*
 * libalpha_cuda.so — C ABI of the B200 (sm_100a) compute backend for alpha's GPT train step.
 *
 * This is the boundary a host binds with FFI (bun:ffi / Node FFI / ctypes): plain
 * pointers, sizes and scalars, no C++ or torch types.  It replaces, for the train-step
 * path, what the reference reaches through its N-API Vulkan bridge
 * (packages/helios/native/helios_vk.c:4403-4432: initDevice, createBuffer, uploadBuffer,
 * readBuffer, destroyBuffer, dispatch, waitIdle, gpuTime, ...) and gives one entry point
 * per method of the reference's Backend interface (packages/core/src/interfaces.ts:38-151)
 * that the step uses.
 *
 * Conventions
 *  - Every function returns 0 on success and a non-zero status otherwise;
 *    alpha_last_error() then returns a message (the reference throws JS exceptions /
 *    napi_throw_error strings, helios_vk.c throughout).  There is no CPU fallback.
 *  - A device buffer is named by an `alpha_buf` (the device address as a 64-bit integer).
 *  - All work is enqueued on one compute stream owned by the library; calls return
 *    without waiting unless stated.  Host reads (alpha_d2h) wait for prior work.
 *  - Tensors are row-major and contiguous unless a leading dimension / stride is passed.
 *  - dtype codes: ALPHA_F32, ALPHA_BF16, ALPHA_I32.  Arithmetic is fp32 whatever the
 *    storage type; GEMM and attention accumulate in fp32.
 */
#ifndef ALPHA_CUDA_H
#define ALPHA_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint64_t alpha_buf;

enum { ALPHA_F32 = 0, ALPHA_BF16 = 1, ALPHA_I32 = 2 };

/* ── runtime ─────────────────────────────────────────────────────────────────────────
 * Replaces helios_vk.c initDevice / destroy / waitIdle / gpuTime (:4403-4432) and the
 * backend's getDeviceInfo() (packages/helios/src/backend.ts, probed by
 * apps/cli/src/commands/train.ts:284-318; vendorId must read 0x10de). */
typedef struct {
  char name[128];
  int32_t vendor_id;          /* 0x10de */
  int32_t sm_count;
  int32_t cc_major, cc_minor;
  uint64_t total_mem;
  uint64_t l2_bytes;
} alpha_device_info_t;

int alpha_init(int device_ordinal);
int alpha_shutdown(void);
const char *alpha_last_error(void);
int alpha_device_info(alpha_device_info_t *out);
int alpha_stream_sync(void);
/* Number of kernels this library has launched since alpha_init (all entry points). */
int alpha_launch_count(uint64_t *out);
/* Raw cudaStream_t of the compute stream (for hosts that want to time with their own events). */
int alpha_stream_handle(uint64_t *out);
/* Waits for all enqueued work, then reports (non-zero + message) if a tensor-core kernel
 * abandoned one of its bounded waits since the last check; such a kernel's output is
 * invalid.  Waits inside the kernels never spin without limit. */
int alpha_check_async_error(void);
/* Test hook for the give-up path of those waits (no reference counterpart): launches, on
 * `blocks` SMs, a kernel with the GEMM's role structure and tensor-memory allocation in which
 * the producer waits on a barrier that nothing signals, with a limit of `limit_us`
 * microseconds (1..100000) instead of the production limit of about a second.  The wait runs
 * out, every role unwinds, tensor memory is freed and the error word is set; nothing faults
 * and the kernel returns by itself.  *roles_left_out = number of warps that left through the
 * give-up path (6 per block).  The next alpha_check_async_error() reports the expiry. */
int alpha_debug_wait_expiry(int blocks, int limit_us, int *roles_left_out);

/* The tensor-core GEMM, attention and norm kernels are launched so that their blocks may
 * become resident and set themselves up while the previous kernel of the stream drains
 * (programmatic dependent launch; each waits for its predecessor before it touches global
 * memory).  families is a bit mask: 1 GEMM, 2 split-K reduce, 4 attention forward,
 * 8 attention backward, 16 norm forward, 32 norm backward; -1 = all (the default),
 * 0 = fully serialised launches (for timing comparisons and fault isolation). */
int alpha_set_launch_overlap(int families);

/* Per-kernel-family device timing (helios_vk.c:3448 gpuTime; backend.ts:5159-5204 profileOp).
 * While enabled, launches of the heavy kernel families are bracketed by events on the
 * compute stream; alpha_profile_read waits, then returns per family the summed device time,
 * the algorithmic work the launches declared (flop for GEMM/attention, bytes for the
 * HBM-bound families) and the launch count, and clears the records.
 * Families: 0 tensor-core GEMM, 1 fp32 GEMM, 2 attention fwd, 3 attention bwd,
 * 4 cross-entropy, 5 AdamW, 6 norms, 7 embedding, 8 elementwise / RoPE (work = elements). */
typedef struct {
  double ms;
  double work;
  int64_t launches;
} alpha_profile_entry_t;
enum { ALPHA_PROFILE_CATEGORIES = 9 };
int alpha_profile_enable(int on);
int alpha_profile_read(alpha_profile_entry_t *out, int n_categories);
/* NVTX ranges for timeline tools: every launch site of the families above opens a range named
 * after its family; a host brackets its own phases (forward, backward, optimizer — the
 * reference times the same phases with host clocks, packages/train/src/trainer.ts:1189-1264)
 * with these two.  Without a tool attached they cost a null-pointer check. */
int alpha_range_push(const char *name);
int alpha_range_pop(void);

/* Events: helios_vk.c gpuTime / waitTimeline / getCompleted (:4403-4432). */
int alpha_event_create(uint64_t *ev);
int alpha_event_record(uint64_t ev);
int alpha_event_sync(uint64_t ev);
int alpha_event_elapsed_ms(uint64_t ev_start, uint64_t ev_end, float *ms);
int alpha_event_destroy(uint64_t ev);

/* ── memory ──────────────────────────────────────────────────────────────────────────
 * Replaces createBuffer / destroyBuffer / uploadBuffer / fillBuffer / readBuffer
 * (helios_vk.c:4403-4432) and the backend's releaseGpuTensor / purgeBufferPools /
 * gpuMemStats (packages/helios/src/backend.ts:688-699; packages/train/src/trainer.ts:998-1044).
 * alpha_alloc serves from a caching pool (freed blocks are reused without cudaMalloc). */
typedef struct {
  uint64_t bytes_in_use;      /* handed out and not yet freed */
  uint64_t bytes_cached;      /* held in the pool, free for reuse */
  uint64_t peak_in_use;
  uint64_t n_device_mallocs;  /* cudaMalloc calls so far */
  uint64_t n_allocs;          /* alpha_alloc calls so far */
} alpha_mem_stats_t;

int alpha_alloc(size_t bytes, alpha_buf *out);
int alpha_free(alpha_buf buf);
int alpha_mem_stats(alpha_mem_stats_t *out);
int alpha_purge_pools(void);
int alpha_memset(alpha_buf dst, int byte_value, size_t bytes);
int alpha_h2d(alpha_buf dst, const void *host_src, size_t bytes);   /* async if host_src is pinned */
int alpha_d2h(void *host_dst, alpha_buf src, size_t bytes);         /* waits for the copy */
/* Enqueue only: host_dst is pinned memory, valid after an event recorded behind the call
 * has completed.  Lets a host read the result of step i while step i+1 is already queued
 * (the reference's trainer reads its loss synchronously, trainer.ts:1247). */
int alpha_d2h_async(void *host_dst, alpha_buf src, size_t bytes);
int alpha_d2d(alpha_buf dst, alpha_buf src, size_t bytes);
int alpha_host_alloc(size_t bytes, void **out);                     /* pinned host memory */
int alpha_host_free(void *p);

/* ── creation / elementwise ──────────────────────────────────────────────────────────
 * Backend.zeros/ones/full (interfaces.ts:42-46), add/sub/mul/div (:49-52), neg/exp/log/
 * sqrt/pow/scale/clamp (:58-64), gelu/relu/silu (:69-71), the optional backward hooks
 * geluBackward/reluBackward/siluBackward/clampBackward/softCap/softCapBackward
 * (:96-107), addInplace/scaleInplace (:113-114), castDtype (:141), siluMul(+Backward)
 * (:99-100), broadcast (:138). */
enum { ALPHA_ADD = 0, ALPHA_SUB = 1, ALPHA_MUL = 2, ALPHA_DIV = 3 };
enum {
  ALPHA_NEG = 0, ALPHA_EXP = 1, ALPHA_LOG = 2, ALPHA_SQRT = 3, ALPHA_RELU = 4, ALPHA_SILU = 5,
  ALPHA_GELU = 6, ALPHA_SCALE = 7, ALPHA_CLAMP = 8, ALPHA_POW = 9, ALPHA_SOFTCAP = 10
};

int alpha_fill(alpha_buf dst, int64_t n, float value, int dtype);
int alpha_binary(int op, alpha_buf a, alpha_buf b, alpha_buf out, int64_t n, int dtype);
/* out[idx] = a[idx . a_strides] op b[idx . b_strides]; element strides, 0 = broadcast; ndim <= 6 */
int alpha_binary_bcast(int op, alpha_buf a, alpha_buf b, alpha_buf out, int ndim,
                       const int64_t *out_shape, const int64_t *a_strides,
                       const int64_t *b_strides, int dtype);
int alpha_unary(int op, alpha_buf a, alpha_buf out, int64_t n, float p0, float p1, int dtype);
/* out = g * d(op)/dx at x; ops: RELU, SILU, GELU, CLAMP(p0,p1), SOFTCAP(p0) */
int alpha_unary_bwd(int op, alpha_buf x, alpha_buf g, alpha_buf out, int64_t n, float p0,
                    float p1, int dtype);
int alpha_add_inplace(alpha_buf a, alpha_buf b, int64_t n, int a_dtype, int b_dtype);
int alpha_scale_inplace(alpha_buf a, float s, int64_t n, int dtype);
int alpha_cast(alpha_buf src, int src_dtype, alpha_buf dst, int dst_dtype, int64_t n);
int alpha_silu_mul_fwd(alpha_buf a, alpha_buf b, alpha_buf out, int64_t n, int dtype);
int alpha_silu_mul_bwd(alpha_buf a, alpha_buf b, alpha_buf g, alpha_buf da, alpha_buf db,
                       int64_t n, int dtype);
int alpha_broadcast(alpha_buf a, alpha_buf out, int ndim, const int64_t *out_shape,
                    const int64_t *a_strides, int dtype);

/* ── reductions / softmax ────────────────────────────────────────────────────────────
 * Backend.sum/mean (interfaces.ts:54-55), softmax/logSoftmax (:72-73), sumOfSquares /
 * totalSumOfSquares / checkFinite (:144-146; packages/train/src/trainer.ts:1314-1375,
 * 1689-1712).  a is viewed as [outer, dim, inner]; out is [outer, inner]. */
int alpha_sum_axis(alpha_buf a, alpha_buf out, int64_t outer, int64_t dim, int64_t inner,
                   float scale, int dtype);
int alpha_softmax(alpha_buf a, alpha_buf out, int64_t rows, int64_t cols, int log_mode, int dtype);
/* out_scalar (f32[1]) = sum over all listed tensors of sum(x^2); one launch pair. */
int alpha_sumsq_multi(const alpha_buf *tensors, const int64_t *counts, const int32_t *dtypes,
                      int n_tensors, alpha_buf out_scalar);
/* out_scalar (f32[1]) = number of non-finite elements */
int alpha_check_finite(alpha_buf a, int64_t n, int dtype, alpha_buf out_scalar);

/* ── layout ops ──────────────────────────────────────────────────────────────────────
 * Backend.transpose / slice (interfaces.ts:77-78), sliceQkv / scatterSlice (:117-121),
 * causalMask / maskedFill (:91-92), dropoutMask / residualDropoutAdd (:110,125). */
int alpha_transpose(alpha_buf a, alpha_buf out, int ndim, const int64_t *shape, int d0, int d1,
                    int dtype);
int alpha_slice_cols(alpha_buf a, alpha_buf out, int64_t rows, int64_t cols, int64_t c0,
                     int64_t c1, int dtype);                           /* out[r, :] = a[r, c0:c1] */
int alpha_scatter_cols(alpha_buf g, alpha_buf out, int64_t rows, int64_t cols, int64_t c0,
                       int64_t c1, int dtype);                         /* zero elsewhere */
int alpha_slice_qkv(alpha_buf a, alpha_buf q, alpha_buf k, alpha_buf v, int64_t rows, int64_t d,
                    int dtype);
int alpha_causal_mask(alpha_buf out, int64_t size);                   /* f32: 0 / -inf */
int alpha_masked_fill(alpha_buf a, alpha_buf mask, alpha_buf out, int64_t n, int64_t mask_n,
                      float value, int dtype);
int alpha_dropout_mask(alpha_buf out, int64_t n, int32_t seed, int32_t counter, float p, int dtype);
int alpha_residual_dropout_add(alpha_buf residual, alpha_buf projected, alpha_buf mask,
                               alpha_buf out, int64_t n, int dtype);

/* ── embedding ───────────────────────────────────────────────────────────────────────
 * Backend.embedding (interfaces.ts:67; cpu_ref.ts:364-385) and embeddingBackward (:105;
 * packages/autograd/src/ops.ts:495-505).  The gather is a bit-exact copy.  The backward is
 * a deterministic scatter-add: each output row is owned by one warp that adds the
 * gradient rows naming it in index order, fp32 — the order of the reference's CPU loop.
 * dw is f32 [vocab, dim] and is fully written (rows nobody names become 0). */
int alpha_embedding_fwd(alpha_buf weight, alpha_buf indices, alpha_buf out, int64_t n_idx,
                        int64_t dim, int64_t vocab, int dtype);
/* out[b,t,:] = wte[tok[b,t],:] + wpe[t,:] in one pass (gpt.ts:362-379) */
int alpha_embedding_pos_fwd(alpha_buf wte, alpha_buf wpe, alpha_buf tokens, alpha_buf out,
                            int64_t batch, int64_t T, int64_t dim, int64_t vocab, int dtype);
int alpha_embedding_bwd(alpha_buf indices, alpha_buf grad, alpha_buf dw, int64_t n_idx,
                        int64_t dim, int64_t vocab, int grad_dtype, int accumulate);

/* ── normalisation ───────────────────────────────────────────────────────────────────
 * Backend.layerNorm (interfaces.ts:68; cpu_ref.ts:387-420) and layerNormBackward (:103;
 * ops.ts:523-569).  dw/db are f32 [dim].  RMSNorm has no reference counterpart (it is
 * asked for by the 350M configuration): y = x * rsqrt(mean(x^2)+eps) * w. */
int alpha_layernorm_fwd(alpha_buf x, alpha_buf w, alpha_buf b, alpha_buf y, int64_t rows,
                        int64_t dim, float eps, int dtype);
/* dx_add: 0, or a tensor shaped like x that is added to the result (dx = dx_add + ...; dx may
 * alias dx_add) — the residual stream's gradient is accumulated in the same pass instead of
 * by a separate addInplace (packages/autograd/src/tape.ts:116-127 does the latter). */
int alpha_layernorm_bwd(alpha_buf x, alpha_buf w, alpha_buf g, alpha_buf dx, alpha_buf dw,
                        alpha_buf db, int64_t rows, int64_t dim, float eps, int dtype,
                        int accumulate_dwdb, alpha_buf dx_add);
int alpha_rmsnorm_fwd(alpha_buf x, alpha_buf w, alpha_buf y, int64_t rows, int64_t dim,
                      float eps, int dtype);
int alpha_rmsnorm_bwd(alpha_buf x, alpha_buf w, alpha_buf g, alpha_buf dx, alpha_buf dw,
                      int64_t rows, int64_t dim, float eps, int dtype, int accumulate_dw,
                      alpha_buf dx_add);

/* ── GEMM ────────────────────────────────────────────────────────────────────────────
 * Backend.matmul (interfaces.ts:53; cpu_ref.ts:166-258), matmulTransposed (:111) and
 * matmulTransposedA (:112); the GELU-fused forward is packages/autograd/src/ops.ts:426-487.
 *   ALPHA_GEMM_NT: C[M,N] = A[M,K] * B[N,K]^T      (forward  x W^T)
 *   ALPHA_GEMM_NN: C[M,N] = A[M,K] * B[K,N]        (dX = G W)
 *   ALPHA_GEMM_TN: C[M,N] = A[K,M]^T * B[K,N]      (dW = G^T X)
 * lda/ldb/ldc/ld_aux are leading dimensions in elements.  in_dtype BF16 runs on the
 * tcgen05 tensor cores (fp32 accumulate in tensor memory); in_dtype F32 runs an fp32 FMA
 * kernel (the fp32 parity mode).  batch > 1 (fp32 only) walks strides in elements.
 * Epilogues:
 *   ALPHA_EPI_NONE      C = acc
 *   ALPHA_EPI_GELU      aux = acc (pre-activation, out dtype), C = gelu(acc)
 *   ALPHA_EPI_ADD       C = acc + aux                     (residual add)
 *   ALPHA_EPI_GELU_BWD  C = acc * gelu'(aux)              (aux = saved pre-activation)
 * accumulate != 0 adds the result to what C already holds (gradient accumulation). */
enum { ALPHA_GEMM_NT = 0, ALPHA_GEMM_NN = 1, ALPHA_GEMM_TN = 2 };
enum { ALPHA_EPI_NONE = 0, ALPHA_EPI_GELU = 1, ALPHA_EPI_ADD = 2, ALPHA_EPI_GELU_BWD = 3 };

int alpha_gemm(int layout, alpha_buf A, alpha_buf B, alpha_buf C, int64_t M, int64_t N, int64_t K,
               int64_t lda, int64_t ldb, int64_t ldc, int in_dtype, int out_dtype, int epilogue,
               alpha_buf aux, int64_t ld_aux, int accumulate);
/* C = A B (NN, bf16 in and out, N = heads * 64) whose epilogue also writes, for every row and
 * head, delta[(row / T) * heads + h][row % T] = sum_d C[row, 64h + d] * O[row, 64h + d] with C as
 * rounded to bf16: the gradient of the attention output (dO = G Wo) together with the row-dots
 * attention's backward needs, in one launch (packages/helios/src/kernels/attention.ts:1217-1231
 * computes them in a pass of their own).  O has leading dimension ld_o; delta is f32. */
int alpha_gemm_nn_rowdot(alpha_buf A, alpha_buf B, alpha_buf C, int64_t M, int64_t N, int64_t K,
                         int64_t lda, int64_t ldb, int64_t ldc, alpha_buf O, int64_t ld_o,
                         alpha_buf delta, int64_t T, int64_t heads);
/* Two weight gradients in one launch: C_i (+)= A_i^T B_i for i = 0, 1 with A_i [K, M_i] and
 * B_i [K, N_i] bf16, C_i f32, both over the same K (accumulate_i != 0: added to what C_i holds).
 * The reference computes every weight gradient with a matmul of its own (packages/autograd/src/
 * ops.ts:200-234); two that would each fill half of the device share a launch here and need no
 * split over K.  A pair that does not qualify (shapes, alignment) runs as two alpha_gemm calls. */
int alpha_gemm_tn_pair(alpha_buf A0, alpha_buf B0, alpha_buf C0, int64_t M0, int64_t N0, int64_t lda0,
                       int64_t ldb0, int64_t ldc0, int accumulate0, alpha_buf A1, alpha_buf B1,
                       alpha_buf C1, int64_t M1, int64_t N1, int64_t lda1, int64_t ldb1, int64_t ldc1,
                       int accumulate1, int64_t K);
int alpha_gemm_batched_f32(int layout, alpha_buf A, alpha_buf B, alpha_buf C, int64_t M, int64_t N,
                           int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t batch,
                           int64_t stride_a, int64_t stride_b, int64_t stride_c);

/* ── attention ───────────────────────────────────────────────────────────────────────
 * Backend.flashAttention / flashAttentionBackward (interfaces.ts:127-135; semantics of
 * packages/helios/src/kernels/attention.ts:427-477,552-558 forward and :1217-1231,
 * 1411-1427 backward): s = scale * q.k, optional soft cap tanh(s/cap)*cap (cap <= 0
 * disables), causal mask, softmax, O = P V, LSE = max + ln(sum).
 * Element (b, h, t, d) of q lives at q + b*q_sb + h*q_sh + t*q_st + d (element strides;
 * the same strides apply to k, v and their gradients; o/do use o_sb/o_sh/o_st).  With
 * q_sb=H*T*D, q_sh=T*D, q_st=D this is the reference's [B*H, T, D] contract; with
 * q_sb=T*3E, q_sh=D, q_st=3E the kernel reads q/k/v in place from the fused QKV GEMM
 * output and no head-split or head-merge copies exist.  lse is f32 [B, H, T]. */
typedef struct {
  int64_t batch, heads, T, D;
  int64_t q_sb, q_sh, q_st;
  int64_t o_sb, o_sh, o_st;
  float scale, soft_cap;
  int32_t dtype;
} alpha_attn_params_t;

int alpha_flash_attn_fwd(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf o, alpha_buf lse,
                         const alpha_attn_params_t *p);
int alpha_flash_attn_bwd(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf o, alpha_buf d_o,
                         alpha_buf lse, alpha_buf dq, alpha_buf dk, alpha_buf dv,
                         const alpha_attn_params_t *p);

/* The same backward when the caller already has delta[b, h, t] = sum_d dO*O (f32 [batch, heads,
 * T]): the forward output is not read.  bf16 with head dim 64 only (the tensor-core kernels);
 * anything else is refused and alpha_flash_attn_bwd should be called.  No reference counterpart:
 * it pairs with alpha_gemm_nn_rowdot, which produces dO and delta in one GEMM. */
int alpha_flash_attn_bwd_delta(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf d_o, alpha_buf lse,
                               alpha_buf delta, alpha_buf dq, alpha_buf dk, alpha_buf dv,
                               const alpha_attn_params_t *p);

/* RoPE (no reference counterpart; asked for by the 350M configuration): rotate-half
 * convention on x[rows=B*T, heads, D] with row stride ld, angle(t,i) = t * theta^(-2i/D);
 * inverse != 0 applies the transposed rotation (the backward). In place when x == out. */
int alpha_rope(alpha_buf x, alpha_buf out, int64_t batch, int64_t T, int64_t heads, int64_t D,
               int64_t ld, float theta, int inverse, int dtype);
/* The same rotation on the q and k column blocks of a fused activation qkv [B*T, 3*heads*D],
 * written with the v block copied alongside to out (same layout; out may equal qkv), one read
 * and one write of every row. */
int alpha_rope_qkv(alpha_buf qkv, alpha_buf out, int64_t batch, int64_t T, int64_t heads, int64_t D,
                   float theta, int inverse, int dtype);

/* ── loss ────────────────────────────────────────────────────────────────────────────
 * Backend.crossEntropy (interfaces.ts:74; cpu_ref.ts:543-563) and crossEntropyBackward
 * (:104; ops.ts:702-729).  logits is [N, V] with leading dimension ld.
 * alpha_softmax_ce_fwd_bwd does both in one pass over each row: loss_mean (f32[1]) gets
 * the mean loss and dlogits gets (softmax - onehot) * grad_scale / N (dlogits may alias
 * logits).  No host synchronisation (the reference's helios path reads back twice,
 * packages/helios/src/backend.ts:2704,4511-4515). */
int alpha_cross_entropy_fwd(alpha_buf logits, alpha_buf targets, alpha_buf loss_mean, int64_t N,
                            int64_t V, int64_t ld, int dtype);
int alpha_cross_entropy_bwd(alpha_buf logits, alpha_buf targets, alpha_buf grad_out_scalar,
                            alpha_buf dlogits, int64_t N, int64_t V, int64_t ld, int dtype);
int alpha_softmax_ce_fwd_bwd(alpha_buf logits, alpha_buf targets, alpha_buf dlogits,
                             alpha_buf loss_mean, int64_t N, int64_t V, int64_t ld,
                             float grad_scale, int dtype);
/* This entry has no counterpart in the reference.  It computes what
 * alpha_cross_entropy_fwd computes — loss_mean (f32[1]) = mean over rows of
 * (logsumexp(row) - row[target]) — but never allocates: no cudaMalloc/cudaFree, no pool
 * memory.  It is meant for hosts that settle their device-memory budget at start-up and may
 * not touch the CUDA allocator later: a loss-evaluation hook next to a trainer that already
 * owns the rest of HBM (where a late cudaMalloc can simply fail), or a latency-bound loop
 * that bans driver allocation calls after warm-up because they synchronise the device.
 * The per-row losses go to a fixed array inside the library image (65536 floats = 256 KiB,
 * held by every GPU that loads the library until the process exits), so N must be
 * <= 65536; larger N is rejected with an error, nothing is computed.  The caller still
 * provides logits, targets and loss_mean.  The first call on a device looks up the array's
 * device address (a one-off set-up): make that first call before starting any stream
 * capture.  All calls share the one array and it keeps whatever the previous call left;
 * that is harmless for consecutive calls (rows [0, N) are rewritten before they are read),
 * but two calls whose kernels overlap on the GPU — other streams, other host threads
 * driving their own work — race on it and must be serialised by the caller. */
int alpha_cross_entropy_fwd_noalloc(alpha_buf logits, alpha_buf targets, alpha_buf loss_mean,
                                    int64_t N, int64_t V, int64_t ld, int dtype);

/* ── optimizer ───────────────────────────────────────────────────────────────────────
 * Backend.adamwStep (interfaces.ts:149-150; packages/train/src/optimizers.ts:84-92):
 *   g = grad*gradScale; if wd>0: p -= lr*wd*p; m = b1 m + (1-b1) g; v = b2 v + (1-b2) g^2;
 *   p -= lr*(m/bc1)/(sqrt(v/bc2)+eps).
 * p, m, v are f32; grad is f32 or bf16; p_shadow (0 or a bf16 buffer) receives the
 * rounded copy of the new p.  alpha_adamw_multi updates many tensors in one launch.
 * If clip_sumsq != 0 the kernel derives the clip coefficient on the device:
 * gnorm = sqrt(*clip_sumsq)*|grad_scale|, coef = gnorm > max_norm ? max_norm/gnorm : 1
 * (packages/train/src/trainer.ts:1650-1656), so no host read sits between the norm and
 * the update. */
typedef struct {
  alpha_buf p, g, m, v, p_shadow;
  int64_t n;
  float weight_decay;
  int32_t grad_dtype;
} alpha_adamw_tensor_t;

int alpha_adamw(alpha_buf p, alpha_buf g, alpha_buf m, alpha_buf v, int64_t n, float lr, float beta1,
                float beta2, float eps, float weight_decay, float bc1, float bc2, float grad_scale,
                int grad_dtype, alpha_buf p_shadow);
int alpha_adamw_multi(const alpha_adamw_tensor_t *tensors, int n_tensors, float lr, float beta1,
                      float beta2, float eps, float bc1, float bc2, float grad_scale,
                      alpha_buf clip_sumsq, float max_norm);

/* ── host-side seeded generator ──────────────────────────────────────────────────────
 * SeededRng of packages/core/src/rng.ts:6-68 (xorshift128+, polar Gaussian with a cached
 * spare) and the weight fill of packages/model/src/gpt.ts:53-58, so that a model created
 * through this library starts from the reference's weights for the same seed.  Pure host
 * code; usable before alpha_init. */
typedef struct {
  uint32_t s0, s1;
  int32_t has_spare;
  double spare;
} alpha_host_rng_t;

int alpha_rng_seed(alpha_host_rng_t *r, uint32_t seed);
double alpha_rng_next(alpha_host_rng_t *r);                     /* uniform in [0, 1) */
double alpha_rng_gauss(alpha_host_rng_t *r);
int alpha_rng_fill_gauss(alpha_host_rng_t *r, float *host_out, int64_t n, double std);

/* ── data parallel ───────────────────────────────────────────────────────────────────
 * No reference counterpart (the reference is single-device, docs/scale.md:3).  One
 * process per GPU; gradients are summed across ranks with NCCL on a side stream that is
 * ordered after the compute stream by an event at enqueue time; alpha_comm_wait orders
 * the compute stream after all collectives enqueued so far. */
int alpha_comm_unique_id(void *out_128_bytes);
int alpha_comm_init_rank(int n_ranks, int rank, const void *unique_id_128_bytes);
int alpha_comm_allreduce_sum(alpha_buf buf, int64_t n, int dtype);
/* A bucket of gradient tensors (same dtype) reduced as one NCCL group = one collective launch. */
int alpha_comm_allreduce_sum_bucket(const alpha_buf *bufs, const int64_t *counts, int n_bufs, int dtype);
int alpha_comm_wait(void);
int alpha_comm_destroy(void);
/* Failure handling of the exchange (host side; no reference counterpart).  alpha_comm_query
 * never blocks: *pending = 1 while collectives enqueued so far are unfinished, *async_error =
 * NCCL's asynchronous error code of the communicator (0 = none).  alpha_comm_abort ends the
 * communicator with ncclCommAbort, which releases collectives that wait for a peer that will
 * never come; the step in flight must be discarded. */
int alpha_comm_query(int *pending, int *async_error);
int alpha_comm_abort(void);

#ifdef __cplusplus
}
#endif
#endif /* ALPHA_CUDA_H */
