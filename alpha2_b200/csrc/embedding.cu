// Embedding gather and its deterministic scatter-add backward.
//
// Reference semantics: packages/tensor/src/cpu_ref.ts:364-385 (out[i,:] = W[idx[i],:], an
// exact copy) and packages/autograd/src/ops.ts:495-505 (dW[idx[i],:] += g[i,:], visiting i
// in ascending order with f32 adds).  The reference's own GPU kernel does this with a racy
// non-atomic read-modify-write (packages/helios/src/kernels/nn.ts:5401-5415); here every
// output row is owned by one group of threads that adds the gradient rows naming it in
// ascending i, so the result is reproducible and, for f32 gradients, bit-identical to the
// CPU loop.
//
// Backward plan (all on the device, no host round trip):
//   1. rank[i]   = #{ j < i : idx[j] == idx[i] }            (tiled O(n^2) compare over a 2-D grid
//                                                             of tile pairs, n = B*T)
//   2. count[v]  = occurrences of v ; start[v] = exclusive prefix sum
//   3. order[start[idx[i]] + rank[i]] = i
//   4. row v: acc = (accumulate ? dW[v] : 0); for k in start[v]..start[v+1]: acc += g[order[k]]
//      (bf16 gradients: rows named more than 64 times — frequent tokens — are summed by a whole
//      block each, as a fixed tree over five segments of the occurrence list)
// Scratch: (2 n + vocab + 1) int32.  Algorithmic bytes: n*dim*e read + vocab*dim*4 written.
#include "common.cuh"

namespace alpha {

template <typename T>
__global__ void __launch_bounds__(256) embedding_fwd_kernel(const T *__restrict__ w, const int32_t *__restrict__ idx,
                                                            T *__restrict__ out, int64_t n_idx, int64_t dim,
                                                            int64_t vocab, bool vec_ok) {
  constexpr int V = Vec16<T>::N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (vec_ok) {
    const int64_t per_row = dim / V, total = n_idx * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const int64_t r = i / per_row, c = (i - r * per_row) * V;
      const int64_t src = idx[r];
      uint4 val = make_uint4(0, 0, 0, 0);
      if (src >= 0 && src < vocab) val = *reinterpret_cast<const uint4 *>(w + src * dim + c);
      *reinterpret_cast<uint4 *>(out + r * dim + c) = val;
    }
  } else {
    const int64_t total = n_idx * dim;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const int64_t r = i / dim, c = i - r * dim;
      const int64_t src = idx[r];
      out[i] = (src >= 0 && src < vocab) ? w[src * dim + c] : from_f32<T>(0.f);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) embedding_pos_fwd_kernel(const T *__restrict__ wte, const T *__restrict__ wpe,
                                                                const int32_t *__restrict__ tok, T *__restrict__ out,
                                                                int64_t n_idx, int64_t T_len, int64_t dim,
                                                                int64_t vocab, bool vec_ok) {
  constexpr int V = Vec16<T>::N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (vec_ok) {
    const int64_t per_row = dim / V, total = n_idx * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const int64_t r = i / per_row, c = (i - r * per_row) * V;
      const int64_t src = tok[r], t = r % T_len;
      float a[V], b[V];
      Vec16<T> va, vb, vo;
      vb.load(wpe + t * dim + c);
      vb.get(b);
      if (src >= 0 && src < vocab) {
        va.load(wte + src * dim + c);
        va.get(a);
      } else {
#pragma unroll
        for (int j = 0; j < V; j++) a[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < V; j++) a[j] += b[j];
      vo.set(a);
      vo.store(out + r * dim + c);
    }
  } else {
    const int64_t total = n_idx * dim;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const int64_t r = i / dim, c = i - r * dim;
      const int64_t src = tok[r], t = r % T_len;
      const float a = (src >= 0 && src < vocab) ? to_f32(wte[src * dim + c]) : 0.f;
      out[i] = from_f32<T>(a + to_f32(wpe[t * dim + c]));
    }
  }
}

constexpr int RANK_TILE = 256;

// rank[i] += #{ j in tile tj, j < i : idx[j] == idx[i] } for i in tile ti (tj <= ti); rank must
// be zero on entry.  Integer atomics: the result does not depend on the order of the blocks.
__global__ void __launch_bounds__(RANK_TILE) emb_rank_kernel(const int32_t *__restrict__ idx, int32_t *__restrict__ rank,
                                                             int32_t *__restrict__ count, int64_t n, int64_t vocab) {
  const int ti = blockIdx.y, tj = blockIdx.x;
  if (tj > ti) return;
  __shared__ int32_t tile[RANK_TILE];
  const int64_t i = (int64_t)ti * RANK_TILE + threadIdx.x, j = (int64_t)tj * RANK_TILE + threadIdx.x;
  tile[threadIdx.x] = j < n ? idx[j] : -2;
  const int32_t mine = i < n ? idx[i] : -1;
  __syncthreads();
  const int lim = tj < ti ? RANK_TILE : (int)threadIdx.x;  // only j < i
  int32_t r = 0;
#pragma unroll 8
  for (int k = 0; k < lim; k++) r += (tile[k] == mine);
  if (i < n) {
    if (r) atomicAdd(&rank[i], r);
    if (tj == ti && mine >= 0 && mine < vocab) atomicAdd(&count[mine], 1);
  }
}

// One block: exclusive prefix sum of count[0..vocab) into start[0..vocab]; in place allowed.
// Every warp owns a contiguous segment and walks it in 32-element chunks with coalesced
// accesses: a first pass sums the segment, the 32 segment sums are scanned with shuffles, a
// second pass writes the running prefix (four chunks of loads in flight at a time).
__global__ void __launch_bounds__(1024) emb_scan_kernel(const int32_t *count, int32_t *start, int64_t vocab) {
  __shared__ int32_t warp_tot[32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int64_t n = vocab + 1;                                  // entry `vocab` holds the total
  const int64_t seg = ((n + 31) / 32 + 31) / 32 * 32;           // per-warp segment, a multiple of 32
  const int64_t b = (int64_t)wid * seg, e = b + seg < n ? b + seg : n;
  int32_t sum = 0;
  for (int64_t i = b + lane; i < e; i += 32) sum += i < vocab ? count[i] : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) warp_tot[wid] = sum;
  __syncthreads();
  if (wid == 0) {
    int32_t w = warp_tot[lane], wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    warp_tot[lane] = wi - w;  // exclusive offset of each warp's segment
  }
  __syncthreads();
  int32_t carry = warp_tot[wid];
  for (int64_t c0 = b; c0 < e; c0 += 128) {
    int32_t v[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const int64_t i = c0 + u * 32 + lane;
      v[u] = (i < e && i < vocab) ? count[i] : 0;
    }
#pragma unroll
    for (int u = 0; u < 4; u++) {
      int32_t incl = v[u];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int32_t t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      const int64_t i = c0 + u * 32 + lane;
      if (i < e) start[i] = carry + incl - v[u];
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
}

__global__ void __launch_bounds__(256) emb_order_kernel(const int32_t *__restrict__ idx, const int32_t *__restrict__ rank,
                                                        const int32_t *__restrict__ start, int32_t *__restrict__ order,
                                                        int64_t n, int64_t vocab) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int32_t v = idx[i];
  if (v >= 0 && v < vocab) order[start[v] + rank[i]] = (int32_t)i;
}

// One thread per (row, 4 output columns); consecutive threads cover consecutive columns.
// Rows that no index names are left alone when accumulating.  With `hot_limit` > 0 a row named
// more than hot_limit times is not summed here: it is appended to hot_rows (its order in that
// list does not matter, each row is summed on its own) for emb_hot_rows_kernel.
template <typename T>
__global__ void __launch_bounds__(256) emb_rowsum_kernel(const T *__restrict__ g, const int32_t *__restrict__ start,
                                                         const int32_t *__restrict__ order, float *__restrict__ dw,
                                                         int64_t vocab, int64_t dim, int accumulate, int hot_limit,
                                                         int32_t *hot_rows, int32_t *hot_count, int hot_cap) {
  const int64_t per_row = (dim + 3) / 4;
  const int64_t total = vocab * per_row;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += stride) {
    const int64_t v = w / per_row, c = (w - v * per_row) * 4;
    const int nc = (int)(dim - c < 4 ? dim - c : 4);
    const int32_t s = start[v], e = start[v + 1];
    if (accumulate && s == e) continue;
    if (hot_limit > 0 && e - s > hot_limit) {
      if (c == 0) {
        const int slot = atomicAdd(hot_count, 1);
        if (slot < hot_cap) hot_rows[slot] = (int32_t)v;
      }
      continue;
    }
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float *dst = dw + v * dim + c;
    if (accumulate)
      for (int j = 0; j < nc; j++) acc[j] = dst[j];
    int32_t k = s;
    // loads are independent of the running sums: batch 8 rows of loads, then add in order
    for (; k + 8 <= e; k += 8) {
      float t[8][4];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const T *src = g + (int64_t)order[k + u] * dim + c;
#pragma unroll
        for (int j = 0; j < 4; j++) t[u][j] = j < nc ? to_f32(src[j]) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; u++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[j] += t[u][j];
    }
    for (; k < e; k++) {
      const T *src = g + (int64_t)order[k] * dim + c;
      for (int j = 0; j < nc; j++) acc[j] += to_f32(src[j]);
    }
    for (int j = 0; j < nc; j++) dst[j] = acc[j];
  }
}

// Rows named many times (frequent tokens): a whole block per row.  The row's occurrence list is
// cut into blockDim.y contiguous segments, segment s is summed in order by the threads
// (threadIdx.x = 8-column group, one 16-byte load per occurrence for bf16), and the segment sums
// are added in segment order — a fixed summation tree, so the result is reproducible (it is not
// the strictly sequential order of the reference loop, which is why fp32 parity runs do not use
// this kernel).  Ten segments: the most frequent token of a Zipf stream takes a seventh of the
// batch, and the length of the longest sequential sum is what this kernel's time is made of.
constexpr int HOT_COLS = 96;    // column groups per pass (768 columns)
constexpr int HOT_SEGS = 10;
constexpr int HOT_W = 8;        // columns per thread
template <typename T>
__global__ void __launch_bounds__(HOT_COLS * HOT_SEGS) emb_hot_rows_kernel(
    const T *__restrict__ g, const int32_t *__restrict__ start, const int32_t *__restrict__ order,
    float *__restrict__ dw, int64_t dim, int accumulate, const int32_t *__restrict__ hot_rows,
    const int32_t *__restrict__ hot_count, int hot_cap) {
  __shared__ float part[HOT_SEGS][HOT_COLS][HOT_W];
  const int n_hot = *hot_count < hot_cap ? *hot_count : hot_cap;
  const int cg = threadIdx.x, seg = threadIdx.y;
  const bool vec_ok = sizeof(T) == 2 && dim % HOT_W == 0 && (reinterpret_cast<uintptr_t>(g) & 15) == 0;
  for (int hidx = blockIdx.x; hidx < n_hot; hidx += gridDim.x) {
    const int64_t v = hot_rows[hidx];
    const int32_t s = start[v], e = start[v + 1];
    const int32_t len = (e - s + HOT_SEGS - 1) / HOT_SEGS;
    const int32_t ks = s + seg * len, ke = ks + len < e ? ks + len : e;
    for (int64_t c0 = 0; c0 < dim; c0 += HOT_COLS * HOT_W) {
      const int64_t c = c0 + cg * HOT_W;
      const int nc = c < dim ? (int)(dim - c < HOT_W ? dim - c : HOT_W) : 0;
      float acc[HOT_W];
#pragma unroll
      for (int j = 0; j < HOT_W; j++) acc[j] = 0.f;
      if (nc > 0) {
        int32_t k = ks;
        // loads are independent of the running sums: eight occurrences of loads, then add in order
        for (; k + 8 <= ke; k += 8) {
          float t[8][HOT_W];
#pragma unroll
          for (int u = 0; u < 8; u++) {
            const T *src = g + (int64_t)order[k + u] * dim + c;
            if (vec_ok) {
              Vec16<T> x;
              x.load(src);
              x.get(t[u]);
            } else {
#pragma unroll
              for (int j = 0; j < HOT_W; j++) t[u][j] = j < nc ? to_f32(src[j]) : 0.f;
            }
          }
#pragma unroll
          for (int u = 0; u < 8; u++)
#pragma unroll
            for (int j = 0; j < HOT_W; j++) acc[j] += t[u][j];
        }
        for (; k < ke; k++) {
          const T *src = g + (int64_t)order[k] * dim + c;
          for (int j = 0; j < nc; j++) acc[j] += to_f32(src[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < HOT_W; j++) part[seg][cg][j] = acc[j];
      __syncthreads();
      if (seg == 0 && nc > 0) {
        float *dst = dw + v * dim + c;
        for (int j = 0; j < nc; j++) {
          float t = accumulate ? dst[j] : 0.f;
#pragma unroll
          for (int q = 0; q < HOT_SEGS; q++) t += part[q][cg][j];
          dst[j] = t;
        }
      }
      __syncthreads();
    }
  }
}

}  // namespace alpha

using namespace alpha;

extern "C" {

int alpha_embedding_fwd(alpha_buf weight, alpha_buf indices, alpha_buf out, int64_t n_idx, int64_t dim,
                        int64_t vocab, int dtype) {
  ALPHA_REQUIRE_INIT();
  if (n_idx == 0 || dim == 0) return 0;
  ProfScope prof(PROF_EMBED, 2.0 * n_idx * dim * dtype_size(dtype));
  const bool a16 = (weight & 15) == 0 && (out & 15) == 0;
  if (dtype == ALPHA_F32) {
    const bool vec = a16 && dim % 4 == 0;
    embedding_fwd_kernel<float><<<grid_for(n_idx * dim / 4 + 1, 256, 16), 256, 0, g_stream>>>(
        ptr<float>(weight), ptr<int32_t>(indices), ptr<float>(out), n_idx, dim, vocab, vec);
  } else if (dtype == ALPHA_BF16) {
    const bool vec = a16 && dim % 8 == 0;
    embedding_fwd_kernel<__nv_bfloat16><<<grid_for(n_idx * dim / 8 + 1, 256, 16), 256, 0, g_stream>>>(
        ptr<__nv_bfloat16>(weight), ptr<int32_t>(indices), ptr<__nv_bfloat16>(out), n_idx, dim, vocab, vec);
  } else {
    return set_error("alpha_embedding_fwd: unsupported dtype %d", dtype);
  }
  ALPHA_LAUNCHED();
  return 0;
}

int alpha_embedding_pos_fwd(alpha_buf wte, alpha_buf wpe, alpha_buf tokens, alpha_buf out, int64_t batch, int64_t T,
                            int64_t dim, int64_t vocab, int dtype) {
  ALPHA_REQUIRE_INIT();
  const int64_t n_idx = batch * T;
  if (n_idx == 0 || dim == 0) return 0;
  ProfScope prof(PROF_EMBED, 3.0 * n_idx * dim * dtype_size(dtype));
  const bool a16 = (wte & 15) == 0 && (wpe & 15) == 0 && (out & 15) == 0;
  if (dtype == ALPHA_F32) {
    embedding_pos_fwd_kernel<float><<<grid_for(n_idx * dim / 4 + 1, 256, 16), 256, 0, g_stream>>>(
        ptr<float>(wte), ptr<float>(wpe), ptr<int32_t>(tokens), ptr<float>(out), n_idx, T, dim, vocab,
        a16 && dim % 4 == 0);
  } else if (dtype == ALPHA_BF16) {
    embedding_pos_fwd_kernel<__nv_bfloat16><<<grid_for(n_idx * dim / 8 + 1, 256, 16), 256, 0, g_stream>>>(
        ptr<__nv_bfloat16>(wte), ptr<__nv_bfloat16>(wpe), ptr<int32_t>(tokens), ptr<__nv_bfloat16>(out), n_idx, T,
        dim, vocab, a16 && dim % 8 == 0);
  } else {
    return set_error("alpha_embedding_pos_fwd: unsupported dtype %d", dtype);
  }
  ALPHA_LAUNCHED();
  return 0;
}

int alpha_embedding_bwd(alpha_buf indices, alpha_buf grad, alpha_buf dw, int64_t n_idx, int64_t dim, int64_t vocab,
                        int grad_dtype, int accumulate) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(grad_dtype == ALPHA_F32 || grad_dtype == ALPHA_BF16, "alpha_embedding_bwd: unsupported dtype %d",
              grad_dtype);
  ALPHA_CHECK(n_idx < (1ll << 31) && vocab < (1ll << 31), "alpha_embedding_bwd: sizes exceed int32");
  if (vocab == 0 || dim == 0) return 0;
  if (n_idx == 0) {
    if (!accumulate) ALPHA_CUDA(cudaMemsetAsync(ptr<void>(dw), 0, (size_t)vocab * dim * 4, g_stream));
    return 0;
  }
  ProfScope prof(PROF_EMBED, (double)n_idx * dim * dtype_size(grad_dtype));
  void *scratch = nullptr;
  constexpr int HOT_CAP = 1024;
  const size_t n_ints = (size_t)2 * n_idx + vocab + 1 + HOT_CAP + 1;
  if (pool_alloc(n_ints * sizeof(int32_t), &scratch)) return 1;
  int32_t *rank = (int32_t *)scratch, *order = rank + n_idx, *start = order + n_idx;
  int32_t *hot_rows = start + vocab + 1, *hot_count = hot_rows + HOT_CAP;
  ALPHA_CUDA(cudaMemsetAsync(rank, 0, (size_t)n_idx * sizeof(int32_t), g_stream));
  ALPHA_CUDA(cudaMemsetAsync(start, 0, (size_t)(vocab + 1 + HOT_CAP + 1) * sizeof(int32_t), g_stream));
  const int32_t *idx = ptr<int32_t>(indices);
  const unsigned nt = (unsigned)((n_idx + RANK_TILE - 1) / RANK_TILE);
  emb_rank_kernel<<<dim3(nt, nt), RANK_TILE, 0, g_stream>>>(idx, rank, start, n_idx, vocab);
  g_launches++;
  emb_scan_kernel<<<1, 1024, 0, g_stream>>>(start, start, vocab);
  g_launches++;
  emb_order_kernel<<<(unsigned)((n_idx + 255) / 256), 256, 0, g_stream>>>(idx, rank, start, order, n_idx, vocab);
  g_launches++;
  const int grid = grid_for(vocab * ((dim + 3) / 4), 256, 8);
  if (grad_dtype == ALPHA_F32) {
    // strictly sequential sums: bit-identical to the reference loop
    emb_rowsum_kernel<float><<<grid, 256, 0, g_stream>>>(ptr<float>(grad), start, order, ptr<float>(dw), vocab, dim,
                                                         accumulate, 0, nullptr, nullptr, 0);
  } else {
    // more than HOT_CAP frequent rows cannot occur: a row is hot above 64 occurrences and
    // n_idx / 64 <= HOT_CAP is checked here
    const int hot_limit = n_idx / 64 <= HOT_CAP ? 64 : 0;
    emb_rowsum_kernel<__nv_bfloat16><<<grid, 256, 0, g_stream>>>(ptr<__nv_bfloat16>(grad), start, order,
                                                                 ptr<float>(dw), vocab, dim, accumulate, hot_limit,
                                                                 hot_rows, hot_count, HOT_CAP);
    if (hot_limit > 0) {
      g_launches++;
      emb_hot_rows_kernel<__nv_bfloat16><<<g_sm_count, dim3(HOT_COLS, HOT_SEGS), 0, g_stream>>>(
          ptr<__nv_bfloat16>(grad), start, order, ptr<float>(dw), dim, accumulate, hot_rows, hot_count, HOT_CAP);
    }
  }
  pool_free(scratch);
  ALPHA_LAUNCHED();
  return 0;
}

}  // extern "C"
