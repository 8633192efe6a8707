// Runtime of libalpha_cuda.so: device set-up, error strings, the compute stream, events,
// the caching device allocator and host<->device copies.
//
// It stands where the reference has its N-API Vulkan bridge
// (packages/helios/native/helios_vk.c: initDevice, createBuffer/destroyBuffer with a slab
// sub-allocator :818-822, uploadBuffer/readBuffer through a staging ring :683, one
// timeline semaphore, timestamp queries) — rebuilt on the CUDA runtime: one stream,
// cudaEvents, and a size-binned pool so that steady-state training never calls cudaMalloc.
#include <stdarg.h>
#include <string.h>

#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace alpha {

cudaStream_t g_stream = nullptr;
int g_device = -1;
int g_sm_count = 148;
bool g_inited = false;
int g_init_epoch = 0;
unsigned long long g_launches = 0;
int g_overlap_launches = ~0;
int g_overlap_hold = 0;

static thread_local char t_err[1024] = "";

int set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
  return 1;
}

// ── caching allocator ───────────────────────────────────────────────────────
// Blocks are rounded up to a size class and kept, once freed, in a per-class free list.
// All kernels run on one stream, so a freed block may be handed out again at once: work
// that still reads it was enqueued earlier on the same stream than anything the new
// owner enqueues.  (The side stream used for collectives is ordered by events, comm.cu.)
struct Pool {
  std::mutex mu;
  std::map<size_t, std::vector<void *>> free_lists;
  std::unordered_map<void *, size_t> live;   // ptr -> class size (handed out)
  std::unordered_map<void *, size_t> owned;  // every cudaMalloc'd block
  uint64_t in_use = 0, cached = 0, peak = 0, n_malloc = 0, n_alloc = 0;
};
static Pool g_pool;

static size_t size_class(size_t bytes) {
  if (bytes == 0) bytes = 1;
  if (bytes <= (1u << 20)) return (bytes + 511) & ~size_t(511);            // 512 B steps to 1 MiB
  if (bytes <= (64u << 20)) return (bytes + (1u << 20) - 1) & ~size_t((1u << 20) - 1);  // 1 MiB steps
  return (bytes + (8u << 20) - 1) & ~size_t((8u << 20) - 1);                // 8 MiB steps
}

int pool_alloc(size_t bytes, void **out) {
  const size_t cls = size_class(bytes);
  std::lock_guard<std::mutex> lk(g_pool.mu);
  g_pool.n_alloc++;
  void *p = nullptr;
  auto it = g_pool.free_lists.find(cls);
  if (it != g_pool.free_lists.end() && !it->second.empty()) {
    p = it->second.back();
    it->second.pop_back();
    g_pool.cached -= cls;
  } else {
    cudaError_t e = cudaMalloc(&p, cls);
    if (e != cudaSuccess) {
      // Give cached blocks back to the driver and retry once.
      cudaGetLastError();
      cudaStreamSynchronize(g_stream);
      for (auto &kv : g_pool.free_lists) {
        for (void *q : kv.second) {
          cudaFree(q);
          g_pool.owned.erase(q);
        }
        kv.second.clear();
      }
      g_pool.cached = 0;
      e = cudaMalloc(&p, cls);
      if (e != cudaSuccess) {
        cudaGetLastError();
        return set_error("alpha_alloc: cudaMalloc(%zu) -> %s", cls, cudaGetErrorString(e));
      }
    }
    g_pool.n_malloc++;
    g_pool.owned[p] = cls;
  }
  g_pool.live[p] = cls;
  g_pool.in_use += cls;
  if (g_pool.in_use > g_pool.peak) g_pool.peak = g_pool.in_use;
  *out = p;
  return 0;
}

int pool_free(void *p) {
  if (!p) return 0;
  std::lock_guard<std::mutex> lk(g_pool.mu);
  auto it = g_pool.live.find(p);
  if (it == g_pool.live.end()) return set_error("alpha_free: %p is not a live buffer of this library", p);
  const size_t cls = it->second;
  g_pool.live.erase(it);
  g_pool.in_use -= cls;
  g_pool.cached += cls;
  g_pool.free_lists[cls].push_back(p);
  return 0;
}

// ── content-addressed table cache ───────────────────────────────────────────
struct TableEntry {
  void *first;                        // device copy
  std::vector<unsigned char> host;    // the bytes it was made from: a hit is a byte-for-byte match
};
struct TableCache {
  std::mutex mu;
  std::unordered_map<uint64_t, TableEntry> entries;
};
static TableCache g_tables;

static void tables_clear() {
  std::lock_guard<std::mutex> lk(g_tables.mu);
  for (auto &kv : g_tables.entries) cudaFree(kv.second.first);
  g_tables.entries.clear();
}

int table_upload(const void *host, size_t bytes, const void **dev) {
  uint64_t h = 1469598103934665603ull;
  const unsigned char *b = (const unsigned char *)host;
  for (size_t i = 0; i < bytes; i++) h = (h ^ b[i]) * 1099511628211ull;
  h ^= bytes * 0x9e3779b97f4a7c15ull;
  std::lock_guard<std::mutex> lk(g_tables.mu);
  auto it = g_tables.entries.find(h);
  if (it != g_tables.entries.end()) {
    if (it->second.host.size() == bytes && memcmp(it->second.host.data(), host, bytes) == 0) {
      *dev = it->second.first;
      return 0;
    }
    // same hash, other contents: a kernel given the cached table would read wrong pointers
    cudaStreamSynchronize(g_stream);
    cudaFree(it->second.first);
    g_tables.entries.erase(it);
  }
  if (g_tables.entries.size() >= 256) {  // a changing workload: start over
    cudaStreamSynchronize(g_stream);
    for (auto &kv : g_tables.entries) cudaFree(kv.second.first);
    g_tables.entries.clear();
  }
  void *d = nullptr;
  cudaError_t e = cudaMalloc(&d, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return set_error("table_upload: cudaMalloc(%zu) -> %s", bytes, cudaGetErrorString(e));
  }
  e = cudaMemcpyAsync(d, host, bytes, cudaMemcpyHostToDevice, g_stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(g_stream);
  if (e != cudaSuccess) {
    cudaFree(d);
    return set_error("table_upload: copy -> %s", cudaGetErrorString(e));
  }
  g_tables.entries[h] = TableEntry{d, std::vector<unsigned char>(b, b + bytes)};
  *dev = d;
  return 0;
}

static int pool_purge(bool everything) {
  std::lock_guard<std::mutex> lk(g_pool.mu);
  cudaStreamSynchronize(g_stream);
  for (auto &kv : g_pool.free_lists) {
    for (void *q : kv.second) {
      cudaFree(q);
      g_pool.owned.erase(q);
    }
    kv.second.clear();
  }
  g_pool.cached = 0;
  if (everything) {
    for (auto &kv : g_pool.owned) cudaFree(kv.first);
    g_pool.owned.clear();
    g_pool.live.clear();
    g_pool.in_use = 0;
  }
  return 0;
}

}  // namespace alpha

using namespace alpha;

extern "C" {

const char *alpha_last_error(void) { return t_err; }

int alpha_init(int device_ordinal) {
  if (g_inited) {
    if (device_ordinal == g_device) return 0;
    return set_error("alpha_init: already initialised on device %d (one device per process)", g_device);
  }
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    cudaGetLastError();
    return set_error("alpha_init: no CUDA device is visible (%s); this library has no CPU fallback",
                     e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  }
  ALPHA_CHECK(device_ordinal >= 0 && device_ordinal < n, "alpha_init: device %d out of range [0,%d)",
              device_ordinal, n);
  ALPHA_CUDA(cudaSetDevice(device_ordinal));
  cudaDeviceProp prop;
  ALPHA_CUDA(cudaGetDeviceProperties(&prop, device_ordinal));
  ALPHA_CHECK(prop.major == 10, "alpha_init: device %d is sm_%d%d; this library holds sm_100a code only",
              device_ordinal, prop.major, prop.minor);
  g_sm_count = prop.multiProcessorCount;
  ALPHA_CUDA(cudaStreamCreateWithFlags(&g_stream, cudaStreamNonBlocking));
  g_device = device_ordinal;
  g_launches = 0;
  g_init_epoch++;
  g_inited = true;
  return 0;
}

int alpha_shutdown(void) {
  if (!g_inited) return 0;
  alpha_comm_destroy();
  cudaStreamSynchronize(g_stream);
  tables_clear();
  rope_tables_clear();
  tc::tc_error_word_free();
  pool_purge(true);
  cudaStreamDestroy(g_stream);
  g_stream = nullptr;
  g_inited = false;
  g_device = -1;
  return 0;
}

int alpha_set_launch_overlap(int families) {
  g_overlap_launches = families;
  return 0;
}

int alpha_device_info(alpha_device_info_t *out) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(out != nullptr, "alpha_device_info: null output");
  cudaDeviceProp prop;
  ALPHA_CUDA(cudaGetDeviceProperties(&prop, g_device));
  memset(out, 0, sizeof(*out));
  strncpy(out->name, prop.name, sizeof(out->name) - 1);
  out->vendor_id = 0x10de;
  out->sm_count = prop.multiProcessorCount;
  out->cc_major = prop.major;
  out->cc_minor = prop.minor;
  out->total_mem = prop.totalGlobalMem;
  out->l2_bytes = (uint64_t)prop.l2CacheSize;
  return 0;
}

int alpha_stream_sync(void) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CUDA(cudaStreamSynchronize(g_stream));
  return 0;
}

int alpha_launch_count(uint64_t *out) {
  ALPHA_CHECK(out != nullptr, "alpha_launch_count: null output");
  *out = g_launches;
  return 0;
}

int alpha_stream_handle(uint64_t *out) {
  ALPHA_REQUIRE_INIT();
  *out = (uint64_t)(uintptr_t)g_stream;
  return 0;
}

int alpha_event_create(uint64_t *ev) {
  ALPHA_REQUIRE_INIT();
  cudaEvent_t e;
  ALPHA_CUDA(cudaEventCreate(&e));
  *ev = (uint64_t)(uintptr_t)e;
  return 0;
}
int alpha_event_record(uint64_t ev) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CUDA(cudaEventRecord((cudaEvent_t)(uintptr_t)ev, g_stream));
  return 0;
}
int alpha_event_sync(uint64_t ev) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CUDA(cudaEventSynchronize((cudaEvent_t)(uintptr_t)ev));
  return 0;
}
int alpha_event_elapsed_ms(uint64_t a, uint64_t b, float *ms) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)(uintptr_t)a, (cudaEvent_t)(uintptr_t)b));
  return 0;
}
int alpha_event_destroy(uint64_t ev) {
  ALPHA_CUDA(cudaEventDestroy((cudaEvent_t)(uintptr_t)ev));
  return 0;
}

int alpha_alloc(size_t bytes, alpha_buf *out) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(out != nullptr, "alpha_alloc: null output");
  void *p = nullptr;
  if (pool_alloc(bytes, &p)) return 1;
  *out = (alpha_buf)(uintptr_t)p;
  return 0;
}

int alpha_free(alpha_buf buf) {
  ALPHA_REQUIRE_INIT();
  return pool_free(ptr<void>(buf));
}

int alpha_mem_stats(alpha_mem_stats_t *out) {
  ALPHA_CHECK(out != nullptr, "alpha_mem_stats: null output");
  std::lock_guard<std::mutex> lk(g_pool.mu);
  out->bytes_in_use = g_pool.in_use;
  out->bytes_cached = g_pool.cached;
  out->peak_in_use = g_pool.peak;
  out->n_device_mallocs = g_pool.n_malloc;
  out->n_allocs = g_pool.n_alloc;
  return 0;
}

int alpha_purge_pools(void) {
  ALPHA_REQUIRE_INIT();
  return pool_purge(false);
}

int alpha_memset(alpha_buf dst, int byte_value, size_t bytes) {
  ALPHA_REQUIRE_INIT();
  if (bytes == 0) return 0;
  ALPHA_CUDA(cudaMemsetAsync(ptr<void>(dst), byte_value, bytes, g_stream));
  return 0;
}

int alpha_h2d(alpha_buf dst, const void *host_src, size_t bytes) {
  ALPHA_REQUIRE_INIT();
  if (bytes == 0) return 0;
  ALPHA_CHECK(host_src != nullptr && dst != 0, "alpha_h2d: null pointer");
  // Pageable sources are staged by the runtime before the call returns; pinned sources
  // (alpha_host_alloc) are copied asynchronously on the compute stream.
  ALPHA_CUDA(cudaMemcpyAsync(ptr<void>(dst), host_src, bytes, cudaMemcpyHostToDevice, g_stream));
  return 0;
}

int alpha_d2h(void *host_dst, alpha_buf src, size_t bytes) {
  ALPHA_REQUIRE_INIT();
  if (bytes == 0) return 0;
  ALPHA_CHECK(host_dst != nullptr && src != 0, "alpha_d2h: null pointer");
  ALPHA_CUDA(cudaMemcpyAsync(host_dst, ptr<void>(src), bytes, cudaMemcpyDeviceToHost, g_stream));
  ALPHA_CUDA(cudaStreamSynchronize(g_stream));
  return 0;
}

// Enqueues the copy and returns; host_dst must be pinned (alpha_host_alloc) and may be read
// once an event recorded after this call has completed (alpha_event_record / alpha_event_sync).
int alpha_d2h_async(void *host_dst, alpha_buf src, size_t bytes) {
  ALPHA_REQUIRE_INIT();
  if (bytes == 0) return 0;
  ALPHA_CHECK(host_dst != nullptr && src != 0, "alpha_d2h_async: null pointer");
  ALPHA_CUDA(cudaMemcpyAsync(host_dst, ptr<void>(src), bytes, cudaMemcpyDeviceToHost, g_stream));
  return 0;
}

int alpha_d2d(alpha_buf dst, alpha_buf src, size_t bytes) {
  ALPHA_REQUIRE_INIT();
  if (bytes == 0) return 0;
  ALPHA_CUDA(cudaMemcpyAsync(ptr<void>(dst), ptr<void>(src), bytes, cudaMemcpyDeviceToDevice, g_stream));
  return 0;
}

int alpha_host_alloc(size_t bytes, void **out) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CUDA(cudaMallocHost(out, bytes ? bytes : 1));
  return 0;
}

int alpha_host_free(void *p) {
  if (p) ALPHA_CUDA(cudaFreeHost(p));
  return 0;
}

}  // extern "C"
