// Data-parallel gradient exchange: NCCL all-reduce (sum) over NVLink / NVSwitch.
// No reference counterpart: the reference is single-device (docs/scale.md:3).
//
// One process per GPU.  NCCL is loaded with dlopen so that single-GPU use needs no NCCL at
// all; in a process that has already imported torch the soname resolves to the copy torch
// loaded, so there is one NCCL per process.  Collectives run on a side stream: at enqueue
// time the side stream waits on an event recorded on the compute stream (the producer of
// the bucket has been enqueued before), and alpha_comm_wait makes the compute stream wait
// for everything enqueued on the side stream so far.  NCCL writes its result into this
// GPU's own memory; no kernel of this library reads a peer's memory.
#include <dlfcn.h>
#include <string.h>

#include "common.cuh"

namespace alpha {

typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclSum = 0 };
enum { ncclFloat32 = 7, ncclBfloat16 = 9 };

struct Nccl {
  void *handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
};
static Nccl g_nccl;
static ncclComm_t g_comm = nullptr;
static cudaStream_t g_comm_stream = nullptr;
static cudaEvent_t g_ev_ready = nullptr, g_ev_done = nullptr, g_ev_probe = nullptr;
static int g_nranks = 1;

static int load_nccl() {
  if (g_nccl.handle) return 0;
  const char *names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char *n : names) {
    g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (g_nccl.handle) break;
  }
  if (!g_nccl.handle) return set_error("alpha_comm: cannot load libnccl.so.2 (%s)", dlerror());
#define SYM(field, name)                                                                   \
  *(void **)(&g_nccl.field) = dlsym(g_nccl.handle, name);                                  \
  if (!g_nccl.field) return set_error("alpha_comm: symbol %s missing from libnccl", name);
  SYM(GetUniqueId, "ncclGetUniqueId")
  SYM(CommInitRank, "ncclCommInitRank")
  SYM(AllReduce, "ncclAllReduce")
  SYM(GroupStart, "ncclGroupStart")
  SYM(GroupEnd, "ncclGroupEnd")
  SYM(CommDestroy, "ncclCommDestroy")
  SYM(CommAbort, "ncclCommAbort")
  SYM(CommGetAsyncError, "ncclCommGetAsyncError")
  SYM(GetErrorString, "ncclGetErrorString")
#undef SYM
  return 0;
}

#define ALPHA_NCCL(call)                                                                              \
  do {                                                                                                \
    ncclResult_t r_ = (call);                                                                         \
    if (r_ != 0) return set_error("%s:%d %s -> %s", __FILE__, __LINE__, #call, g_nccl.GetErrorString(r_)); \
  } while (0)

}  // namespace alpha

using namespace alpha;

extern "C" {

int alpha_comm_unique_id(void *out_128_bytes) {
  ALPHA_CHECK(out_128_bytes != nullptr, "alpha_comm_unique_id: null output");
  if (load_nccl()) return 1;
  ncclUniqueId id;
  ALPHA_NCCL(g_nccl.GetUniqueId(&id));
  memcpy(out_128_bytes, &id, sizeof(id));
  return 0;
}

int alpha_comm_init_rank(int n_ranks, int rank, const void *unique_id_128_bytes) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(n_ranks >= 1 && rank >= 0 && rank < n_ranks, "alpha_comm_init_rank: bad rank %d of %d", rank, n_ranks);
  ALPHA_CHECK(g_comm == nullptr, "alpha_comm_init_rank: communicator already exists");
  g_nranks = n_ranks;
  if (n_ranks == 1) return 0;  // nothing to exchange
  if (load_nccl()) return 1;
  ncclUniqueId id;
  memcpy(&id, unique_id_128_bytes, sizeof(id));
  ALPHA_CUDA(cudaStreamCreateWithFlags(&g_comm_stream, cudaStreamNonBlocking));
  ALPHA_CUDA(cudaEventCreateWithFlags(&g_ev_ready, cudaEventDisableTiming));
  ALPHA_CUDA(cudaEventCreateWithFlags(&g_ev_done, cudaEventDisableTiming));
  ALPHA_CUDA(cudaEventCreateWithFlags(&g_ev_probe, cudaEventDisableTiming));
  ALPHA_NCCL(g_nccl.CommInitRank(&g_comm, n_ranks, id, rank));
  return 0;
}

int alpha_comm_allreduce_sum(alpha_buf buf, int64_t n, int dtype) {
  ALPHA_REQUIRE_INIT();
  if (g_nranks == 1 || n == 0) return 0;
  ALPHA_CHECK(g_comm != nullptr, "alpha_comm_allreduce_sum: alpha_comm_init_rank was not called");
  ALPHA_CHECK(dtype == ALPHA_F32 || dtype == ALPHA_BF16, "alpha_comm_allreduce_sum: unsupported dtype %d", dtype);
  ALPHA_CUDA(cudaEventRecord(g_ev_ready, g_stream));
  ALPHA_CUDA(cudaStreamWaitEvent(g_comm_stream, g_ev_ready, 0));
  g_overlap_hold = 2;  // give the collective's blocks an ordinary kernel boundary to start at
  ALPHA_NCCL(g_nccl.AllReduce(ptr<void>(buf), ptr<void>(buf), (size_t)n, dtype == ALPHA_F32 ? ncclFloat32 : ncclBfloat16,
                              ncclSum, g_comm, g_comm_stream));
  return 0;
}

// One bucket = several gradient tensors reduced as one NCCL group: a single collective launch
// on the side stream moves all of them (sizes of tens of MB keep the launch count per step
// small and the NVLink transfers long).
int alpha_comm_allreduce_sum_bucket(const alpha_buf *bufs, const int64_t *counts, int n_bufs, int dtype) {
  ALPHA_REQUIRE_INIT();
  if (g_nranks == 1 || n_bufs == 0) return 0;
  ALPHA_CHECK(g_comm != nullptr, "alpha_comm_allreduce_sum_bucket: alpha_comm_init_rank was not called");
  ALPHA_CHECK(bufs != nullptr && counts != nullptr && n_bufs > 0, "alpha_comm_allreduce_sum_bucket: bad arguments");
  ALPHA_CHECK(dtype == ALPHA_F32 || dtype == ALPHA_BF16, "alpha_comm_allreduce_sum_bucket: unsupported dtype %d", dtype);
  ALPHA_CUDA(cudaEventRecord(g_ev_ready, g_stream));
  ALPHA_CUDA(cudaStreamWaitEvent(g_comm_stream, g_ev_ready, 0));
  g_overlap_hold = 2;  // give the collective's blocks an ordinary kernel boundary to start at
  ALPHA_NCCL(g_nccl.GroupStart());
  for (int i = 0; i < n_bufs; i++) {
    if (counts[i] == 0) continue;
    ncclResult_t r = g_nccl.AllReduce(ptr<void>(bufs[i]), ptr<void>(bufs[i]), (size_t)counts[i],
                                      dtype == ALPHA_F32 ? ncclFloat32 : ncclBfloat16, ncclSum, g_comm, g_comm_stream);
    if (r != 0) {
      g_nccl.GroupEnd();
      return set_error("alpha_comm_allreduce_sum_bucket: ncclAllReduce -> %s", g_nccl.GetErrorString(r));
    }
  }
  ALPHA_NCCL(g_nccl.GroupEnd());
  return 0;
}

int alpha_comm_wait(void) {
  ALPHA_REQUIRE_INIT();
  if (g_nranks == 1 || g_comm == nullptr) return 0;
  ALPHA_CUDA(cudaEventRecord(g_ev_done, g_comm_stream));
  ALPHA_CUDA(cudaStreamWaitEvent(g_stream, g_ev_done, 0));
  return 0;
}

// Host-side view of the exchange, without blocking: *pending = 1 while collectives enqueued so
// far have not completed on the device, *async_error = NCCL's asynchronous error code for the
// communicator (0 = none; a peer that died or a network fault shows up here, not as a return
// code of the enqueue).  A host that must not wait for ever polls this against a deadline and
// calls alpha_comm_abort when the deadline passes or an error appears.
int alpha_comm_query(int *pending, int *async_error) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(pending != nullptr && async_error != nullptr, "alpha_comm_query: null output");
  *pending = 0;
  *async_error = 0;
  if (g_nranks == 1 || g_comm == nullptr) return 0;
  ALPHA_CUDA(cudaEventRecord(g_ev_probe, g_comm_stream));
  cudaError_t q = cudaEventQuery(g_ev_probe);
  if (q == cudaErrorNotReady) {
    *pending = 1;
  } else if (q != cudaSuccess) {
    return set_error("alpha_comm_query: cudaEventQuery -> %s", cudaGetErrorString(q));
  }
  ncclResult_t ae = 0;
  ALPHA_NCCL(g_nccl.CommGetAsyncError(g_comm, &ae));
  *async_error = (int)ae;
  return 0;
}

static void comm_release_streams() {
  if (g_comm_stream) { cudaStreamDestroy(g_comm_stream); g_comm_stream = nullptr; }
  if (g_ev_ready) { cudaEventDestroy(g_ev_ready); g_ev_ready = nullptr; }
  if (g_ev_done) { cudaEventDestroy(g_ev_done); g_ev_done = nullptr; }
  if (g_ev_probe) { cudaEventDestroy(g_ev_probe); g_ev_probe = nullptr; }
  g_nranks = 1;
}

// Gives up on the communicator: ncclCommAbort makes collectives that are still waiting for a
// peer return, so the side stream drains and the process can report the failure and leave (or
// build a new communicator with the ranks that remain).  Gradients touched by an aborted
// collective are undefined; the step must be discarded.
int alpha_comm_abort(void) {
  if (g_comm) {
    ncclResult_t r = g_nccl.CommAbort(g_comm);
    g_comm = nullptr;
    if (g_comm_stream) cudaStreamSynchronize(g_comm_stream);
    comm_release_streams();
    if (r != 0) return set_error("alpha_comm_abort: ncclCommAbort -> %s", g_nccl.GetErrorString(r));
    return 0;
  }
  comm_release_streams();
  return 0;
}

int alpha_comm_destroy(void) {
  if (g_comm) {
    cudaStreamSynchronize(g_comm_stream);
    g_nccl.CommDestroy(g_comm);
    g_comm = nullptr;
  }
  comm_release_streams();
  return 0;
}

}  // extern "C"
