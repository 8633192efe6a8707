// A probe of the bounded waits' give-up path.
//
// Every spin-wait of the tensor-core kernels goes through mbar_wait (tc_common.cuh): when a
// barrier does not complete within the limit, the waiter raises the block's abort flag, every
// role leaves its loop, tensor memory is given back, the library's error word is set and
// alpha_check_async_error() reports it.  In a healthy run that path never executes.  This
// kernel makes it execute without anything going wrong on the device: it is the GEMM's
// skeleton — barrier set-up, tensor-memory allocation by warp 1, a producer warp, an MMA warp
// and four epilogue warps, the same teardown — but nothing is ever copied or multiplied, so
// the producer's "stage is free" barrier is never signalled.  With a limit of about a
// millisecond the producer gives up first; the other roles, waiting on barriers of their own,
// see the flag and follow.  No copy is in flight, nothing is out of bounds, the kernel
// returns by itself.
#include "tc_common.cuh"

namespace alpha {
namespace tc {

constexpr int PROBE_THREADS = 192;       // producer, MMA and four epilogue warps, as in the GEMM
constexpr uint32_t PROBE_TMEM_COLS = 64;

__global__ void __launch_bounds__(PROBE_THREADS, 1)
wait_expiry_probe_kernel(uint32_t *err, uint32_t *roles_left, long long limit_cycles) {
  __shared__ __align__(8) uint64_t bars[3];
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_word;
  volatile uint32_t *abort_flag = &abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t empty_bar = smem_u32(&bars[0]), full_bar = smem_u32(&bars[1]), tfull_bar = smem_u32(&bars[2]);
  if (threadIdx.x == 0) {
    mbar_init(empty_bar, 1);
    mbar_init(full_bar, 1);
    mbar_init(tfull_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), PROBE_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  bool ok;
  if (warp == 0) {
    // producer: waits for a stage to be handed back, as after the first trip round the ring;
    // parity 0 of a fresh barrier is the phase that has not completed — nobody will arrive
    ok = mbar_wait_limited(empty_bar, 0, abort_flag, limit_cycles);
  } else if (warp == 1) {
    // MMA issuer: waits for the producer's tile (ten times the producer's patience, so the
    // producer is the one that gives up and this warp leaves through the flag)
    ok = mbar_wait_limited(full_bar, 0, abort_flag, 10 * limit_cycles);
  } else {
    // epilogue: waits for a finished accumulator
    ok = mbar_wait_limited(tfull_bar, 0, abort_flag, 10 * limit_cycles);
  }
  if (!ok && lane == 0 && roles_left) atomicAdd(roles_left, 1u);

  // ── teardown, as in the GEMM ──
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 200000ll) {
    }
    if (threadIdx.x == 0 && err) atomicExch(err, 0x7E000000u | (uint32_t)(blockIdx.x & 0xFFFF));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, PROBE_TMEM_COLS);
  }
}

}  // namespace tc
}  // namespace alpha

using namespace alpha;

// Runs the probe on `blocks` SMs with a wait limit of `limit_us` microseconds (1 .. 100000) and
// returns how many warps left through the give-up path in *roles_left_out (6 per block when
// it works).  The error word is left set: the next alpha_check_async_error() must report it.
extern "C" int alpha_debug_wait_expiry(int blocks, int limit_us, int *roles_left_out) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(blocks >= 1 && blocks <= 1024, "alpha_debug_wait_expiry: blocks %d out of range [1, 1024]", blocks);
  ALPHA_CHECK(limit_us >= 1 && limit_us <= 100000, "alpha_debug_wait_expiry: limit %d us out of range [1, 100000]",
              limit_us);
  uint32_t *err = tc::tc_error_word();
  ALPHA_CHECK(err != nullptr, "alpha_debug_wait_expiry: no device error word");
  int khz = 0;
  ALPHA_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, g_device));
  const long long cycles = (long long)limit_us * (khz > 0 ? khz : 1500000) / 1000;
  void *cnt = nullptr;
  if (pool_alloc(sizeof(uint32_t), &cnt)) return 1;
  ALPHA_CUDA(cudaMemsetAsync(cnt, 0, sizeof(uint32_t), g_stream));
  tc::wait_expiry_probe_kernel<<<blocks, tc::PROBE_THREADS, 0, g_stream>>>(err, (uint32_t *)cnt, cycles);
  ALPHA_LAUNCHED();
  uint32_t host = 0;
  ALPHA_CUDA(cudaMemcpyAsync(&host, cnt, sizeof(host), cudaMemcpyDeviceToHost, g_stream));
  ALPHA_CUDA(cudaStreamSynchronize(g_stream));
  pool_free(cnt);
  if (roles_left_out) *roles_left_out = (int)host;
  return 0;
}
