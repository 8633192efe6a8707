// Per-kernel-family device timing.  The reference times single dispatches with Vulkan
// timestamp queries (packages/helios/native/helios_vk.c:3448 gpuTime;
// packages/helios/src/backend.ts:5159-5204 profileOp); here the launch sites of the heavy
// kernel families record CUDA events on the compute stream while profiling is switched on,
// and alpha_profile_read sums their elapsed times and the algorithmic work they declared.
//
// NVTX: the same launch sites, and the host's step phases (alpha_range_push / alpha_range_pop,
// the counterpart of the reference's per-phase timers, packages/train/src/trainer.ts:1189-1264),
// open NVTX ranges, so that a timeline tool shows which family and phase a kernel belongs to.
// NVTX v3 is header-only and does nothing (a null function-pointer check) when no tool is attached.
#include <nvtx3/nvToolsExt.h>

#include <vector>

#include "common.cuh"

namespace alpha {

bool g_profiling = false;

struct ProfRec {
  cudaEvent_t e0, e1;
  int cat;
  double work;
};
static std::vector<ProfRec> g_recs;
static std::vector<cudaEvent_t> g_free_events;
static cudaEvent_t g_open[PROF_NCAT];
static double g_open_work[PROF_NCAT];

static cudaEvent_t get_event() {
  if (!g_free_events.empty()) {
    cudaEvent_t e = g_free_events.back();
    g_free_events.pop_back();
    return e;
  }
  cudaEvent_t e;
  cudaEventCreate(&e);
  return e;
}

static const char *const PROF_NAMES[PROF_NCAT] = {"gemm_tc", "gemm_f32", "attn_fwd", "attn_bwd", "cross_entropy",
                                                  "adamw",   "norm",     "embedding", "elementwise"};
void range_begin(int cat) { nvtxRangePushA(cat >= 0 && cat < PROF_NCAT ? PROF_NAMES[cat] : "alpha"); }
void range_end() { nvtxRangePop(); }

void prof_begin(int cat, double work) {
  cudaEvent_t e = get_event();
  cudaEventRecord(e, g_stream);
  g_open[cat] = e;
  g_open_work[cat] = work;
}

void prof_end(int cat) {
  cudaEvent_t e = get_event();
  cudaEventRecord(e, g_stream);
  g_recs.push_back({g_open[cat], e, cat, g_open_work[cat]});
}

}  // namespace alpha

using namespace alpha;

extern "C" {

int alpha_range_push(const char *name) {
  nvtxRangePushA(name ? name : "alpha");
  return 0;
}

int alpha_range_pop(void) {
  nvtxRangePop();
  return 0;
}

int alpha_profile_enable(int on) {
  ALPHA_REQUIRE_INIT();
  g_profiling = on != 0;
  return 0;
}

int alpha_profile_read(alpha_profile_entry_t *out, int n_categories) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(out != nullptr && n_categories >= PROF_NCAT, "alpha_profile_read: need room for %d categories", PROF_NCAT);
  ALPHA_CUDA(cudaStreamSynchronize(g_stream));
  for (int c = 0; c < n_categories; c++) {
    out[c].ms = 0;
    out[c].work = 0;
    out[c].launches = 0;
  }
  for (auto &r : g_recs) {
    float ms = 0.f;
    cudaEventElapsedTime(&ms, r.e0, r.e1);
    out[r.cat].ms += ms;
    out[r.cat].work += r.work;
    out[r.cat].launches += 1;
    g_free_events.push_back(r.e0);
    g_free_events.push_back(r.e1);
  }
  g_recs.clear();
  return 0;
}

}  // extern "C"
