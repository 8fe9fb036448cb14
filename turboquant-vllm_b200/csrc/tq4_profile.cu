// Optional per-kernel timing: CUDA events recorded on the launching stream around each
// kernel class, read back after the measured region.  Off by default (zero overhead).
#include <cstdlib>
#include <vector>

#include "tq4_common.cuh"

namespace tq4 {

struct Profiler {
  bool on = false;
  int cap = 0;
  int count[TQ4_PROF_KINDS] = {0};
  std::vector<cudaEvent_t> ev[TQ4_PROF_KINDS][2];
};
static Profiler g_prof;

void prof_begin(int kind, cudaStream_t st) {
  if (!g_prof.on || g_prof.count[kind] >= g_prof.cap) return;
  cudaEventRecord(g_prof.ev[kind][0][g_prof.count[kind]], st);
}
void prof_end(int kind, cudaStream_t st) {
  if (!g_prof.on || g_prof.count[kind] >= g_prof.cap) return;
  cudaEventRecord(g_prof.ev[kind][1][g_prof.count[kind]], st);
  ++g_prof.count[kind];
}

bool pdl_enabled() {
  static const bool on = getenv("TQ4_NO_PDL") == nullptr;
  return on;
}

}  // namespace tq4

extern "C" int tq4_profile_start(int max_samples) {
  using namespace tq4;
  if (max_samples <= 0 || max_samples > (1 << 20)) return TQ4_ERR_INVALID_ARG;
  for (int k = 0; k < TQ4_PROF_KINDS; ++k) {
    for (int s = 0; s < 2; ++s) {
      while ((int)g_prof.ev[k][s].size() < max_samples) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) return TQ4_ERR_CUDA;
        g_prof.ev[k][s].push_back(e);
      }
    }
    g_prof.count[k] = 0;
  }
  g_prof.cap = max_samples;
  g_prof.on = true;
  return TQ4_OK;
}

extern "C" int tq4_profile_stop(void) {
  tq4::g_prof.on = false;
  return TQ4_OK;
}

extern "C" int tq4_profile_read(int kind, float* ms_out, int max_out) {
  using namespace tq4;
  if (kind < 0 || kind >= TQ4_PROF_KINDS || (!ms_out && max_out > 0)) return -1;
  const int n = g_prof.count[kind] < max_out ? g_prof.count[kind] : max_out;
  for (int i = 0; i < n; ++i) {
    if (cudaEventSynchronize(g_prof.ev[kind][1][i]) != cudaSuccess) return -1;
    if (cudaEventElapsedTime(&ms_out[i], g_prof.ev[kind][0][i], g_prof.ev[kind][1][i]) != cudaSuccess)
      return -1;
  }
  return n;
}
