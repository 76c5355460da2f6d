// Optional per-kernel timing for benchmarks: when enabled, every kernel launch of the library is
// bracketed by a pair of CUDA events recorded on the launch stream, and the totals per kernel name
// can be read back after a synchronize.  Disabled by default (zero overhead beyond one branch).
// Events are host-side driver objects; no device memory is allocated here.
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace rwkvb200 {

int& last_cuda_error_slot() {
  static int e = 0;
  return e;
}

namespace {
struct Rec { int name; cudaEvent_t a, b; };
std::mutex g_mu;
bool g_on = false;
std::vector<std::string> g_names;
std::vector<Rec> g_recs;
std::vector<cudaEvent_t> g_pool;
constexpr size_t MAX_RECS = 1 << 16;

cudaEvent_t get_event() {
  if (!g_pool.empty()) { cudaEvent_t e = g_pool.back(); g_pool.pop_back(); return e; }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}
}  // namespace

ProfScope::ProfScope(const char* name, cudaStream_t st) : st_(st), idx_(-1) {
  if (!g_on) return;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_recs.size() >= MAX_RECS) return;
  int n = -1;
  for (size_t i = 0; i < g_names.size(); ++i) if (g_names[i] == name) { n = (int)i; break; }
  if (n < 0) { g_names.push_back(name); n = (int)g_names.size() - 1; }
  Rec r{n, get_event(), get_event()};
  if (!r.a || !r.b) return;
  cudaEventRecord(r.a, st_);
  g_recs.push_back(r);
  idx_ = (int)g_recs.size() - 1;
}

ProfScope::~ProfScope() {
  if (idx_ < 0) return;
  std::lock_guard<std::mutex> lk(g_mu);
  cudaEventRecord(g_recs[idx_].b, st_);
}

}  // namespace rwkvb200

using namespace rwkvb200;

extern "C" {

const char* rwkvb200_last_cuda_error(void) {
  static char buf[96];
  const int e = last_cuda_error_slot();
  if (e < 99999) return cudaGetErrorString((cudaError_t)e);
  if (e == 99999) return "device status word not available";
  snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed with CUresult %d", e - 100000);
  return buf;
}

void rwkvb200_profile_enable(int on) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_on = on != 0;
}

void rwkvb200_profile_reset(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  for (auto& r : g_recs) { g_pool.push_back(r.a); g_pool.push_back(r.b); }
  g_recs.clear();
  g_names.clear();
}

int rwkvb200_profile_count(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  return (int)g_names.size();
}

int rwkvb200_profile_get(int i, char* name, int name_len, float* total_ms, int* launches) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (i < 0 || i >= (int)g_names.size() || !name || name_len <= 0 || !total_ms || !launches) return RWKVB200_E_SHAPE;
  float tot = 0.f;
  int n = 0;
  for (auto& r : g_recs) {
    if (r.name != i) continue;
    if (cudaEventSynchronize(r.b) != cudaSuccess) return RWKVB200_E_CUDA;
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, r.a, r.b) != cudaSuccess) return RWKVB200_E_CUDA;
    tot += ms;
    ++n;
  }
  strncpy(name, g_names[i].c_str(), name_len - 1);
  name[name_len - 1] = 0;
  *total_ms = tot;
  *launches = n;
  return RWKVB200_OK;
}

}  // extern "C"
