// Process-wide plumbing of libapt_b200: last-error text, launch counter and
// the optional event-based per-kernel timer.
#include <stdarg.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace apt {

static thread_local char g_err[512] = "";
static std::atomic<int64_t> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// ---- profiler: a growing list of (tag, begin, end) event pairs.
struct ProfRec {
  const char* tag;
  cudaEvent_t beg, end;
};
static std::atomic<int> g_prof_on{0};
static std::mutex g_prof_mu;
static std::vector<ProfRec> g_prof;
static const size_t kProfMax = 1 << 16;

// Events are pooled: after a read they go back to the free list, so a steady
// loop creates no events.
static std::vector<cudaEvent_t> g_free_events;

static bool take_event(cudaEvent_t* ev) {
  if (!g_free_events.empty()) {
    *ev = g_free_events.back();
    g_free_events.pop_back();
    return true;
  }
  return cudaEventCreate(ev) == cudaSuccess;
}

ProfScope::ProfScope(const char* t, cudaStream_t s) : tag(t), stream(s), slot(-1) {
  if (!g_prof_on.load(std::memory_order_relaxed)) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (g_prof.size() >= kProfMax) return;
  ProfRec r;
  r.tag = t;
  if (!take_event(&r.beg)) return;
  if (!take_event(&r.end)) {
    g_free_events.push_back(r.beg);
    return;
  }
  cudaEventRecord(r.beg, s);
  g_prof.push_back(r);
  slot = (int)g_prof.size() - 1;
}
ProfScope::~ProfScope() {
  if (slot < 0) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if ((size_t)slot < g_prof.size()) cudaEventRecord(g_prof[slot].end, stream);
}

}  // namespace apt

extern "C" {

const char* apt_last_error(void) { return apt::g_err; }
int apt_version(void) { return 100; }
int64_t apt_launch_count(void) { return apt::g_launches.load(); }
void apt_launch_count_reset(void) { apt::g_launches.store(0); }

int apt_memcpy_async(void* dst, const void* src, size_t nbytes, void* stream) {
  if (nbytes == 0) return APT_OK;
  APT_CHECK_ARG(dst && src, "apt_memcpy_async: null pointer");
  APT_CUDA(cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDefault, (cudaStream_t)stream));
  return APT_OK;
}

int apt_profile_enable(int on) {
  apt::g_prof_on.store(on ? 1 : 0);
  return APT_OK;
}

int apt_profile_read(const char* tag, double* total_ms, int64_t* launches) {
  APT_CHECK_ARG(tag && total_ms && launches, "apt_profile_read: null argument");
  std::lock_guard<std::mutex> lk(apt::g_prof_mu);
  double ms = 0.0;
  int64_t n = 0;
  std::vector<apt::ProfRec> keep;
  for (auto& r : apt::g_prof) {
    if (strcmp(r.tag, tag) != 0) {
      keep.push_back(r);
      continue;
    }
    float t = 0.f;
    cudaError_t e = cudaEventSynchronize(r.end);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&t, r.beg, r.end);
    apt::g_free_events.push_back(r.beg);
    apt::g_free_events.push_back(r.end);
    if (e != cudaSuccess) {
      apt::set_error("apt_profile_read(%s): %s", tag, cudaGetErrorString(e));
      apt::g_prof.swap(keep);
      return APT_ERR_CUDA;
    }
    ms += t;
    ++n;
  }
  apt::g_prof.swap(keep);
  *total_ms = ms;
  *launches = n;
  return APT_OK;
}

}  // extern "C"
