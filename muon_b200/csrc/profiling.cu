#include "profiling.h"

#include "common.cuh"

#include <atomic>
#include <mutex>
#include <vector>

namespace mb {

namespace {
std::atomic<int64_t> g_counts[K_KIND_COUNT];
std::atomic<bool> g_timing{false};
struct Interval {
  int kind;
  double work;
  int64_t tag;
  cudaEvent_t start, stop;
};
std::vector<Interval> g_intervals;
std::mutex g_mu;
thread_local int64_t* t_recorder = nullptr;
// Intervals folded away by compact(): per-kind totals that the next timing_collect adds in.
double g_folded_ms[K_KIND_COUNT] = {};
double g_folded_work[K_KIND_COUNT] = {};
int64_t g_folded_launches[K_KIND_COUNT] = {};
constexpr size_t kMaxPendingIntervals = 1 << 16;

// Called with g_mu held once the list is long: intervals whose stop event has completed are
// added to the per-kind totals and their events destroyed, so a run that enables timing and
// never collects keeps a bounded number of events and a bounded list.
void compact_locked() {
  size_t kept = 0;
  for (size_t i = 0; i < g_intervals.size(); ++i) {
    const Interval& iv = g_intervals[i];
    float t = 0.f;
    if (cudaEventQuery(iv.stop) == cudaSuccess && cudaEventElapsedTime(&t, iv.start, iv.stop) == cudaSuccess) {
      if (iv.kind >= 0 && iv.kind < K_KIND_COUNT) {
        g_folded_ms[iv.kind] += t;
        g_folded_work[iv.kind] += iv.work;
        g_folded_launches[iv.kind] += 1;
      }
      cudaEventDestroy(iv.start);
      cudaEventDestroy(iv.stop);
    } else {
      (void)cudaGetLastError();  // cudaErrorNotReady is not an error here
      g_intervals[kept++] = iv;
    }
  }
  g_intervals.resize(kept);
}
}  // namespace

LaunchScope::LaunchScope(int kind, double work, cudaStream_t stream, int64_t tag)
    : kind_(kind), work_(work), stream_(stream), tag_(tag) {
  g_counts[kind].fetch_add(1, std::memory_order_relaxed);
  if (t_recorder) t_recorder[kind] += 1;
  if (g_timing.load(std::memory_order_relaxed)) {
    if (cudaEventCreate(&start_) == cudaSuccess) cudaEventRecord(start_, stream_);
    else start_ = nullptr;
  }
}

LaunchScope::~LaunchScope() {
  if (!start_) return;
  cudaEvent_t stop = nullptr;
  if (cudaEventCreate(&stop) != cudaSuccess) {
    cudaEventDestroy(start_);
    return;
  }
  cudaEventRecord(stop, stream_);
  std::lock_guard<std::mutex> lk(g_mu);
  g_intervals.push_back({kind_, work_, tag_, start_, stop});
  if (g_intervals.size() >= kMaxPendingIntervals) compact_locked();
}

void timing_enable(bool on) { g_timing.store(on); }
bool timing_enabled() { return g_timing.load(std::memory_order_relaxed); }
void set_launch_recorder(int64_t* recorder) { t_recorder = recorder; }
void add_launch_counts(const int64_t* counts) {
  for (int k = 0; k < K_KIND_COUNT; ++k)
    if (counts[k]) g_counts[k].fetch_add(counts[k], std::memory_order_relaxed);
}

int timing_collect(double* ms, double* work, int64_t* launches, int n_kinds) {
  std::vector<Interval> taken;
  for (int k = 0; k < n_kinds; ++k) {
    ms[k] = 0.0;
    work[k] = 0.0;
    launches[k] = 0;
  }
  {
    std::lock_guard<std::mutex> lk(g_mu);
    taken.swap(g_intervals);
    for (int k = 0; k < K_KIND_COUNT; ++k) {
      if (k < n_kinds) {
        ms[k] = g_folded_ms[k];
        work[k] = g_folded_work[k];
        launches[k] = g_folded_launches[k];
      }
      g_folded_ms[k] = g_folded_work[k] = 0.0;
      g_folded_launches[k] = 0;
    }
  }
  int rc = OK;
  for (const Interval& iv : taken) {
    float t = 0.f;
    cudaError_t e = cudaEventSynchronize(iv.stop);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&t, iv.start, iv.stop);
    if (e != cudaSuccess && rc == OK)
      rc = set_error(ERR_CUDA, "timing_collect: %s", cudaGetErrorString(e));
    if (e == cudaSuccess && iv.kind < n_kinds) {
      ms[iv.kind] += t;
      work[iv.kind] += iv.work;
      launches[iv.kind] += 1;
    }
    cudaEventDestroy(iv.start);
    cudaEventDestroy(iv.stop);
  }
  return rc;
}

int timing_collect_records(int max_records, int* kinds, int64_t* tags, double* ms, double* work,
                           int* n_out) {
  std::vector<Interval> taken;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    taken.swap(g_intervals);
  }
  int n = 0, rc = OK;
  for (const Interval& iv : taken) {
    float t = 0.f;
    cudaError_t e = cudaEventSynchronize(iv.stop);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&t, iv.start, iv.stop);
    if (e != cudaSuccess && rc == OK)
      rc = set_error(ERR_CUDA, "timing_collect_records: %s", cudaGetErrorString(e));
    if (e == cudaSuccess && n < max_records) {
      kinds[n] = iv.kind;
      tags[n] = iv.tag;
      ms[n] = t;
      work[n] = iv.work;
      ++n;
    }
    cudaEventDestroy(iv.start);
    cudaEventDestroy(iv.stop);
  }
  *n_out = n;
  return rc;
}

void launch_counts(int64_t* counts, int n_kinds) {
  for (int k = 0; k < n_kinds && k < K_KIND_COUNT; ++k) counts[k] = g_counts[k].load();
}

}  // namespace mb
