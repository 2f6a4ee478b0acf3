// Launch accounting and optional per-kernel CUDA-event timing for the library's kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mb {

enum KernelKind : int {
  K_NS_LINE1 = 0,   // work unit: algorithmic FLOPs, m(m+1)k per matrix
  K_NS_LINE2 = 1,   // m*m*(m+1)
  K_NS_LINE3 = 2,   // 2*m*m*n
  K_PROLOGUE = 3,   // work unit: algorithmic HBM bytes
  K_EPILOGUE = 4,
  K_AOL_RESCALE = 5,
  K_FRO_NORMALIZE = 6,
  K_ADAM = 7,
  K_KIND_COUNT = 8,
};

// Counts the launch; when timing is enabled also brackets it with two events recorded on
// `stream` (the launching stream), so the interval covers exactly this kernel.
class LaunchScope {
 public:
  // `tag` is free-form and only reported back by timing_collect_records.
  LaunchScope(int kind, double work, cudaStream_t stream, int64_t tag = 0);
  ~LaunchScope();

 private:
  int kind_;
  double work_;
  cudaStream_t stream_;
  int64_t tag_;
  cudaEvent_t start_ = nullptr;
};

// While timing is on every launch keeps two events until it is collected. Once 65536 launches
// are pending, those that have completed are folded into per-kind totals (which the next
// timing_collect adds in; timing_collect_records no longer lists them), so a long run that
// never collects holds a bounded number of events.
void timing_enable(bool on);
bool timing_enabled();
// While a recorder is installed on the calling thread, every LaunchScope it creates adds one to
// recorder[kind] (used to remember which kernels a captured graph holds). Pass nullptr to remove.
void set_launch_recorder(int64_t* recorder);
// Adds per-kind launch counts (a replayed graph's kernels) to the process totals.
void add_launch_counts(const int64_t* counts);
// Waits for all recorded intervals, adds them up per kind and forgets them.
int timing_collect(double* ms, double* work, int64_t* launches, int n_kinds);
// Same, but one entry per launch (in launch order), at most `max_records`.
int timing_collect_records(int max_records, int* kinds, int64_t* tags, double* ms, double* work,
                           int* n_out);
void launch_counts(int64_t* counts, int n_kinds);

}  // namespace mb
