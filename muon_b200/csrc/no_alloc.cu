// Newton-Schulz orthogonalisation for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at the point where they need the
// optimizer step: code running inside a region where the framework's allocator is frozen
// (a memory-planned graph, a real-time loop with a fixed memory budget) or a plugin that
// is handed buffers and nothing else. muon_b200_ns_run needs a caller-provided workspace;
// this variant keeps its scratch (one ping-pong copy of X, the Gram matrix A, its row-scaled
// copy, B and the row scales) in a fixed array that is part of the library image.
//
// Consequences of that choice, all documented on the entry point:
//   * every GPU on which the library is loaded holds kStaticScratchBytes until exit;
//   * problems whose scratch exceeds it are rejected;
//   * all calls share the array, so calls that overlap on one GPU race;
//   * the first call on a device looks up the array's device address and should therefore
//     come before any stream capture.
#include "../../include/muon_b200.h"

#include "common.cuh"
#include "elementwise.h"
#include "ns_driver.h"
#include "ns_gemm.h"

#include <mutex>

using namespace mb;

namespace {

constexpr size_t kStaticScratchBytes = 64u << 20;  // 64 MiB

// In host code this name is only a stand-in for the device symbol; its device address is
// obtained per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_mu;
void* g_scratch_addr[64] = {nullptr};

int scratch_for_current_device(unsigned char** out) {
  int dev = 0;
  MB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(ERR_UNSUPPORTED, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    MB_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_scratch));
    if (!p || (reinterpret_cast<uintptr_t>(p) & 255))
      return set_error(ERR_CUDA, "static scratch address %p is unusable", p);
    g_scratch_addr[dev] = p;
  }
  *out = static_cast<unsigned char*>(g_scratch_addr[dev]);
  return OK;
}

// Byte range [lo, hi) that a [batch, m, n] bf16 tensor with the given pitches touches.
void byte_range(const void* p, int64_t ld, int64_t bs, int batch, int64_t m, int64_t n,
                uintptr_t* lo, uintptr_t* hi) {
  const int64_t last = (int64_t)(batch - 1) * bs + (m - 1) * ld + n;  // one past the last element
  *lo = reinterpret_cast<uintptr_t>(p);
  *hi = *lo + (uintptr_t)last * 2;
}

}  // namespace

extern "C" {

int64_t muon_b200_ns_static_scratch_bytes(void) { return (int64_t)kStaticScratchBytes; }

int64_t muon_b200_ns_static_required_bytes(int batch, int64_t m, int64_t n) {
  return ns_scratch_bytes(batch, m, n);
}

int muon_b200_ns_run_static(const void* x, int64_t ldx, int64_t x_bs, void* out, int64_t ldo,
                            int64_t o_bs, int batch, int64_t m, int64_t n, int mode, int steps,
                            const float* coeffs, float eps, muon_b200_stream_t stream) {
  if (!x || !out) return set_error(ERR_INVALID_ARG, "ns_run_static: null pointer");
  if (batch < 1 || m < 1 || n < m)
    return set_error(ERR_INVALID_ARG, "ns_run_static needs batch >= 1 and 1 <= m <= n");
  int rc = ns_check_mode(mode, &steps, coeffs);
  if (rc != OK) return rc;
  if (mode == MUON_B200_NS_AOL4_FP8)
    return set_error(ERR_UNSUPPORTED, "ns_run_static: the e4m3 variant needs a caller workspace (muon_b200_ns_run)");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (ldx % 8) || (ldo % 8) || (x_bs % 8) || (o_bs % 8) || ldx < n || ldo < n)
    return set_error(ERR_ALIGNMENT,
                     "ns_run_static: x and out must be 16-byte aligned with pitches %% 8 == 0 and >= n");
  if (batch > 1 && (x_bs < (m - 1) * ldx + n || o_bs < (m - 1) * ldo + n))
    return set_error(ERR_INVALID_ARG, "ns_run_static: batch pitch shorter than one matrix");
  const int64_t need = muon_b200_ns_static_required_bytes(batch, m, n);
  if (need > (int64_t)kStaticScratchBytes)
    return set_error(ERR_UNSUPPORTED,
                     "ns_run_static: batch=%d of %lld x %lld needs %lld bytes of scratch, the built-in "
                     "array holds %lld; use muon_b200_ns_run with a caller workspace",
                     batch, (long long)m, (long long)n, (long long)need,
                     (long long)kStaticScratchBytes);
  {
    // With an even iteration count `out` is the ping-pong buffer and is written while x is
    // still being copied in, so any overlap of the two ranges (not only x == out) corrupts x.
    uintptr_t xl, xh, ol, oh;
    byte_range(x, ldx, x_bs, batch, m, n, &xl, &xh);
    byte_range(out, ldo, o_bs, batch, m, n, &ol, &oh);
    if (xl < oh && ol < xh)
      return set_error(ERR_INVALID_ARG, "ns_run_static: out must not overlap x");
  }
  unsigned char* base = nullptr;
  rc = scratch_for_current_device(&base);
  if (rc != OK) return rc;

  // Same launch sequence as muon_b200_ns_run, never replayed from a graph (instantiating one
  // allocates driver resources).
  return ns_run_with_scratch(x, DT_BF16, m, n, ldx, x_bs, static_cast<__nv_bfloat16*>(out), ldo, o_bs, base,
                             batch, mode, steps, coeffs, eps, /*replay=*/false,
                             static_cast<cudaStream_t>(stream));
}

}  // extern "C"
