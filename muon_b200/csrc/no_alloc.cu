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

inline int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

const float kAol4[4][3] = {{4.0098f, -7.0585f, 2.4635f},
                           {3.4585f, -5.5479f, 2.5959f},
                           {2.7573f, -3.2939f, 1.4254f},
                           {2.7215f, -3.0494f, 1.3169f}};
const float kClassic[3] = {3.4445f, -4.7750f, 2.0315f};
constexpr int kFroChunksMax = 296;

struct Slot {
  __nv_bfloat16* p;
  int64_t ld, bs;
};

}  // namespace

extern "C" {

int64_t muon_b200_ns_static_scratch_bytes(void) { return (int64_t)kStaticScratchBytes; }

int64_t muon_b200_ns_static_required_bytes(int batch, int64_t m, int64_t n) {
  if (batch < 1 || m < 1 || n < m) return -1;
  const int64_t ldn = round_up(n, 8), ldm = round_up(m, 8);
  const int64_t xs = round_up(batch * m * ldn * 2, 256);
  const int64_t as = round_up(batch * m * ldm * 2, 256);
  const int64_t per_matrix = ldm > kFroChunksMax ? ldm : kFroChunksMax;
  return xs + 3 * as + round_up((int64_t)batch * per_matrix * 4, 256);
}

int muon_b200_ns_run_static(const void* x, int64_t ldx, int64_t x_bs, void* out, int64_t ldo,
                            int64_t o_bs, int batch, int64_t m, int64_t n, int mode, int steps,
                            const float* coeffs, float eps, muon_b200_stream_t stream) {
  if (!x || !out) return set_error(ERR_INVALID_ARG, "ns_run_static: null pointer");
  if (x == out) return set_error(ERR_INVALID_ARG, "ns_run_static: out must not alias x");
  if (batch < 1 || m < 1 || n < m)
    return set_error(ERR_INVALID_ARG, "ns_run_static needs batch >= 1 and 1 <= m <= n");
  if (mode != MUON_B200_NS_AOL4 && mode != MUON_B200_NS_CLASSIC5)
    return set_error(ERR_INVALID_ARG, "unknown NS mode %d", mode);
  if (steps < 0 || steps > 64) return set_error(ERR_INVALID_ARG, "NS steps out of range: %d", steps);
  if (steps == 0) steps = (mode == MUON_B200_NS_AOL4) ? 4 : 5;
  if (!coeffs && mode == MUON_B200_NS_AOL4 && steps > 4)
    return set_error(ERR_INVALID_ARG, "the AOL table has 4 iterations; pass coeffs for %d", steps);
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (ldx % 8) || (ldo % 8) || (x_bs % 8) || (o_bs % 8) || ldx < n || ldo < n)
    return set_error(ERR_ALIGNMENT,
                     "ns_run_static: x and out must be 16-byte aligned with pitches %% 8 == 0 and >= n");
  const int64_t need = muon_b200_ns_static_required_bytes(batch, m, n);
  if (need > (int64_t)kStaticScratchBytes)
    return set_error(ERR_UNSUPPORTED,
                     "ns_run_static: batch=%d of %lld x %lld needs %lld bytes of scratch, the built-in "
                     "array holds %lld; use muon_b200_ns_run with a caller workspace",
                     batch, (long long)m, (long long)n, (long long)need,
                     (long long)kStaticScratchBytes);
  unsigned char* base = nullptr;
  int rc = scratch_for_current_device(&base);
  if (rc != OK) return rc;

  const int64_t ldn = round_up(n, 8), ldm = round_up(m, 8);
  const int64_t xs = round_up(batch * m * ldn * 2, 256);
  const int64_t as = round_up(batch * m * ldm * 2, 256);
  const int64_t a_bs = m * ldm;
  Slot S{reinterpret_cast<__nv_bfloat16*>(base), ldn, m * ldn};
  __nv_bfloat16* A = reinterpret_cast<__nv_bfloat16*>(base + xs);
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(base + xs + as);  // row-scaled copy of A
  __nv_bfloat16* B = reinterpret_cast<__nv_bfloat16*>(base + xs + 2 * as);
  float* fscratch = reinterpret_cast<float*>(base + xs + 3 * as);
  Slot O{static_cast<__nv_bfloat16*>(out), ldo, o_bs};
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  // The iteration ping-pongs between two buffers and must end in `out`: with an even number of
  // iterations it starts there, with an odd number it starts in the built-in buffer.
  Slot cur = (steps % 2 == 0) ? O : S;
  Slot oth = (steps % 2 == 0) ? S : O;
  for (int b = 0; b < batch; ++b)
    MB_CUDA_CHECK(cudaMemcpy2DAsync(cur.p + (int64_t)b * cur.bs, (size_t)cur.ld * 2,
                                    static_cast<const __nv_bfloat16*>(x) + (int64_t)b * x_bs,
                                    (size_t)ldx * 2, (size_t)n * 2, (size_t)m,
                                    cudaMemcpyDeviceToDevice, st));

  // Nothing in the scratch has to start at zero: A, B, the scaled copy, the row scales and the
  // ping-pong buffer are each written in full before they are read.
  bool have_gram = false;
  if (mode == MUON_B200_NS_AOL4) {
    rc = launch_ns_gemm(MODE_SYRK, cur.p, cur.ld, cur.bs, cur.p, cur.ld, cur.bs, A, ldm, a_bs, batch,
                        m, m, n, 1.f, 0.f, ADD_SYMMETRIC, st);
    if (rc != OK) return rc;
    rc = launch_aol_rescale(cur.p, cur.ld, cur.bs, A, As, ldm, a_bs, fscratch, ldm, (int)m, (int)n,
                            batch, eps, st);
    if (rc != OK) return rc;
    have_gram = true;
  } else {
    const int chunks = (int)(m < kFroChunksMax ? m : kFroChunksMax);
    rc = launch_fro_normalize(cur.p, cur.ld, cur.bs, (int)m, (int)n, batch, eps, fscratch, chunks, st);
    if (rc != OK) return rc;
  }
  for (int k = 0; k < steps; ++k) {
    float a, b, c;
    if (coeffs) {
      a = coeffs[3 * k]; b = coeffs[3 * k + 1]; c = coeffs[3 * k + 2];
    } else if (mode == MUON_B200_NS_AOL4) {
      a = kAol4[k][0]; b = kAol4[k][1]; c = kAol4[k][2];
    } else {
      a = kClassic[0]; b = kClassic[1]; c = kClassic[2];
    }
    if (have_gram) {
      rc = launch_ns_gemm(MODE_AXPBY, As, ldm, a_bs, As, ldm, a_bs, B, ldm, a_bs, batch, m, m, m, c,
                          b, ADD_ROW_SCALED, st, A, fscratch, ldm);
    } else {
      rc = launch_ns_gemm(MODE_SYRK, cur.p, cur.ld, cur.bs, cur.p, cur.ld, cur.bs, A, ldm, a_bs,
                          batch, m, m, n, 1.f, 0.f, ADD_SYMMETRIC, st);
      if (rc != OK) return rc;
      rc = launch_ns_gemm(MODE_AXPBY, A, ldm, a_bs, A, ldm, a_bs, B, ldm, a_bs, batch, m, m, m, c, b,
                          ADD_SYMMETRIC, st);
    }
    have_gram = false;
    if (rc != OK) return rc;
    rc = launch_ns_gemm(MODE_BX, B, ldm, a_bs, cur.p, cur.ld, cur.bs, oth.p, oth.ld, oth.bs, batch, m,
                        n, m, a, 0.f, ADD_GENERIC, st);
    if (rc != OK) return rc;
    Slot t = cur; cur = oth; oth = t;
  }
  return OK;
}

}  // extern "C"
