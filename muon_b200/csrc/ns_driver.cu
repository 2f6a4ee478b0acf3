// Launch sequence of one Newton-Schulz orthogonalisation (reference
// zeropower_via_newtonschulz5, muon.py:778-795, and the classic iteration of its commented
// block, muon.py:282-289).
#include "../../include/muon_b200.h"

#include "common.cuh"
#include "elementwise.h"
#include "ns_driver.h"
#include "ns_gemm.h"
#include "profiling.h"

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

namespace mb {

namespace {
// Coefficients (a, b, c) per iteration.
const float kAol4[4][3] = {{4.0098f, -7.0585f, 2.4635f},   // muon.py:754-759
                           {3.4585f, -5.5479f, 2.5959f},
                           {2.7573f, -3.2939f, 1.4254f},
                           {2.7215f, -3.0494f, 1.3169f}};
const float kClassic[3] = {3.4445f, -4.7750f, 2.0315f};    // muon.py:276
}  // namespace

int ns_check_mode(int mode, int* steps, const float* coeffs) {
  if (mode != MUON_B200_NS_AOL4 && mode != MUON_B200_NS_CLASSIC5)
    return set_error(ERR_INVALID_ARG, "unknown NS mode %d", mode);
  if (*steps < 0 || *steps > 64) return set_error(ERR_INVALID_ARG, "NS steps out of range: %d", *steps);
  if (*steps == 0) *steps = (mode == MUON_B200_NS_AOL4) ? 4 : 5;
  if (!coeffs && mode == MUON_B200_NS_AOL4 && *steps > 4)
    return set_error(ERR_INVALID_ARG, "the AOL table has 4 iterations; pass coeffs for %d", *steps);
  return OK;
}

int ns_iterate(const NsBuffers& buf, int batch, int64_t m, int64_t n, int mode, int steps,
               const float* coeffs, float eps, cudaStream_t st, int* result_index) {
  int cur = 0;
  int rc;
  bool have_gram = false;
  if (mode == MUON_B200_NS_AOL4) {
    // Gram matrix once, shared by the rescale and the first iteration (muon.py:778-785).
    rc = launch_ns_gemm(MODE_SYRK, buf.x[0], buf.ldx[0], buf.x_bs[0], buf.x[0], buf.ldx[0], buf.x_bs[0],
                        buf.A, buf.ldm, buf.a_bs, batch, m, m, n, 1.f, 0.f, ADD_SYMMETRIC, st);
    if (rc != OK) return rc;
    // A / s goes to its own buffer with A's pitches, so the symmetric unscaled A and 1/s remain
    // for line 2's epilogue.
    rc = launch_aol_rescale(buf.x[0], buf.ldx[0], buf.x_bs[0], buf.A, buf.A_scaled, buf.ldm, buf.a_bs,
                            buf.fscratch, buf.f_bs, (int)m, (int)n, batch, eps, st);
    if (rc != OK) return rc;
    have_gram = true;
  } else {
    const int chunks = (int)(m < kFroChunksMax ? m : kFroChunksMax);
    rc = launch_fro_normalize(buf.x[0], buf.ldx[0], buf.x_bs[0], (int)m, (int)n, batch, eps, buf.fscratch,
                              chunks, st);
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
    __nv_bfloat16* X = buf.x[cur];
    const int64_t ldx = buf.ldx[cur], xbs = buf.x_bs[cur];
    if (have_gram) {
      // First AOL iteration: the operand is A / s (rows scaled, not symmetric); the addend
      // beta * (A / s) is rebuilt per element from the symmetric A and 1/s.
      rc = launch_ns_gemm(MODE_AXPBY, buf.A_scaled, buf.ldm, buf.a_bs, buf.A_scaled, buf.ldm, buf.a_bs,
                          buf.B, buf.ldm, buf.a_bs, batch, m, m, m, c, b, ADD_ROW_SCALED, st, buf.A,
                          buf.fscratch, buf.f_bs);
    } else {
      rc = launch_ns_gemm(MODE_SYRK, X, ldx, xbs, X, ldx, xbs, buf.A, buf.ldm, buf.a_bs, batch, m, m, n,
                          1.f, 0.f, ADD_SYMMETRIC, st);
      if (rc != OK) return rc;
      // A comes straight from line 1 and is exactly symmetric.
      rc = launch_ns_gemm(MODE_AXPBY, buf.A, buf.ldm, buf.a_bs, buf.A, buf.ldm, buf.a_bs, buf.B, buf.ldm,
                          buf.a_bs, batch, m, m, m, c, b, ADD_SYMMETRIC, st);
    }
    have_gram = false;
    if (rc != OK) return rc;
    rc = launch_ns_gemm(MODE_BX, buf.B, buf.ldm, buf.a_bs, X, ldx, xbs, buf.x[cur ^ 1], buf.ldx[cur ^ 1],
                        buf.x_bs[cur ^ 1], batch, m, n, m, a, 0.f, ADD_GENERIC, st);
    if (rc != OK) return rc;
    cur ^= 1;
  }
  if (result_index) *result_index = cur;
  return OK;
}

// ---------------------------------------------------------------------------
// Graph replay
// ---------------------------------------------------------------------------
namespace {

constexpr int kGraphMaxSteps = 8;         // longer coefficient lists are launched directly
constexpr double kGraphMaxFlops = 2e12;   // above ~1.5 ms of device work the launches are hidden
constexpr size_t kGraphCacheEntries = 128;

struct GraphKey {  // plain data, compared with memcmp: keep it free of padding garbage (memset)
  NsBuffers buf;
  int64_t m, n;
  int batch, mode, steps, has_coeffs, device, reserved_sms;
  float eps;
  float coeffs[3 * kGraphMaxSteps];
};

struct GraphEntry {
  GraphKey key;
  cudaGraphExec_t exec = nullptr;  // nullptr: capture failed once, launch directly from now on
  int64_t counts[K_KIND_COUNT] = {};
  int result_index = 0;
  uint64_t last_use = 0;
};

std::mutex g_graph_mu;
std::vector<GraphEntry> g_graphs;
uint64_t g_graph_clock = 0;
cudaStream_t g_capture_stream[64] = {};
std::atomic<int> g_graph_on{-1};  // -1: not decided yet (environment), 0 / 1

}  // namespace

void set_graph_replay(bool on) { g_graph_on.store(on ? 1 : 0); }

bool graph_replay_enabled() {
  int v = g_graph_on.load();
  if (v < 0) {
    const char* e = std::getenv("MUON_B200_GRAPH");
    v = (e && (e[0] == '0' || e[0] == 'n' || e[0] == 'f')) ? 0 : 1;
    g_graph_on.store(v);
  }
  return v == 1;
}

int ns_iterate_replayed(const NsBuffers& buf, int batch, int64_t m, int64_t n, int mode, int steps,
                        const float* coeffs, float eps, cudaStream_t stream, int* result_index) {
  const double flops = (double)batch * steps * ((double)m * (m + 1) * n + (double)m * m * (m + 1) + 2.0 * m * m * n);
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (!graph_replay_enabled() || timing_enabled() || steps > kGraphMaxSteps || flops > kGraphMaxFlops ||
      cudaStreamIsCapturing(stream, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) {
    (void)cudaGetLastError();
    return ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, stream, result_index);
  }
  int dev = 0;
  MB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, stream, result_index);

  GraphKey key;
  std::memset(&key, 0, sizeof(key));
  key.buf = buf;
  key.m = m; key.n = n; key.batch = batch; key.mode = mode; key.steps = steps;
  key.has_coeffs = coeffs ? 1 : 0;
  key.device = dev;
  key.reserved_sms = get_reserved_sms();
  key.eps = eps;
  if (coeffs) std::memcpy(key.coeffs, coeffs, sizeof(float) * 3 * steps);

  std::lock_guard<std::mutex> lk(g_graph_mu);
  GraphEntry* hit = nullptr;
  for (GraphEntry& e : g_graphs)
    if (std::memcmp(&e.key, &key, sizeof(key)) == 0) { hit = &e; break; }
  if (hit) {
    hit->last_use = ++g_graph_clock;
    if (!hit->exec) return ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, stream, result_index);
    MB_CUDA_CHECK(cudaGraphLaunch(hit->exec, stream));
    add_launch_counts(hit->counts);
    if (result_index) *result_index = hit->result_index;
    return OK;
  }

  // First use: capture the launch sequence on the library's own stream (the caller's may be the
  // legacy default stream, which cannot be captured). Thread-local mode: other threads' CUDA
  // calls do not disturb the capture. Nothing executes until the graph is launched below.
  if (!g_capture_stream[dev])
    MB_CUDA_CHECK(cudaStreamCreateWithFlags(&g_capture_stream[dev], cudaStreamNonBlocking));
  GraphEntry fresh;
  fresh.key = key;
  fresh.last_use = ++g_graph_clock;
  cudaGraph_t graph = nullptr;
  int rc = OK;
  if (cudaStreamBeginCapture(g_capture_stream[dev], cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
    set_launch_recorder(fresh.counts);
    rc = ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, g_capture_stream[dev], &fresh.result_index);
    set_launch_recorder(nullptr);
    const cudaError_t ended = cudaStreamEndCapture(g_capture_stream[dev], &graph);
    // The launches above were only recorded: take them out of the process totals again; the
    // replay below (or the direct launch) counts them.
    int64_t undo[K_KIND_COUNT];
    for (int k = 0; k < K_KIND_COUNT; ++k) undo[k] = -fresh.counts[k];
    add_launch_counts(undo);
    if (rc != OK) {
      // A launcher refused (bad argument, or a call the capture does not allow): nothing to
      // cache; the direct launch reports the error, if it is one, against the caller's stream.
      if (graph) cudaGraphDestroy(graph);
      (void)cudaGetLastError();
      return ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, stream, result_index);
    }
    if (ended != cudaSuccess || !graph ||
        cudaGraphInstantiate(&fresh.exec, graph, 0) != cudaSuccess) {
      fresh.exec = nullptr;
    }
    if (graph) cudaGraphDestroy(graph);
  }
  (void)cudaGetLastError();
  if (g_graphs.size() >= kGraphCacheEntries) {
    size_t oldest = 0;
    for (size_t i = 1; i < g_graphs.size(); ++i)
      if (g_graphs[i].last_use < g_graphs[oldest].last_use) oldest = i;
    if (g_graphs[oldest].exec) cudaGraphExecDestroy(g_graphs[oldest].exec);
    g_graphs.erase(g_graphs.begin() + oldest);
  }
  g_graphs.push_back(fresh);
  if (!fresh.exec) return ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, stream, result_index);
  MB_CUDA_CHECK(cudaGraphLaunch(fresh.exec, stream));
  add_launch_counts(fresh.counts);
  if (result_index) *result_index = fresh.result_index;
  return OK;
}

}  // namespace mb
