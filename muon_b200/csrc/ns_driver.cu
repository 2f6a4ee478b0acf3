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
  if (mode != MUON_B200_NS_AOL4 && mode != MUON_B200_NS_CLASSIC5 && mode != MUON_B200_NS_AOL4_FP8)
    return set_error(ERR_INVALID_ARG, "unknown NS mode %d", mode);
  if (*steps < 0 || *steps > 64) return set_error(ERR_INVALID_ARG, "NS steps out of range: %d", *steps);
  if (*steps == 0) *steps = (mode == MUON_B200_NS_CLASSIC5) ? 5 : 4;
  if (!coeffs && mode != MUON_B200_NS_CLASSIC5 && *steps > 4)
    return set_error(ERR_INVALID_ARG, "the AOL table has 4 iterations; pass coeffs for %d", *steps);
  return OK;
}

int ns_iterate(const NsBuffers& buf, int batch, int64_t m, int64_t n, int mode, int steps,
               const float* coeffs, float eps, cudaStream_t st, int* result_index, const UpdateSpec* upd) {
  int cur = 0;
  int rc;
  bool have_gram = false;
  const bool classic = mode == MUON_B200_NS_CLASSIC5;
  // (its only line 3 already carries the normalisation factor)
  if (classic && steps == 1 && upd)
    return set_error(ERR_INVALID_ARG, "a one-step classic iteration cannot apply the update itself");
  // e4m3 products only where they pay and where their rounding noise averages out: the error of a
  // Gram entry falls with 1/sqrt(n), and below about a thousand columns it is no longer small
  // against the bf16 algorithm's own (measured: 1.2e-2 rel-Fro at n >= 2304, 2e-2 at n = 328).
  // Smaller matrices are iterated in bf16 in this mode too.
  const bool fp8 = mode == MUON_B200_NS_AOL4_FP8 && n >= kFp8MinCols;
  if (fp8 && (!buf.x8 || !buf.e8)) return set_error(ERR_INVALID_ARG, "the e4m3 variant needs its two extra buffers");
  // Power-of-two scales of the e4m3 copies. Rows of X have norm about 1 after the rescale, so its
  // entries are about 1/sqrt(n): sx brings them to about 1 (and a whole row's norm stays below the
  // e4m3 maximum of 448). E = A - I has entries well below 1: se = 64.
  SplitK sk;
  sk.partial = buf.splitk;
  sk.bytes = buf.splitk_bytes;
  float sx = 1.f;
  while (sx < 256.f && sx * sx * 2.f <= (float)n) sx *= 2.f;  // 2^round(log2(sqrt(n))), capped
  const float se = 64.f;
  if (mode != MUON_B200_NS_CLASSIC5) {
    // Gram matrix once, shared by the rescale and the first iteration (muon.py:778-785).
    rc = launch_ns_gemm(MODE_SYRK, buf.x[0], buf.ldx[0], buf.x_bs[0], buf.x[0], buf.ldx[0], buf.x_bs[0],
                        buf.A, buf.ldm, buf.a_bs, batch, m, m, n, 1.f, 0.f, ADD_SYMMETRIC, st, nullptr, nullptr,
                        0, nullptr, nullptr, nullptr, &sk);
    if (rc != OK) return rc;
    // A / s goes to its own buffer with A's pitches, so the symmetric unscaled A and 1/s remain
    // for line 2's epilogue.
    rc = launch_aol_rescale(buf.x[0], buf.ldx[0], buf.x_bs[0], buf.A, buf.A_scaled, buf.ldm, buf.a_bs,
                            buf.fscratch, buf.f_bs, (int)m, (int)n, batch, eps, st);
    if (rc != OK) return rc;
    have_gram = true;
  } else {
    // muon.py:282: the factor 1 / (||X|| + eps) per matrix; the first line 1 and the first line 3
    // apply it (squared, plain) to their outputs, X itself stays as it is.
    if (!buf.fro_scales) return set_error(ERR_INVALID_ARG, "the classic iteration needs room for its scale factors");
    const int chunks = (int)(m < kFroChunks ? m : kFroChunks);
    rc = launch_fro_scales(buf.x[0], buf.ldx[0], buf.x_bs[0], (int)m, (int)n, batch, eps, buf.fscratch, chunks,
                           buf.tile_sumsq, buf.tile_bs, (int)buf.tile_count, buf.fro_scales, st);
    if (rc != OK) return rc;
  }

  for (int k = 0; k < steps; ++k) {
    float a, b, c;
    if (coeffs) {
      a = coeffs[3 * k]; b = coeffs[3 * k + 1]; c = coeffs[3 * k + 2];
    } else if (mode != MUON_B200_NS_CLASSIC5) {
      a = kAol4[k][0]; b = kAol4[k][1]; c = kAol4[k][2];
    } else {
      a = kClassic[0]; b = kClassic[1]; c = kClassic[2];
    }
    __nv_bfloat16* X = buf.x[cur];
    const int64_t ldx = buf.ldx[cur], xbs = buf.x_bs[cur];
    // e4m3 variant: the first iteration (Gram matrix for the rescale, row-scaled line 2) stays in
    // bf16; from the second on lines 1 and 2 take e4m3 operands; line 3 is always bf16 and leaves
    // the e4m3 copy of its output for the next line 1.
    Fp8Spec l3_out;
    if (fp8 && k + 1 < steps) {
      l3_out.kind = F8_EXTRA_OUT;
      l3_out.out8 = buf.x8;
      l3_out.ldo8 = buf.ld8n;
      l3_out.out8_bs = buf.x8_bs;
      l3_out.out8_scale = sx;
    }
    if (fp8 && !have_gram) {
      Fp8Spec l1;
      l1.kind = F8_OPERANDS;
      l1.op8 = buf.x8;
      l1.ld8 = buf.ld8n;
      l1.bs8 = buf.x8_bs;
      l1.out8 = buf.e8;
      l1.ldo8 = buf.ld8m;
      l1.out8_bs = buf.e8_bs;
      l1.out8_scale = se;
      l1.acc_scale = 1.f / (sx * sx);
      rc = launch_ns_gemm(MODE_SYRK, X, ldx, xbs, X, ldx, xbs, buf.A, buf.ldm, buf.a_bs, batch, m, m, n,
                          1.f, 0.f, ADD_SYMMETRIC, st, nullptr, nullptr, 0, &l1);
      if (rc != OK) return rc;
      // b*A + c*A*A = c*E*E + (b + 2c)*A - c*I with E = A - I (see Fp8Spec)
      Fp8Spec l2;
      l2.kind = F8_OPERANDS;
      l2.op8 = buf.e8;
      l2.ld8 = buf.ld8m;
      l2.bs8 = buf.e8_bs;
      l2.diag = -c;
      rc = launch_ns_gemm(MODE_AXPBY, buf.A, buf.ldm, buf.a_bs, buf.A, buf.ldm, buf.a_bs, buf.B, buf.ldm,
                          buf.a_bs, batch, m, m, m, c / (se * se), b + 2.f * c, ADD_SYMMETRIC, st, nullptr,
                          nullptr, 0, &l2);
      if (rc != OK) return rc;
      rc = launch_ns_gemm(MODE_BX, buf.B, buf.ldm, buf.a_bs, X, ldx, xbs, buf.x[cur ^ 1], buf.ldx[cur ^ 1],
                          buf.x_bs[cur ^ 1], batch, m, n, m, a, 0.f, ADD_GENERIC, st, nullptr, nullptr, 0,
                          l3_out.kind != F8_NONE ? &l3_out : nullptr, k + 1 == steps ? upd : nullptr);
      if (rc != OK) return rc;
      cur ^= 1;
      continue;
    }
    if (have_gram) {
      // First AOL iteration: the operand is A / s (rows scaled, not symmetric); the addend
      // beta * (A / s) is rebuilt per element from the symmetric A and 1/s.
      rc = launch_ns_gemm(MODE_AXPBY, buf.A_scaled, buf.ldm, buf.a_bs, buf.A_scaled, buf.ldm, buf.a_bs,
                          buf.B, buf.ldm, buf.a_bs, batch, m, m, m, c, b, ADD_ROW_SCALED, st, buf.A,
                          buf.fscratch, buf.f_bs);
    } else {
      rc = launch_ns_gemm(MODE_SYRK, X, ldx, xbs, X, ldx, xbs, buf.A, buf.ldm, buf.a_bs, batch, m, m, n,
                          1.f, 0.f, ADD_SYMMETRIC, st, nullptr, nullptr, 0, nullptr, nullptr,
                          classic && k == 0 ? buf.fro_scales + batch : nullptr, &sk);
      if (rc != OK) return rc;
      // A comes straight from line 1 and is exactly symmetric.
      rc = launch_ns_gemm(MODE_AXPBY, buf.A, buf.ldm, buf.a_bs, buf.A, buf.ldm, buf.a_bs, buf.B, buf.ldm,
                          buf.a_bs, batch, m, m, m, c, b, ADD_SYMMETRIC, st);
    }
    have_gram = false;
    if (rc != OK) return rc;
    rc = launch_ns_gemm(MODE_BX, buf.B, buf.ldm, buf.a_bs, X, ldx, xbs, buf.x[cur ^ 1], buf.ldx[cur ^ 1],
                        buf.x_bs[cur ^ 1], batch, m, n, m, a, 0.f, ADD_GENERIC, st, nullptr, nullptr, 0,
                        l3_out.kind != F8_NONE ? &l3_out : nullptr, k + 1 == steps ? upd : nullptr,
                        classic && k == 0 ? buf.fro_scales : nullptr);
    if (rc != OK) return rc;
    cur ^= 1;
  }
  if (result_index) *result_index = cur;
  return OK;
}

namespace {
inline int64_t round_up_i64(int64_t v, int64_t a) { return (v + a - 1) / a * a; }
}  // namespace

int64_t ns_fp8_extra_bytes(int batch, int64_t m, int64_t n) {
  return round_up_i64(batch * m * fp8_pitch(n), 256) + round_up_i64(batch * m * fp8_pitch(m), 256);
}

int64_t ns_classic_extra_bytes(int batch, int64_t m, int64_t n) {
  return round_up_i64((int64_t)batch * classic_tiles_max(m, n) * 4, 256);
}

int64_t ns_scratch_bytes(int batch, int64_t m, int64_t n, int mode, bool split_k) {
  if (batch < 1 || m < 1 || n < m) return -1;
  const int64_t ldn = round_up_i64(n, 8), ldm = round_up_i64(m, 8);
  const int64_t xs = round_up_i64(batch * m * ldn * 2, 256);
  const int64_t as = round_up_i64(batch * m * ldm * 2, 256);
  const int64_t per_matrix = ldm > kFroChunksMax ? ldm : kFroChunksMax;
  return xs + 3 * as + round_up_i64((int64_t)batch * per_matrix * 4, 256) +
         (mode == MUON_B200_NS_AOL4_FP8 ? ns_fp8_extra_bytes(batch, m, n) : 0) +
         (split_k ? round_up_i64(splitk_scratch_bytes(batch, m, n), 256) : 0);
}

int ns_run_with_scratch(const void* src, int dtype, int64_t rows, int64_t cols, int64_t ld_src,
                        int64_t src_bs, __nv_bfloat16* out, int64_t ldo, int64_t o_bs,
                        unsigned char* scratch, int batch, int mode, int steps, const float* coeffs,
                        float eps, bool replay, cudaStream_t st, bool split_k) {
  const bool tall = rows > cols;
  const int64_t m = tall ? cols : rows, n = tall ? rows : cols;
  const int64_t ldn = round_up_i64(n, 8), ldm = round_up_i64(m, 8);
  const int64_t xs = round_up_i64(batch * m * ldn * 2, 256);
  const int64_t as = round_up_i64(batch * m * ldm * 2, 256);
  // The iteration ping-pongs between two buffers and must end in `out`: with an even number of
  // iterations it starts there, with an odd number it starts in the scratch buffer.
  const int o = (steps % 2 == 0) ? 0 : 1;  // index of `out` among the two iterate buffers
  NsBuffers buf{};
  buf.x[o] = out;
  buf.ldx[o] = ldo;
  buf.x_bs[o] = o_bs;
  buf.x[o ^ 1] = reinterpret_cast<__nv_bfloat16*>(scratch);
  buf.ldx[o ^ 1] = ldn;
  buf.x_bs[o ^ 1] = m * ldn;
  buf.A = reinterpret_cast<__nv_bfloat16*>(scratch + xs);
  buf.A_scaled = reinterpret_cast<__nv_bfloat16*>(scratch + xs + as);  // row-scaled copy of A
  buf.B = reinterpret_cast<__nv_bfloat16*>(scratch + xs + 2 * as);
  buf.ldm = ldm;
  buf.a_bs = m * ldm;
  buf.fscratch = reinterpret_cast<float*>(scratch + xs + 3 * as);
  buf.f_bs = ldm;
  if (mode == MUON_B200_NS_AOL4_FP8) {
    const int64_t per_matrix = ldm > kFroChunksMax ? ldm : kFroChunksMax;
    unsigned char* extra = scratch + xs + 3 * as + round_up_i64((int64_t)batch * per_matrix * 4, 256);
    buf.ld8n = fp8_pitch(n);
    buf.ld8m = fp8_pitch(m);
    buf.x8_bs = m * buf.ld8n;
    buf.e8_bs = m * buf.ld8m;
    buf.x8 = extra;
    buf.e8 = extra + round_up_i64(batch * buf.x8_bs, 256);
  }
  // (classic iteration: the caller's matrices arrive through the cast kernel, so the driver sums
  // over X itself; tile_sumsq stays null)
  buf.fro_scales = fro_scales_in(buf.fscratch, batch, ldm);
  buf.splitk_bytes = split_k ? splitk_scratch_bytes(batch, m, n) : 0;
  if (buf.splitk_bytes > 0) {
    const int64_t per_matrix = ldm > kFroChunksMax ? ldm : kFroChunksMax;
    buf.splitk = reinterpret_cast<float*>(scratch + xs + 3 * as + round_up_i64((int64_t)batch * per_matrix * 4, 256) +
                                          (mode == MUON_B200_NS_AOL4_FP8 ? ns_fp8_extra_bytes(batch, m, n) : 0));
  }
  // muon.py:760-764: cast, transposition of tall inputs, contiguous copy.
  int rc = launch_cast_bf16(src, dtype, ld_src, src_bs, buf.x[0], buf.ldx[0], buf.x_bs[0], (int)rows,
                            (int)cols, batch, tall ? 1 : 0, 1.0f, st);
  if (rc != OK) return rc;
  // Nothing in the scratch has to start at zero: A, B, the scaled copy, the row scales and the
  // iterate buffer are each written in full before they are read.
  int where = 0;
  rc = replay ? ns_iterate_replayed(buf, batch, m, n, mode, steps, coeffs, eps, st, &where)
              : ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, st, &where);
  if (rc != OK) return rc;
  if (where != o) return set_error(ERR_CUDA, "Newton-Schulz result landed in the wrong buffer");
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
  // fused update (all zero without one): the graph holds the parameter addresses and the
  // step's learning rate, so a run with a changing learning rate never comes back to a graph
  void* upd_param[kMaxUpdateTensors];
  int64_t upd_rows, upd_cols;
  int upd_dtype;
  float upd_scale, upd_decay, upd_neg_lr;
};

struct GraphEntry {
  GraphKey key;
  cudaGraphExec_t exec = nullptr;  // nullptr: seen once so far, or capture failed (see `failed`)
  bool failed = false;             // capture or instantiation failed: launch directly from now on
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
                        const float* coeffs, float eps, cudaStream_t stream, int* result_index,
                        const UpdateSpec* upd) {
  const double flops = (double)batch * steps * ((double)m * (m + 1) * n + (double)m * m * (m + 1) + 2.0 * m * m * n);
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (!graph_replay_enabled() || timing_enabled() || steps > kGraphMaxSteps || flops > kGraphMaxFlops ||
      cudaStreamIsCapturing(stream, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) {
    (void)cudaGetLastError();
    return ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, stream, result_index, upd);
  }
  int dev = 0;
  MB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, stream, result_index, upd);

  GraphKey key;
  std::memset(&key, 0, sizeof(key));
  key.buf = buf;
  key.m = m; key.n = n; key.batch = batch; key.mode = mode; key.steps = steps;
  key.has_coeffs = coeffs ? 1 : 0;
  key.device = dev;
  key.reserved_sms = get_reserved_sms();
  key.eps = eps;
  if (coeffs) std::memcpy(key.coeffs, coeffs, sizeof(float) * 3 * steps);
  if (upd) {
    for (int b = 0; b < batch && b < kMaxUpdateTensors; ++b) key.upd_param[b] = upd->param[b];
    key.upd_rows = upd->rows; key.upd_cols = upd->cols; key.upd_dtype = upd->dtype + 1;
    key.upd_scale = upd->scale; key.upd_decay = upd->decay; key.upd_neg_lr = upd->neg_lr;
  }

  std::lock_guard<std::mutex> lk(g_graph_mu);
  GraphEntry* hit = nullptr;
  for (GraphEntry& e : g_graphs)
    if (std::memcmp(&e.key, &key, sizeof(key)) == 0) { hit = &e; break; }
  if (hit) {
    hit->last_use = ++g_graph_clock;
    if (hit->failed) return ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, stream, result_index, upd);
    if (hit->exec) {
      MB_CUDA_CHECK(cudaGraphLaunch(hit->exec, stream));
      add_launch_counts(hit->counts);
      if (result_index) *result_index = hit->result_index;
      return OK;
    }
  } else {
    // First sighting of these buffers: launch directly and only remember them. A graph is built
    // when the same buffers come back (an optimizer's cached workspace does every step; the
    // output of a one-off functional call does not).
    if (g_graphs.size() >= kGraphCacheEntries) {
      size_t oldest = 0;
      for (size_t i = 1; i < g_graphs.size(); ++i)
        if (g_graphs[i].last_use < g_graphs[oldest].last_use) oldest = i;
      if (g_graphs[oldest].exec) cudaGraphExecDestroy(g_graphs[oldest].exec);
      g_graphs.erase(g_graphs.begin() + oldest);
    }
    GraphEntry seen;
    seen.key = key;
    seen.last_use = ++g_graph_clock;
    g_graphs.push_back(seen);
    return ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, stream, result_index, upd);
  }

  // Second sighting: capture the launch sequence on the library's own stream (the caller's may be
  // the legacy default stream, which cannot be captured). Thread-local mode: other threads' CUDA
  // calls do not disturb the capture. Nothing executes until the graph is launched below.
  if (!g_capture_stream[dev])
    MB_CUDA_CHECK(cudaStreamCreateWithFlags(&g_capture_stream[dev], cudaStreamNonBlocking));
  GraphEntry& fresh = *hit;
  cudaGraph_t graph = nullptr;
  int rc = OK;
  if (cudaStreamBeginCapture(g_capture_stream[dev], cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
    set_launch_recorder(fresh.counts);
    rc = ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, g_capture_stream[dev], &fresh.result_index, upd);
    set_launch_recorder(nullptr);
    const cudaError_t ended = cudaStreamEndCapture(g_capture_stream[dev], &graph);
    // The launches above were only recorded: take them out of the process totals again; the
    // replay below (or the direct launch) counts them.
    int64_t undo[K_KIND_COUNT];
    for (int k = 0; k < K_KIND_COUNT; ++k) undo[k] = -fresh.counts[k];
    add_launch_counts(undo);
    if (rc != OK) {
      // A launcher refused (bad argument, or a call the capture does not allow): no graph for
      // these buffers; the direct launch reports the error, if it is one, on the caller's stream.
      if (graph) cudaGraphDestroy(graph);
      (void)cudaGetLastError();
      fresh.failed = true;
      for (int k = 0; k < K_KIND_COUNT; ++k) fresh.counts[k] = 0;
      return ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, stream, result_index, upd);
    }
    if (ended != cudaSuccess || !graph ||
        cudaGraphInstantiate(&fresh.exec, graph, 0) != cudaSuccess) {
      fresh.exec = nullptr;
    }
    if (graph) cudaGraphDestroy(graph);
  }
  (void)cudaGetLastError();
  if (!fresh.exec) {
    fresh.failed = true;
    return ns_iterate(buf, batch, m, n, mode, steps, coeffs, eps, stream, result_index, upd);
  }
  MB_CUDA_CHECK(cudaGraphLaunch(fresh.exec, stream));
  add_launch_counts(fresh.counts);
  if (result_index) *result_index = fresh.result_index;
  return OK;
}

}  // namespace mb
