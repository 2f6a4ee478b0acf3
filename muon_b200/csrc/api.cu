// C-ABI layer of libmuon_b200: argument checking, the Newton-Schulz driver and the
// composition prologue -> NS -> epilogue. Declarations and the reference lines each
// entry point replaces are in include/muon_b200.h.
#include "../../include/muon_b200.h"

#include "common.cuh"
#include "elementwise.h"
#include "ns_driver.h"
#include "ns_gemm.h"
#include "profiling.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

namespace mb {

namespace {
thread_local char t_err[512] = "";
}

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
  return code;
}
const char* last_error() { return t_err; }

namespace {

inline int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }
inline cudaStream_t as_stream(muon_b200_stream_t s) { return static_cast<cudaStream_t>(s); }
inline __nv_bfloat16* bf(void* p) { return static_cast<__nv_bfloat16*>(p); }
inline const __nv_bfloat16* bf(const void* p) { return static_cast<const __nv_bfloat16*>(p); }

int check_dtype(int dtype) {
  if (dtype != DT_F32 && dtype != DT_BF16 && dtype != DT_F16)
    return set_error(ERR_INVALID_ARG, "dtype must be MUON_B200_F32, MUON_B200_BF16 or MUON_B200_F16 (got %d)",
                     dtype);
  return OK;
}

bool all_aligned16(void* const* ptrs, int n) {
  for (int i = 0; i < n; ++i)
    if (reinterpret_cast<uintptr_t>(ptrs[i]) & 15) return false;
  return true;
}

}  // namespace
}  // namespace mb

using namespace mb;

extern "C" {

int muon_b200_version(void) { return 100; }

const char* muon_b200_last_error(void) { return last_error(); }

int muon_b200_device_status(int* status_out, int reset) {
  int st = 0;
  int rc = read_device_status(&st);
  if (rc != OK) return rc;
  if (status_out) *status_out = st;
  if (reset && st != 0 && (rc = clear_device_status()) != OK) return rc;
  if (st != 0)
    return set_error(ERR_DEVICE_TIMEOUT, "a kernel gave up on a bounded wait (device status %d)",
                     st);
  return OK;
}

int muon_b200_set_reserved_sms(int n) {
  if (n < 0) return set_error(ERR_INVALID_ARG, "reserved SM count must be >= 0");
  set_reserved_sms(n);
  return OK;
}

int muon_b200_get_reserved_sms(void) { return get_reserved_sms(); }

int muon_b200_set_graph_replay(int on) {
  set_graph_replay(on != 0);
  return OK;
}

int muon_b200_get_graph_replay(void) { return graph_replay_enabled() ? 1 : 0; }

int muon_b200_kernel_kinds(void) { return K_KIND_COUNT; }

int muon_b200_launch_counts(int64_t* counts, int n_kinds) {
  if (!counts || n_kinds < 0) return set_error(ERR_INVALID_ARG, "launch_counts: bad arguments");
  launch_counts(counts, n_kinds);
  return OK;
}

int muon_b200_timing_enable(int on) {
  timing_enable(on != 0);
  return OK;
}

int muon_b200_timing_collect(double* ms, double* work, int64_t* launches, int n_kinds) {
  if (!ms || !work || !launches || n_kinds < 0)
    return set_error(ERR_INVALID_ARG, "timing_collect: bad arguments");
  return timing_collect(ms, work, launches, n_kinds);
}

int muon_b200_timing_collect_records(int max_records, int* kinds, int64_t* tags, double* ms,
                                     double* work, int* n_out) {
  if (max_records < 0 || !kinds || !tags || !ms || !work || !n_out)
    return set_error(ERR_INVALID_ARG, "timing_collect_records: bad arguments");
  return timing_collect_records(max_records, kinds, tags, ms, work, n_out);
}

int muon_b200_ns_line1(const void* x, int64_t ldx, int64_t x_bs, void* a_out, int64_t lda,
                       int64_t a_bs, int batch, int64_t m, int64_t k, muon_b200_stream_t stream) {
  return launch_ns_gemm(MODE_SYRK, bf(x), ldx, x_bs, bf(x), ldx, x_bs, bf(a_out), lda, a_bs, batch,
                        m, m, k, 1.f, 0.f, 1, as_stream(stream));
}

int64_t muon_b200_ns_line1_scratch_bytes(int batch, int64_t m, int64_t k) {
  return splitk_scratch_bytes(batch, m, k);
}

int muon_b200_ns_line1_scratch(const void* x, int64_t ldx, int64_t x_bs, void* a_out, int64_t lda,
                               int64_t a_bs, int batch, int64_t m, int64_t k, void* scratch,
                               int64_t scratch_bytes, muon_b200_stream_t stream) {
  SplitK sk;
  sk.partial = static_cast<float*>(scratch);
  sk.bytes = scratch ? scratch_bytes : 0;
  return launch_ns_gemm(MODE_SYRK, bf(x), ldx, x_bs, bf(x), ldx, x_bs, bf(a_out), lda, a_bs, batch,
                        m, m, k, 1.f, 0.f, 1, as_stream(stream), nullptr, nullptr, 0, nullptr, nullptr, nullptr,
                        &sk);
}

int muon_b200_ns_line2(const void* a, int64_t lda, int64_t a_bs, void* b_out, int64_t ldb,
                       int64_t b_bs, int batch, int64_t m, float alpha, float beta,
                       int a_is_symmetric, muon_b200_stream_t stream) {
  if (a == b_out) return set_error(ERR_INVALID_ARG, "ns_line2 output must not alias its input");
  return launch_ns_gemm(MODE_AXPBY, bf(a), lda, a_bs, bf(a), lda, a_bs, bf(b_out), ldb, b_bs, batch,
                        m, m, m, alpha, beta, a_is_symmetric ? 1 : 0, as_stream(stream));
}

int muon_b200_ns_line3(const void* b, int64_t ldb, int64_t b_bs, const void* x, int64_t ldx,
                       int64_t x_bs, void* out, int64_t ldo, int64_t o_bs, int batch, int64_t m,
                       int64_t n, float a, muon_b200_stream_t stream) {
  if (x == out) return set_error(ERR_INVALID_ARG, "ns_line3 output must not alias X");
  return launch_ns_gemm(MODE_BX, bf(b), ldb, b_bs, bf(x), ldx, x_bs, bf(out), ldo, o_bs, batch, m,
                        n, m, a, 0.f, 0, as_stream(stream));
}

int muon_b200_ns_workspace_layout(int batch, int64_t m, int64_t n, muon_b200_ns_layout* out) {
  return muon_b200_ns_workspace_layout_mode(batch, m, n, MUON_B200_NS_AOL4, out);
}

int muon_b200_ns_workspace_layout_mode(int batch, int64_t m, int64_t n, int mode, muon_b200_ns_layout* out) {
  if (!out) return set_error(ERR_INVALID_ARG, "layout output is NULL");
  if (batch < 1 || m < 1 || n < 1)
    return set_error(ERR_INVALID_ARG, "workspace layout needs batch, m, n >= 1");
  if (m > n) return set_error(ERR_INVALID_ARG, "NS works on m x n with m <= n (got %lld x %lld)",
                              (long long)m, (long long)n);
  muon_b200_ns_layout l;
  l.ldn = round_up(n, 8);
  l.ldm = round_up(m, 8);
  l.x_bs = m * l.ldn;
  l.a_bs = m * l.ldm;
  const int64_t xb = round_up(batch * l.x_bs * 2, 256);
  const int64_t ab = round_up(batch * l.a_bs * 2, 256);
  l.x_offset_bytes = 0;
  l.c_offset_bytes = xb;
  l.a_offset_bytes = 2 * xb;
  l.b_offset_bytes = 2 * xb + ab;
  l.partials_offset_bytes = 2 * xb + 2 * ab;
  // fp32 scratch per matrix: Frobenius partial sums (classic) or the AOL row sums s (m floats).
  const int64_t per_matrix = l.ldm > kFroChunksMax ? l.ldm : kFroChunksMax;
  l.total_bytes = l.partials_offset_bytes + round_up((int64_t)batch * per_matrix * 4, 256);
  l.x8_offset_bytes = l.e8_offset_bytes = 0;
  l.ld8n = fp8_pitch(n);
  l.ld8m = fp8_pitch(m);
  if (mode == MUON_B200_NS_AOL4_FP8) {
    l.x8_offset_bytes = l.total_bytes;
    l.e8_offset_bytes = l.x8_offset_bytes + round_up(batch * m * l.ld8n, 256);
    l.total_bytes += ns_fp8_extra_bytes(batch, m, n);
  }
  l.sumsq_offset_bytes = l.sumsq_bs = 0;
  if (mode == MUON_B200_NS_CLASSIC5) {
    l.sumsq_offset_bytes = l.total_bytes;
    l.sumsq_bs = classic_tiles_max(m, n);
    l.total_bytes += ns_classic_extra_bytes(batch, m, n);
  }
  *out = l;
  return OK;
}

namespace {
// Buffers of a Newton-Schulz run inside a workspace laid out by muon_b200_ns_workspace_layout_mode.
int workspace_buffers(void* workspace, int batch, int64_t m, int64_t n, int mode, NsBuffers* out,
                      muon_b200_ns_layout* layout) {
  if (!workspace) return set_error(ERR_INVALID_ARG, "workspace is NULL");
  if (reinterpret_cast<uintptr_t>(workspace) & 255)
    return set_error(ERR_ALIGNMENT, "NS workspace must be 256-byte aligned");
  muon_b200_ns_layout l;
  int rc = muon_b200_ns_workspace_layout_mode(batch, m, n, mode, &l);
  if (rc != OK) return rc;
  char* ws = static_cast<char*>(workspace);
  NsBuffers buf{};
  if (mode == MUON_B200_NS_AOL4_FP8) {
    buf.x8 = reinterpret_cast<uint8_t*>(ws + l.x8_offset_bytes);
    buf.e8 = reinterpret_cast<uint8_t*>(ws + l.e8_offset_bytes);
    buf.ld8n = l.ld8n;
    buf.ld8m = l.ld8m;
    buf.x8_bs = m * l.ld8n;
    buf.e8_bs = m * l.ld8m;
  }
  buf.x[0] = bf(static_cast<void*>(ws + l.x_offset_bytes));
  buf.x[1] = bf(static_cast<void*>(ws + l.c_offset_bytes));
  buf.ldx[0] = buf.ldx[1] = l.ldn;
  buf.x_bs[0] = buf.x_bs[1] = l.x_bs;
  buf.A = bf(static_cast<void*>(ws + l.a_offset_bytes));
  // A / s lives in slot C: it is free until the first line 3 writes it, and m <= n.
  buf.A_scaled = buf.x[1];
  buf.B = bf(static_cast<void*>(ws + l.b_offset_bytes));
  buf.ldm = l.ldm;
  buf.a_bs = l.a_bs;
  buf.fscratch = reinterpret_cast<float*>(ws + l.partials_offset_bytes);
  buf.f_bs = l.ldm;
  buf.fro_scales = fro_scales_in(buf.fscratch, batch, l.ldm);
  *out = buf;
  if (layout) *layout = l;
  return OK;
}
}  // namespace

namespace {
// MUON_B200_NS_HAVE_SUMSQ: takes the flag off `mode`; with it, points the buffers at the per-tile
// sums of squares that muon_b200_prologue_sumsq left in the workspace.
int take_sumsq_flag(int* mode, bool* have) {
  *have = (*mode & MUON_B200_NS_HAVE_SUMSQ) != 0;
  *mode &= ~MUON_B200_NS_HAVE_SUMSQ;
  if (*have && *mode != MUON_B200_NS_CLASSIC5)
    return set_error(ERR_INVALID_ARG, "MUON_B200_NS_HAVE_SUMSQ goes with MUON_B200_NS_CLASSIC5 only");
  return OK;
}
void use_tile_sumsq(void* workspace, const muon_b200_ns_layout& l, NsBuffers* buf) {
  buf->tile_sumsq = reinterpret_cast<const float*>(static_cast<char*>(workspace) + l.sumsq_offset_bytes);
  buf->tile_bs = l.sumsq_bs;
  buf->tile_count = l.sumsq_bs;  // the prologue entry point zeroed what its kernel does not write
}
}  // namespace

int muon_b200_ns_run(void* workspace, int batch, int64_t m, int64_t n, int mode, int steps,
                     const float* coeffs, float eps, int* result_slot, muon_b200_stream_t stream) {
  bool have_sumsq = false;
  int rc = take_sumsq_flag(&mode, &have_sumsq);
  if (rc != OK) return rc;
  rc = ns_check_mode(mode, &steps, coeffs);
  if (rc != OK) return rc;
  NsBuffers buf;
  muon_b200_ns_layout l;
  rc = workspace_buffers(workspace, batch, m, n, mode, &buf, &l);
  if (rc != OK) return rc;
  if (have_sumsq) use_tile_sumsq(workspace, l, &buf);
  return ns_iterate_replayed(buf, batch, m, n, mode, steps, coeffs, eps, as_stream(stream), result_slot);
}

int muon_b200_ns_run_update(void* workspace, int mode, int steps, const float* coeffs, float eps,
                            void* const* params, int count, int64_t rows, int64_t cols, int dtype,
                            double lr, double weight_decay, double scale, muon_b200_stream_t stream) {
  int rc = check_dtype(dtype);
  if (rc != OK) return rc;
  if (!params) return set_error(ERR_INVALID_ARG, "ns_run_update: params is NULL");
  if (count < 1 || rows < 1 || cols < 1)
    return set_error(ERR_INVALID_ARG, "ns_run_update needs count, rows, cols >= 1");
  bool have_sumsq = false;
  rc = take_sumsq_flag(&mode, &have_sumsq);
  if (rc != OK) return rc;
  rc = ns_check_mode(mode, &steps, coeffs);
  if (rc != OK) return rc;
  const bool tall = rows > cols;
  const int64_t m = tall ? cols : rows, n = tall ? rows : cols;
  NsBuffers buf;
  muon_b200_ns_layout l;
  rc = workspace_buffers(workspace, count, m, n, mode, &buf, &l);
  if (rc != OK) return rc;
  if (have_sumsq) use_tile_sumsq(workspace, l, &buf);
  UpdateSpec upd;
  upd.param = params;
  upd.dtype = dtype;
  upd.rows = rows;
  upd.cols = cols;
  upd.scale = (float)scale;
  upd.decay = (float)(1.0 - lr * weight_decay);
  upd.neg_lr = (float)(-lr);
  // (a one-step classic iteration: its only line 3 carries the normalisation factor instead)
  if (update_fusable(upd, count) && !(mode == MUON_B200_NS_CLASSIC5 && steps == 1))
    return ns_iterate_replayed(buf, count, m, n, mode, steps, coeffs, eps, as_stream(stream), nullptr, &upd);
  // Not fusable (tall fp32 parameters, more than 64 of them, rows that are not 16-byte multiples):
  // the iteration, then the update kernel on the same stream.
  int slot = 0;
  rc = ns_iterate_replayed(buf, count, m, n, mode, steps, coeffs, eps, as_stream(stream), &slot);
  if (rc != OK) return rc;
  return muon_b200_epilogue(params, count, rows, cols, dtype, buf.x[slot], l.ldn, l.x_bs, tall ? 1 : 0, lr,
                            weight_decay, scale, stream);
}

int64_t muon_b200_zeropower_scratch_bytes(int batch, int64_t rows, int64_t cols, int mode) {
  return rows <= cols ? ns_scratch_bytes(batch, rows, cols, mode, true) : ns_scratch_bytes(batch, cols, rows, mode, true);
}

int muon_b200_zeropower(const void* g, int dtype, int64_t rows, int64_t cols, int64_t ldg, int64_t g_bs,
                        int batch, void* out, int64_t ldo, int64_t o_bs, void* scratch,
                        int64_t scratch_bytes, int mode, int steps, const float* coeffs, float eps,
                        muon_b200_stream_t stream) {
  if (!g || !out || !scratch) return set_error(ERR_INVALID_ARG, "zeropower: null pointer");
  if (dtype < DT_F32 || dtype > DT_F64) return set_error(ERR_INVALID_ARG, "zeropower: unknown element type %d", dtype);
  if (batch < 1 || rows < 1 || cols < 1 || rows > INT32_MAX || cols > INT32_MAX)
    return set_error(ERR_INVALID_ARG, "zeropower needs batch, rows, cols >= 1");
  int rc = ns_check_mode(mode, &steps, coeffs);
  if (rc != OK) return rc;
  const int64_t m = rows <= cols ? rows : cols, n = rows <= cols ? cols : rows;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (ldo % 8) || (o_bs % 8) || ldo < n ||
      (batch > 1 && o_bs < (m - 1) * ldo + n))
    return set_error(ERR_ALIGNMENT, "zeropower: out must be 16-byte aligned with pitches %% 8 == 0 and >= n");
  if (ldg < cols || (batch > 1 && g_bs < (rows - 1) * ldg + cols))
    return set_error(ERR_INVALID_ARG, "zeropower: input pitch shorter than a row or a matrix");
  if (reinterpret_cast<uintptr_t>(scratch) & 255)
    return set_error(ERR_ALIGNMENT, "zeropower: scratch must be 256-byte aligned");
  const int64_t need = ns_scratch_bytes(batch, m, n, mode, true);
  if (scratch_bytes < need)
    return set_error(ERR_INVALID_ARG, "zeropower: scratch too small: %lld bytes given, %lld needed",
                     (long long)scratch_bytes, (long long)need);
  return ns_run_with_scratch(g, dtype, rows, cols, ldg, g_bs, bf(out), ldo, o_bs,
                             static_cast<unsigned char*>(scratch), batch, mode, steps, coeffs, eps,
                             /*replay=*/true, as_stream(stream), /*split_k=*/true);
}

int muon_b200_cast_bf16(const void* src, int dtype, int64_t rows, int64_t cols, int64_t ld_src,
                        int64_t src_bs, void* dst, int64_t ld_dst, int64_t dst_bs, int batch,
                        int transpose, float scale, muon_b200_stream_t stream) {
  if (!src || !dst) return set_error(ERR_INVALID_ARG, "cast: null pointer");
  if (batch < 1 || rows < 1 || cols < 1 || rows > INT32_MAX || cols > INT32_MAX)
    return set_error(ERR_INVALID_ARG, "cast needs batch, rows, cols >= 1");
  if (ld_src < cols || ld_dst < (transpose ? rows : cols))
    return set_error(ERR_INVALID_ARG, "cast: pitch shorter than a row");
  return launch_cast_bf16(src, dtype, ld_src, src_bs, bf(dst), ld_dst, dst_bs, (int)rows, (int)cols, batch,
                          transpose ? 1 : 0, scale, as_stream(stream));
}

int muon_b200_prologue(void* const* grads, void* const* moms, int count, int64_t rows,
                       int64_t cols, int dtype, double beta, int nesterov, void* x, int64_t ldx,
                       int64_t x_bs, int transpose_out, muon_b200_stream_t stream) {
  return muon_b200_prologue_sumsq(grads, moms, count, rows, cols, dtype, beta, nesterov, x, ldx, x_bs,
                                  transpose_out, nullptr, 0, stream);
}

int muon_b200_prologue_sumsq(void* const* grads, void* const* moms, int count, int64_t rows,
                             int64_t cols, int dtype, double beta, int nesterov, void* x, int64_t ldx,
                             int64_t x_bs, int transpose_out, float* sumsq, int64_t sumsq_bs,
                             muon_b200_stream_t stream) {
  int rc = check_dtype(dtype);
  if (rc != OK) return rc;
  if (!grads || !moms || !x) return set_error(ERR_INVALID_ARG, "null pointer passed to prologue");
  if (count < 1 || rows < 1 || cols < 1 || rows > INT32_MAX || cols > INT32_MAX)
    return set_error(ERR_INVALID_ARG, "prologue needs count, rows, cols >= 1");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (ldx % 8) || (x_bs % 8))
    return set_error(ERR_ALIGNMENT, "prologue X must be 16-byte aligned with pitches %% 8 == 0");
  if (ldx < (transpose_out ? rows : cols))
    return set_error(ERR_INVALID_ARG, "prologue X pitch %lld is shorter than a row", (long long)ldx);
  const int vec = dtype == DT_F32 ? 4 : 8;
  if (sumsq) {
    const int tiles = prologue_tiles((int)rows, (int)cols, dtype);
    if (sumsq_bs < tiles)
      return set_error(ERR_INVALID_ARG, "prologue: %lld sums of squares per tensor, the kernel writes %d",
                       (long long)sumsq_bs, tiles);
    // entries past the kernel's tiles count as zero when the sums are added up
    if (sumsq_bs > tiles)
      MB_CUDA_CHECK(cudaMemsetAsync(sumsq, 0, sizeof(float) * (size_t)sumsq_bs * count, as_stream(stream)));
  }
  for (int base = 0; base < count; base += kMaxTensors) {
    const int n = count - base < kMaxTensors ? count - base : kMaxTensors;
    PrologueArgs a{};
    for (int i = 0; i < n; ++i) {
      if (!grads[base + i] || !moms[base + i])
        return set_error(ERR_INVALID_ARG, "prologue tensor %d has a null pointer", base + i);
      a.grad[i] = grads[base + i];
      a.mom[i] = moms[base + i];
    }
    a.x = bf(x) + (int64_t)base * x_bs;
    a.x_bs = x_bs;
    a.ldx = ldx;
    a.count = n;
    a.rows = (int)rows;
    a.cols = (int)cols;
    a.nesterov = nesterov ? 1 : 0;
    a.vec_ok = (cols % vec == 0) && all_aligned16(grads + base, n) && all_aligned16(moms + base, n);
    a.w_mom = (float)(1.0 - beta);
    a.beta = (float)beta;
    a.sumsq = sumsq ? sumsq + (int64_t)base * sumsq_bs : nullptr;
    a.sumsq_bs = sumsq_bs;
    rc = launch_prologue(a, dtype, transpose_out ? 1 : 0, as_stream(stream));
    if (rc != OK) return rc;
  }
  return OK;
}

int muon_b200_epilogue_push(void* const* params, void* const* peer_params, int n_peers, int count,
                            int64_t rows, int64_t cols, int dtype, const void* u, int64_t ldu,
                            int64_t u_bs, int u_transposed, double lr, double weight_decay,
                            double scale, muon_b200_stream_t stream) {
  int rc = check_dtype(dtype);
  if (rc != OK) return rc;
  if (!params || !u) return set_error(ERR_INVALID_ARG, "null pointer passed to epilogue");
  if (count < 1 || rows < 1 || cols < 1 || rows > INT32_MAX || cols > INT32_MAX)
    return set_error(ERR_INVALID_ARG, "epilogue needs count, rows, cols >= 1");
  if (n_peers < 0 || n_peers > kMaxPeers || (n_peers > 0 && !peer_params))
    return set_error(ERR_INVALID_ARG, "epilogue: between 0 and %d peer copies per parameter (got %d)",
                     kMaxPeers, n_peers);
  if ((reinterpret_cast<uintptr_t>(u) & 15) || (ldu % 8) || (u_bs % 8))
    return set_error(ERR_ALIGNMENT, "epilogue U must be 16-byte aligned with pitches %% 8 == 0");
  const int vec = dtype == DT_F32 ? 4 : 8;
  for (int base = 0; base < count; base += kMaxTensors) {
    const int n = count - base < kMaxTensors ? count - base : kMaxTensors;
    EpilogueArgs a{};
    EpiloguePeers peers{};
    peers.n_peers = n_peers;
    bool aligned = (cols % vec == 0) && all_aligned16(params + base, n);
    for (int i = 0; i < n; ++i) {
      if (!params[base + i])
        return set_error(ERR_INVALID_ARG, "epilogue tensor %d has a null pointer", base + i);
      a.param[i] = params[base + i];
      for (int r = 0; r < n_peers; ++r) {
        void* q = peer_params[(int64_t)r * count + base + i];
        if (!q) return set_error(ERR_INVALID_ARG, "epilogue tensor %d has a null peer pointer", base + i);
        peers.param[r][i] = q;
        aligned = aligned && (reinterpret_cast<uintptr_t>(q) & 15) == 0;
      }
    }
    a.u = bf(u) + (int64_t)base * u_bs;
    a.u_bs = u_bs;
    a.ldu = ldu;
    a.count = n;
    a.rows = (int)rows;
    a.cols = (int)cols;
    a.vec_ok = aligned;
    a.scale = (float)scale;
    a.decay = (float)(1.0 - lr * weight_decay);
    a.neg_lr = (float)(-lr);
    rc = launch_epilogue(a, dtype, u_transposed ? 1 : 0, as_stream(stream), n_peers > 0 ? &peers : nullptr);
    if (rc != OK) return rc;
  }
  return OK;
}

int muon_b200_epilogue(void* const* params, int count, int64_t rows, int64_t cols, int dtype,
                       const void* u, int64_t ldu, int64_t u_bs, int u_transposed, double lr,
                       double weight_decay, double scale, muon_b200_stream_t stream) {
  return muon_b200_epilogue_push(params, nullptr, 0, count, rows, cols, dtype, u, ldu, u_bs, u_transposed,
                                 lr, weight_decay, scale, stream);
}

int muon_b200_muon_step(void* const* params, void* const* grads, void* const* moms, int count,
                        int64_t rows, int64_t cols, int dtype, double lr, double weight_decay,
                        double beta, int nesterov, double scale, int ns_mode, int ns_steps,
                        const float* ns_coeffs, float ns_eps, void* workspace,
                        int64_t workspace_bytes, muon_b200_stream_t stream) {
  if (count < 1 || rows < 1 || cols < 1)
    return set_error(ERR_INVALID_ARG, "muon_step needs count, rows, cols >= 1");
  if (!workspace) return set_error(ERR_INVALID_ARG, "workspace is NULL");
  const bool tall = rows > cols;  // the iteration runs on the transposed matrix (muon.py:761-762)
  const int64_t m = tall ? cols : rows;
  const int64_t n = tall ? rows : cols;
  muon_b200_ns_layout l;
  int rc = muon_b200_ns_workspace_layout_mode(count, m, n, ns_mode, &l);
  if (rc != OK) return rc;
  if (workspace_bytes < l.total_bytes)
    return set_error(ERR_INVALID_ARG, "workspace too small: %lld bytes given, %lld needed",
                     (long long)workspace_bytes, (long long)l.total_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) & 255)
    return set_error(ERR_ALIGNMENT, "NS workspace must be 256-byte aligned");
  char* ws = static_cast<char*>(workspace);
  // classic iteration: the prologue kernel sums the squares of X while it writes it (muon.py:282)
  const bool classic = ns_mode == MUON_B200_NS_CLASSIC5;
  rc = muon_b200_prologue_sumsq(grads, moms, count, rows, cols, dtype, beta, nesterov,
                                ws + l.x_offset_bytes, l.ldn, l.x_bs, tall ? 1 : 0,
                                classic ? reinterpret_cast<float*>(ws + l.sumsq_offset_bytes) : nullptr,
                                l.sumsq_bs, stream);
  if (rc != OK) return rc;
  return muon_b200_ns_run_update(workspace, classic ? (ns_mode | MUON_B200_NS_HAVE_SUMSQ) : ns_mode, ns_steps,
                                 ns_coeffs, ns_eps, params, count, rows, cols, dtype, lr, weight_decay, scale,
                                 stream);
}

int muon_b200_adam(void* const* params, void* const* grads, void* const* exp_avg,
                   void* const* exp_avg_sq, const int64_t* numel, const int64_t* steps, int count,
                   int dtype, double lr, double weight_decay, double beta1, double beta2,
                   double eps, muon_b200_stream_t stream) {
  int rc = check_dtype(dtype);
  if (rc != OK) return rc;
  if (!params || !grads || !exp_avg || !exp_avg_sq || !numel || !steps)
    return set_error(ERR_INVALID_ARG, "null pointer passed to adam");
  if (count < 0) return set_error(ERR_INVALID_ARG, "adam count is negative");
  int sms = 0;
  if ((rc = device_sm_count(&sms)) != OK) return rc;
  const int per_block = adam_elems_per_block(dtype);
  const int vec = dtype == DT_F32 ? 4 : 8;
  (void)vec;
  for (int base = 0; base < count; base += kMaxTensors) {
    const int n = count - base < kMaxTensors ? count - base : kMaxTensors;
    AdamArgs a{};
    a.count = n;
    a.block_start[0] = 0;
    for (int i = 0; i < n; ++i) {
      const int k = base + i;
      if (!params[k] || !grads[k] || !exp_avg[k] || !exp_avg_sq[k])
        return set_error(ERR_INVALID_ARG, "adam tensor %d has a null pointer", k);
      if (numel[k] < 0 || steps[k] < 1)
        return set_error(ERR_INVALID_ARG, "adam tensor %d: numel must be >= 0 and step >= 1", k);
      a.param[i] = params[k];
      a.grad[i] = grads[k];
      a.exp_avg[i] = exp_avg[k];
      a.exp_avg_sq[i] = exp_avg_sq[k];
      a.numel[i] = numel[k];
      a.bc1[i] = (float)(1.0 - std::pow(beta1, (double)steps[k]));
      a.bc2[i] = (float)(1.0 - std::pow(beta2, (double)steps[k]));
      const uintptr_t bits = reinterpret_cast<uintptr_t>(params[k]) |
                             reinterpret_cast<uintptr_t>(grads[k]) |
                             reinterpret_cast<uintptr_t>(exp_avg[k]) |
                             reinterpret_cast<uintptr_t>(exp_avg_sq[k]);
      a.vec_ok[i] = (bits & 15) == 0;
      const int64_t blocks = (numel[k] + per_block - 1) / per_block;
      if (blocks + a.block_start[i] > INT32_MAX)
        return set_error(ERR_UNSUPPORTED, "adam tensor %d is too large for one launch", k);
      a.block_start[i + 1] = a.block_start[i] + (int)blocks;
    }
    a.w1 = (float)(1.0 - beta1);
    a.w2 = (float)(1.0 - beta2);
    a.eps = (float)eps;
    a.decay = (float)(1.0 - lr * weight_decay);
    a.neg_lr = (float)(-lr);
    rc = launch_adam(a, dtype, as_stream(stream));
    if (rc != OK) return rc;
  }
  return OK;
}

}  // extern "C"
