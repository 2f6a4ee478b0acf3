/*
 * muon_b200 — C ABI of the B200 (sm_100a) Muon optimizer-step library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream; nothing here
 * depends on PyTorch. All work is enqueued on the given stream and no entry point
 * synchronises, except muon_b200_device_status. Unless stated otherwise the library
 * neither allocates nor frees device memory: buffers, workspaces included, belong to
 * the caller.
 *
 * Return value: 0 on success, a negative code on failure (see MUON_B200_ERR_*); the
 * text of the last failure on the calling thread is available from
 * muon_b200_last_error(). There is no CPU fallback: on a device that is not sm_100
 * every compute entry point fails with MUON_B200_ERR_UNSUPPORTED.
 *
 * "Reference" citations are file:line of thib-s/Muon's muon.py, the module whose
 * functions these entry points replace.
 */
#ifndef MUON_B200_H_
#define MUON_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MUON_B200_OK 0
#define MUON_B200_ERR_INVALID_ARG (-1)
#define MUON_B200_ERR_ALIGNMENT (-2)
#define MUON_B200_ERR_CUDA (-3)
#define MUON_B200_ERR_UNSUPPORTED (-4)
#define MUON_B200_ERR_DEVICE_TIMEOUT (-5)

/* Element types. Parameters, gradients and optimizer state (prologue, epilogue, muon_step, adam)
 * are float32, bfloat16 or float16 (the update is fused into the last GEMM for the first two; a
 * float16 parameter gets the update kernel). The reference's elementwise code would also run on
 * float64 parameters (muon.py:9-10, :66-67, :105-109); this library computes in float32 registers
 * and does not take them. The input of muon_b200_zeropower and muon_b200_cast_bf16 may be any of
 * the four, like the cast at muon.py:760. */
#define MUON_B200_F32 0
#define MUON_B200_BF16 1
#define MUON_B200_F16 2
#define MUON_B200_F64 3

/* Newton-Schulz variants. AOL4 is what the reference executes (muon.py:748-799);
 * CLASSIC5 is the Frobenius-normalised quintic iteration the reference documents in
 * its commented block (muon.py:263-291). */
#define MUON_B200_NS_AOL4 0
#define MUON_B200_NS_CLASSIC5 1
/* AOL4 with the two symmetric products of iterations 2..4 taken in 8-bit floating point (e4m3,
 * fp32 accumulation, twice the tensor-core rate): line 1 multiplies e4m3(X * 2^k), line 2 is
 * rewritten as c*E*E + (b + 2c)*A - c*I with E = A - I so that only the small matrix E is
 * quantised; the first iteration (which fixes the row scales) and every line 3 stay in bf16.
 * No counterpart in the reference. Its output differs from AOL4's by about 1e-2 relative
 * Frobenius norm on wide and tall matrices (singular values within [0.97, 1.035] instead of
 * [0.985, 1.015]) and by up to 4e-2 on square ones; matrices with fewer than 1024 columns
 * (after transposing tall ones) are iterated in bf16 in this mode too, because the rounding noise
 * of an e4m3 Gram entry only averages out over a long row. It is off unless asked for. */
#define MUON_B200_NS_AOL4_FP8 2

/* Upper bound on tensors per call of the multi-tensor entry points is unlimited;
 * internally they are processed in launches of this many. */
#define MUON_B200_TENSORS_PER_LAUNCH 32

typedef void* muon_b200_stream_t; /* a cudaStream_t */

/* Library version as major*10000 + minor*100 + patch. */
int muon_b200_version(void);

/* Message of the last error raised on the calling thread ("" if none). */
const char* muon_b200_last_error(void);

/* Synchronises the current device and reads the device-side status word that kernels
 * set when a bounded wait inside them runs out (0 = healthy). If reset != 0 the word
 * is cleared afterwards. Returns MUON_B200_ERR_DEVICE_TIMEOUT when the word is set. */
int muon_b200_device_status(int* status_out, int reset);

/* The Newton-Schulz GEMMs run as persistent grids that fill the device. A caller that runs
 * other kernels concurrently on another stream (the copy kernels of a collective that overlaps
 * the step) can ask the grids to leave n SMs free. Process-wide, default 0. No counterpart in
 * the reference. */
int muon_b200_set_reserved_sms(int n);
int muon_b200_get_reserved_sms(void);

/* A short Newton-Schulz run (a few matrices of a few hundred rows) is thirteen kernels of a few
 * microseconds each; issued one by one they cost more host time than device time. By default
 * muon_b200_ns_run (and muon_b200_muon_step, which calls it) therefore captures its launch
 * sequence into a CUDA graph the first time it sees a given workspace address, batch, shape,
 * mode and coefficient list, and replays the graph afterwards; runs with more than about 2 TFLOP
 * of work, streams that are themselves being captured and per-kernel timing use plain launches.
 * Graph instantiation allocates driver resources (this is the other exception to "never
 * allocates"; muon_b200_ns_run_static never uses it). Process-wide switch, default on; the
 * environment variable MUON_B200_GRAPH=0 sets the default to off. No counterpart in the
 * reference, whose driver is compiled by torch.compile (muon.py:748). */
int muon_b200_set_graph_replay(int on);
int muon_b200_get_graph_replay(void);

/* ---- Peer memory for the distributed step's exchange ---------------------------------
 * These four are the exceptions to "never allocates, never maps": they create and remove
 * address-space mappings of OTHER processes' device memory. They have no counterpart in the
 * reference, whose exchange is dist.all_gather (muon.py:68). */

/* Exports the cudaMalloc allocation that contains ptr: writes the 64-byte CUDA IPC handle, the
 * offset of ptr inside that allocation and (optionally) the allocation's size. */
int muon_b200_ipc_export(const void* ptr, void* handle64, int64_t* offset_out,
                         int64_t* alloc_bytes_out);
/* Maps a peer process's allocation on the CURRENT device with peer access enabled and returns
 * its base address. A process must open a given handle only once (cache by the 64 bytes). */
int muon_b200_ipc_open(const void* handle64, void** base_out);
int muon_b200_ipc_close(void* base);
/* Enqueues n device-to-device copies of `bytes` bytes from src to dst[0..n) on `stream`. With
 * destinations obtained from muon_b200_ipc_open these are copy-engine transfers over NVLink
 * and occupy no SM. */
int muon_b200_push_copies(void* const* dst, int n, const void* src, int64_t bytes,
                          muon_b200_stream_t stream);

/* ---- Accounting and per-kernel timing -----------------------------------------------
 * Kernel kinds, in the order of every array below:
 *   0 NS line 1, 1 NS line 2, 2 NS line 3 (work unit: algorithmic FLOPs, symmetric products
 *   counted once), 3 prologue, 4 epilogue, 5 AOL rescale, 6 Frobenius normalise, 7 Adam
 *   (work unit: algorithmic HBM bytes). No counterpart in the reference. */
int muon_b200_kernel_kinds(void);
/* Kernel launches issued by this process since load, per kind. */
int muon_b200_launch_counts(int64_t* counts, int n_kinds);
/* While enabled, every launch is bracketed by two CUDA events recorded on the launching
 * stream. Meant for measurement runs: creating the events costs host time. */
int muon_b200_timing_enable(int on);
/* Waits for the recorded intervals; returns per kind the summed device time (ms), summed
 * work units and number of launches since the last collect, and forgets them. */
int muon_b200_timing_collect(double* ms, double* work, int64_t* launches, int n_kinds);
/* Same data, one record per launch in launch order (at most max_records; the rest is dropped).
 * tags[i] describes the launch: for the NS lines (M << 40) | (K << 16) | (batch << 4) | flags (for line 3 the K field holds N),
 * with flag bit 0 = line 2 ran with a_is_symmetric, bit 1 = two-CTA kernel; 0 for other kinds. */
int muon_b200_timing_collect_records(int max_records, int* kinds, int64_t* tags, double* ms,
                                     double* work, int* n_out);

/* ---- Newton-Schulz GEMM lines ---------------------------------------------------
 * All matrices are bf16, row-major with a pitch (ld*, in elements, multiple of 8) and a
 * batch pitch (*_bs, in elements, multiple of 8; ignored when batch == 1). Pointers
 * must be 16-byte aligned. */

/* A[b] = X[b] · X[b]ᵀ, X is m x k, A is m x m, exactly symmetric.
 * Replaces ns_line_1 (muon.py:420-456) and its kernel (muon.py:349-417). */
int muon_b200_ns_line1(const void* x, int64_t ldx, int64_t x_bs, void* a_out, int64_t lda,
                       int64_t a_bs, int batch, int64_t m, int64_t k, muon_b200_stream_t stream);

/* muon_b200_ns_line1 with a scratch area: when the product has so few output tiles that most SMs
 * would idle (one or a few matrices of a few hundred rows with a long k), the contraction is cut
 * into slices that run on different SMs, their fp32 partial sums go to `scratch`, and a second
 * launch adds them in slice order and stores the result (deterministic; differs from the unsplit
 * product only by the order of the fp32 additions). scratch: 256-byte aligned, at least
 * muon_b200_ns_line1_scratch_bytes(batch, m, k) bytes (0 = this size is never split); NULL or too
 * small: same as muon_b200_ns_line1. muon_b200_zeropower splits the same way inside its scratch
 * area; muon_b200_ns_run, muon_b200_ns_run_update, muon_b200_muon_step and
 * muon_b200_ns_run_static never split, so that what they compute for a matrix does not depend on
 * how many matrices share the call. */
int muon_b200_ns_line1_scratch(const void* x, int64_t ldx, int64_t x_bs, void* a_out, int64_t lda,
                               int64_t a_bs, int batch, int64_t m, int64_t k, void* scratch,
                               int64_t scratch_bytes, muon_b200_stream_t stream);
int64_t muon_b200_ns_line1_scratch_bytes(int batch, int64_t m, int64_t k);

/* B[b] = alpha · A[b] · A[b]ᵀ + beta · A[b], A is m x m. Only the lower triangle of the
 * product is computed and it is mirrored; the addend beta·A is taken per element, so A
 * may be non-symmetric. With a_is_symmetric != 0 the caller asserts A == Aᵀ bit for bit
 * and the kernel mirrors finished values instead of re-reading A.
 * Replaces ns_line_2 (muon.py:547-588, kernel :464-544). */
int muon_b200_ns_line2(const void* a, int64_t lda, int64_t a_bs, void* b_out, int64_t ldb,
                       int64_t b_bs, int batch, int64_t m, float alpha, float beta,
                       int a_is_symmetric, muon_b200_stream_t stream);

/* OUT[b] = a · X[b] + B[b] · X[b], B is m x m, X and OUT are m x n. OUT must not alias X.
 * Replaces ns_line_3 (muon.py:705-746, kernel :639-702). */
int muon_b200_ns_line3(const void* b, int64_t ldb, int64_t b_bs, const void* x, int64_t ldx,
                       int64_t x_bs, void* out, int64_t ldo, int64_t o_bs, int batch, int64_t m,
                       int64_t n, float a, muon_b200_stream_t stream);

/* ---- Newton-Schulz driver ---------------------------------------------------------
 * The workspace of a batch of `batch` matrices of m x n (m <= n) holds, in this order,
 * X and C ([batch, m, ldn] bf16), A and B ([batch, m, ldm] bf16) and a small fp32
 * reduction area. Layout query (all outputs in bytes / elements as named): */
typedef struct muon_b200_ns_layout {
  int64_t total_bytes;
  int64_t x_offset_bytes, c_offset_bytes, a_offset_bytes, b_offset_bytes, partials_offset_bytes;
  int64_t ldn, x_bs; /* pitch and batch pitch of X and C, in elements */
  int64_t ldm, a_bs; /* pitch and batch pitch of A and B, in elements */
  /* MUON_B200_NS_AOL4_FP8 only (0 otherwise): the e4m3 copies of X ([batch, m, ld8n] bytes) and of
   * A - I ([batch, m, ld8m] bytes) that the iteration keeps beside the bf16 matrices */
  int64_t x8_offset_bytes, e8_offset_bytes, ld8n, ld8m;
  /* MUON_B200_NS_CLASSIC5 only (0 otherwise): sumsq_bs floats per matrix, starting at
   * sumsq_offset_bytes, for the sums of squares that muon_b200_prologue_sumsq leaves */
  int64_t sumsq_offset_bytes, sumsq_bs;
} muon_b200_ns_layout;

/* Layout for MUON_B200_NS_AOL4; also enough for MUON_B200_NS_CLASSIC5 without
 * MUON_B200_NS_HAVE_SUMSQ. */
int muon_b200_ns_workspace_layout(int batch, int64_t m, int64_t n, muon_b200_ns_layout* out);
/* Layout for a given mode: MUON_B200_NS_AOL4_FP8 needs about a quarter more, MUON_B200_NS_CLASSIC5
 * a few floats per 64 x 64 elements more (the sumsq area). */
int muon_b200_ns_workspace_layout_mode(int batch, int64_t m, int64_t n, int mode, muon_b200_ns_layout* out);

/* Orthogonalises the `batch` matrices already stored (bf16, m x n, m <= n) in slot X of
 * `workspace` (laid out by muon_b200_ns_workspace_layout_mode for the same mode). mode is one of
 * the MUON_B200_NS_* constants; steps = 0 picks the mode's default (4, or 5 for CLASSIC5); coeffs is NULL or steps triples (a, b, c); eps is the clamp
 * (AOL) or the additive term (classic). On return *result_slot is 0 if the result is in
 * slot X and 1 if it is in slot C. `workspace` must be 256-byte aligned.
 * Replaces zeropower_via_newtonschulz5 (muon.py:748-799) from line 778 on. */
int muon_b200_ns_run(void* workspace, int batch, int64_t m, int64_t n, int mode, int steps,
                     const float* coeffs, float eps, int* result_slot, muon_b200_stream_t stream);

/* Flag to OR into `mode` (MUON_B200_NS_CLASSIC5 only) of muon_b200_ns_run and
 * muon_b200_ns_run_update: the X in the workspace was written by muon_b200_prologue_sumsq together
 * with its sums of squares (into the sumsq area of a workspace laid out for the classic mode), so
 * the Frobenius norm of muon.py:282 is taken from those instead of from another pass over X. In
 * either case X is not divided by its norm in memory: the first Gram product and the first
 * line 3 multiply their outputs by 1/(||X|| + eps)^2 and 1/(||X|| + eps). */
#define MUON_B200_NS_HAVE_SUMSQ 0x100

/* muon_b200_ns_run followed by the update epilogue (muon_b200_epilogue) of the `count` parameters
 * whose bf16 matrices the workspace holds, with the update done by the last GEMM of the iteration
 * itself where that is possible: its epilogue reads the parameter, applies
 * p = p*(1 - lr*wd) - lr * bf16(U*scale) with the roundings of muon_b200_epilogue and writes the
 * parameter back, so the orthogonalised matrix never goes to memory. Fused for bfloat16 parameters
 * of either orientation and for float32 parameters with rows <= cols, up to 64 per call, rows a
 * multiple of 16 bytes; otherwise the iteration is followed by the epilogue kernel on the same
 * stream. rows, cols, dtype, lr, weight_decay, scale as for muon_b200_epilogue; the workspace is
 * laid out for (count, min(rows, cols), max(rows, cols), mode). Replaces muon.py:13-14 and :66-67
 * (:98-99) for a group of parameters. */
int muon_b200_ns_run_update(void* workspace, int mode, int steps, const float* coeffs, float eps,
                            void* const* params, int count, int64_t rows, int64_t cols, int dtype,
                            double lr, double weight_decay, double scale, muon_b200_stream_t stream);

/* The whole of zeropower_via_newtonschulz5 (muon.py:748-799) in one call, with caller-owned input
 * and output: g is [batch, rows, cols] of element type dtype (MUON_B200_F32/BF16/F16/F64), pitch ldg
 * and batch pitch g_bs in elements, and is not modified. It is cast to bf16 (muon.py:760),
 * transposed when rows > cols (muon.py:761-762) and orthogonalised; out receives the result of the
 * m x n problem, m = min(rows, cols), n = max(rows, cols), as bf16 [batch, m, n] with pitch ldo >= n
 * and batch pitch o_bs (multiples of 8, out 16-byte aligned) -- for rows > cols that is the
 * transpose of the reference's return value, exactly the buffer its final .mT is a view of
 * (muon.py:797-798). scratch: 256-byte aligned, at least
 * muon_b200_zeropower_scratch_bytes(batch, rows, cols, mode) bytes, contents irrelevant before and
 * after. mode, steps, coeffs, eps as for muon_b200_ns_run; graph replay applies when the same
 * buffers come back. */
int muon_b200_zeropower(const void* g, int dtype, int64_t rows, int64_t cols, int64_t ldg, int64_t g_bs,
                        int batch, void* out, int64_t ldo, int64_t o_bs, void* scratch,
                        int64_t scratch_bytes, int mode, int steps, const float* coeffs, float eps,
                        muon_b200_stream_t stream);
int64_t muon_b200_zeropower_scratch_bytes(int batch, int64_t rows, int64_t cols, int mode);

/* dst = bf16(float(src) * scale), src [batch, rows, cols] of element type dtype, dst bf16
 * [batch, rows, cols] or, with transpose != 0, [batch, cols, rows]; pitches in elements. src and
 * dst may be the same bf16 buffer when transpose == 0 (used for the aspect scale of muon.py:14).
 * Replaces G.to(torch.bfloat16), .mT and .contiguous() (muon.py:760-764). */
int muon_b200_cast_bf16(const void* src, int dtype, int64_t rows, int64_t cols, int64_t ld_src,
                        int64_t src_bs, void* dst, int64_t ld_dst, int64_t dst_bs, int batch,
                        int transpose, float scale, muon_b200_stream_t stream);

/* Newton-Schulz for callers that cannot allocate device memory: hosts whose allocator is
 * frozen while the step runs (memory-planned graphs, fixed-budget real-time loops) and
 * plugins that are handed buffers and nothing else. Same computation as muon_b200_ns_run, but
 * the scratch (ping-pong copy of X, Gram matrix, its row-scaled copy, B, row scales) is a
 * 64 MiB array built into the library instead of a caller workspace. This entry point has no
 * counterpart in the reference.
 *   x    bf16 [batch, m, n], m <= n, pitch ldx, batch pitch x_bs (elements); not modified.
 *   out  bf16 [batch, m, n], pitch ldo, batch pitch o_bs; receives the result; its byte range
 *        must not overlap x's (checked; with an even step count out doubles as a work buffer).
 * Pointers 16-byte aligned, pitches multiples of 8 and >= n. Other arguments as muon_b200_ns_run.
 * The device that `stream` belongs to must be the current device of the calling thread: the
 * built-in array is looked up for the current device.
 * Limits and caveats:
 *   - every GPU on which the library is loaded holds the 64 MiB until the process exits;
 *   - a problem needing more than muon_b200_ns_static_scratch_bytes() is rejected with
 *     MUON_B200_ERR_UNSUPPORTED (muon_b200_ns_static_required_bytes tells how much it needs);
 *   - all calls share the one array and it keeps the previous call's contents (nothing in it
 *     has to start at zero: every part is written before it is read), so two calls that overlap
 *     on a GPU, from any streams or threads, race: serialise them;
 *   - the first call on a device looks up the array's device address; make that call before
 *     starting any stream capture.
 * Calls no cudaMalloc/cudaFree or other allocating routine. */
int muon_b200_ns_run_static(const void* x, int64_t ldx, int64_t x_bs, void* out, int64_t ldo,
                            int64_t o_bs, int batch, int64_t m, int64_t n, int mode, int steps,
                            const float* coeffs, float eps, muon_b200_stream_t stream);
int64_t muon_b200_ns_static_scratch_bytes(void);
int64_t muon_b200_ns_static_required_bytes(int batch, int64_t m, int64_t n);

/* ---- Elementwise stages, multi-tensor ------------------------------------------------
 * `count` tensors of identical shape rows x cols (a 4-D conv filter is passed as
 * rows = size(0), cols = numel / size(0), muon.py:11-12) and identical dtype. */

/* Momentum prologue, in place on grads and moms (muon.py:9-10) and bf16 cast into the NS
 * input X (muon.py:760-764): X of tensor i starts at x + i*x_bs elements, pitch ldx; with
 * transpose_out != 0 it is written transposed ([cols, rows]), which is how tall
 * parameters enter the iteration. */
int muon_b200_prologue(void* const* grads, void* const* moms, int count, int64_t rows,
                       int64_t cols, int dtype, double beta, int nesterov, void* x, int64_t ldx,
                       int64_t x_bs, int transpose_out, muon_b200_stream_t stream);

/* muon_b200_prologue that also sums the squares of the bf16 values it writes (the Frobenius norm of
 * the classic iteration, muon.py:282, fused into the pass that produces X): sumsq receives, for
 * tensor i, sumsq_bs floats at sumsq + i * sumsq_bs whose sum is ||X_i||_F^2 (one per tile of the
 * kernel, the rest zero). sumsq = NULL: plain muon_b200_prologue. For a workspace laid out with
 * muon_b200_ns_workspace_layout_mode(..., MUON_B200_NS_CLASSIC5, &l): sumsq = workspace +
 * l.sumsq_offset_bytes, sumsq_bs = l.sumsq_bs, then run with MUON_B200_NS_HAVE_SUMSQ. */
int muon_b200_prologue_sumsq(void* const* grads, void* const* moms, int count, int64_t rows,
                             int64_t cols, int dtype, double beta, int nesterov, void* x, int64_t ldx,
                             int64_t x_bs, int transpose_out, float* sumsq, int64_t sumsq_bs,
                             muon_b200_stream_t stream);

/* Update epilogue, in place on params (muon.py:14 and :66-67):
 * p = p*(1 - lr*wd) - lr * bf16(U*scale). U of tensor i is at u + i*u_bs, pitch ldu, and is
 * [rows, cols], or [cols, rows] when u_transposed != 0. */
int muon_b200_epilogue(void* const* params, int count, int64_t rows, int64_t cols, int dtype,
                       const void* u, int64_t ldu, int64_t u_bs, int u_transposed, double lr,
                       double weight_decay, double scale, muon_b200_stream_t stream);

/* The same update, with every new parameter value also stored into n_peers (0..7) other copies of
 * the parameter: peer_params[r * count + i] is the address, valid on the current device, of
 * parameter i in peer r's memory (from muon_b200_ipc_open, or any peer-accessible allocation of
 * the same layout). The stores are plain global stores issued by the kernel that computes the
 * value, so the exchange of the distributed step rides on the update itself and is complete when
 * the kernel is. Replaces the update and the all_gather that follows it (muon.py:66-68). */
int muon_b200_epilogue_push(void* const* params, void* const* peer_params, int n_peers, int count,
                            int64_t rows, int64_t cols, int dtype, const void* u, int64_t ldu,
                            int64_t u_bs, int u_transposed, double lr, double weight_decay,
                            double scale, muon_b200_stream_t stream);

/* Whole Muon update of `count` same-shape parameters: prologue -> NS -> epilogue, using
 * `workspace` (>= muon_b200_ns_workspace_layout(count, min(rows,cols), max(rows,cols))
 * bytes). scale is the factor of muon.py:14, evaluated by the caller on the original
 * gradient shape. Replaces the body of the per-parameter loop of SingleDeviceMuon.step
 * (muon.py:94-99) for a group of parameters. */
int muon_b200_muon_step(void* const* params, void* const* grads, void* const* moms, int count,
                        int64_t rows, int64_t cols, int dtype, double lr, double weight_decay,
                        double beta, int nesterov, double scale, int ns_mode, int ns_steps,
                        const float* ns_coeffs, float ns_eps, void* workspace,
                        int64_t workspace_bytes, muon_b200_stream_t stream);

/* Fused Adam step on `count` tensors of any sizes (numel[i] elements each), in place on
 * params, exp_avg and exp_avg_sq; steps[i] is the 1-based step count of tensor i after
 * the increment. Replaces adam_update and the two parameter ops that follow it
 * (muon.py:104-109, :193-197). */
int muon_b200_adam(void* const* params, void* const* grads, void* const* exp_avg,
                   void* const* exp_avg_sq, const int64_t* numel, const int64_t* steps, int count,
                   int dtype, double lr, double weight_decay, double beta1, double beta2,
                   double eps, muon_b200_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* MUON_B200_H_ */
