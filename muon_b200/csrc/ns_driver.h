// The Newton-Schulz iteration as a sequence of kernel launches over caller-chosen buffers.
// Shared by muon_b200_ns_run (buffers inside a caller workspace) and muon_b200_ns_run_static
// (buffers inside the library's built-in scratch), so that the coefficient tables and the
// launch order exist once.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "ns_gemm.h"

namespace mb {

constexpr int kFroChunksMax = 296;  // floats per matrix the fp32 area holds at least
// Partial sums per matrix when the driver takes the Frobenius norm over X itself: fewer than
// kFroChunksMax, so that the last 2 * batch floats of the fp32 area stay free for the factors
// 1 / (||X|| + eps) and their squares.
constexpr int kFroChunks = 288;
constexpr int kFp8MinCols = 1024;   // MUON_B200_NS_AOL4_FP8: narrower matrices stay in bf16

struct NsBuffers {
  // The iterate ping-pongs between x[0] (holds the input on entry) and x[1]; both are
  // [batch, m, n] bf16 with their own pitches (elements).
  __nv_bfloat16* x[2];
  int64_t ldx[2], x_bs[2];
  // Square scratch matrices [batch, m, ldm]: the Gram matrix A, its row-scaled copy (AOL mode
  // only; may alias x[1], which is not written before the first line 3) and B.
  __nv_bfloat16* A;
  __nv_bfloat16* A_scaled;
  __nv_bfloat16* B;
  int64_t ldm, a_bs;
  // fp32 scratch, per matrix max(ldm, kFroChunksMax) floats: row scales 1/s or Frobenius partials.
  float* fscratch;
  int64_t f_bs;
  // MUON_B200_NS_AOL4_FP8 only: e4m3 copies X8 = e4m3(X * sx) [batch, m, ld8n] and
  // E8 = e4m3((A - I) * se) [batch, m, ld8m] (pitches in bytes, multiples of 16).
  uint8_t* x8;
  uint8_t* e8;
  int64_t ld8n, x8_bs, ld8m, e8_bs;
  // MUON_B200_NS_CLASSIC5 only: fro_scales (inside fscratch, see fro_scales_in) receives
  // 1 / (||X|| + eps) of every matrix and, batch floats further, its square. tile_sumsq, when not null, holds tile_count partial sums of squares
  // per matrix (matrix b at tile_sumsq + b * tile_bs) that the prologue kernel left while it
  // produced x[0]; without it the driver sums over x[0] itself.
  float* fro_scales;
  const float* tile_sumsq;
  int64_t tile_bs;
  int64_t tile_count;
  // fp32 partial sums of a line 1 that is split along K (launches with few tiles; see SplitK in
  // ns_gemm.h), splitk_bytes of them; null (every caller but the functional zeropower): never split.
  float* splitk;
  int64_t splitk_bytes;
};

// Floats per matrix of the fp32 area, and where the classic iteration keeps its two factors per
// matrix inside it (the last 2 * batch floats).
inline int64_t fscratch_per_matrix(int64_t ldm) { return ldm > kFroChunksMax ? ldm : kFroChunksMax; }
inline float* fro_scales_in(float* fscratch, int batch, int64_t ldm) {
  return fscratch + (int64_t)batch * fscratch_per_matrix(ldm) - 2 * (int64_t)batch;
}
// Bytes a workspace for the classic iteration adds for the prologue kernel's per-tile sums of
// squares: at most one tile per 64 x 64 elements, in either orientation of the parameter.
inline int64_t classic_tiles_max(int64_t m, int64_t n) { return ((m + 63) / 64) * ((n + 63) / 64); }
int64_t ns_classic_extra_bytes(int batch, int64_t m, int64_t n);

// Pitches (bytes) of the e4m3 copies and the bytes they add to a workspace or scratch area.
inline int64_t fp8_pitch(int64_t cols) { return (cols + 15) / 16 * 16; }
int64_t ns_fp8_extra_bytes(int batch, int64_t m, int64_t n);

// steps > 0; coeffs is NULL (the mode's table) or steps triples (a, b, c). On success
// *result_index tells which of x[0] / x[1] holds the result (steps % 2). With `upd` (which must be
// update_fusable) the last line 3 applies its output to the parameters instead of storing it: no
// buffer holds the result then.
int ns_iterate(const NsBuffers& buf, int batch, int64_t m, int64_t n, int mode, int steps,
               const float* coeffs, float eps, cudaStream_t stream, int* result_index,
               const UpdateSpec* upd = nullptr);

// Same launch sequence, replayed from a CUDA graph when that pays: a short iteration (a few
// matrices of a few hundred rows) is thirteen kernels of microseconds each, and issuing them one
// by one costs more host time than they take on the device. The first call for a given set of
// buffers, sizes and coefficients captures the sequence on a stream the library owns (nothing
// runs during capture), instantiates the graph and launches it on `stream`; later calls only
// launch it. Falls back to ns_iterate when the work is large enough to hide its launches, when
// per-kernel timing is on, when `stream` is itself being captured, or when graph replay is
// switched off (set_graph_replay(false) or MUON_B200_GRAPH=0). Graph instantiation allocates
// driver-side resources, so callers that must not allocate use ns_iterate.
int ns_iterate_replayed(const NsBuffers& buf, int batch, int64_t m, int64_t n, int mode, int steps,
                        const float* coeffs, float eps, cudaStream_t stream, int* result_index,
                        const UpdateSpec* upd = nullptr);
void set_graph_replay(bool on);
bool graph_replay_enabled();

// Bytes of scratch ns_run_with_scratch needs for `batch` matrices of m x n (m <= n): one
// [batch, m, ldn] iterate buffer, three [batch, m, ldm] squares, the fp32 area and, with
// `split_k`, room for the partial sums of a Gram product that is split along K. -1 on bad sizes.
int64_t ns_scratch_bytes(int batch, int64_t m, int64_t n, int mode = 0, bool split_k = false);

// Newton-Schulz with caller-owned input and output and a scratch area of ns_scratch_bytes():
// `src` ([batch, rows, cols], element type `dtype` (a DType), pitches in elements) is cast to bf16,
// transposed when rows > cols, into whichever iterate buffer makes the result land in `out`
// ([batch, m, n] bf16, m = min(rows, cols)); the iteration ping-pongs between `out` and the
// scratch. `replay` allows graph replay (see ns_iterate_replayed). `split_k` allows line 1 to be
// split along K when the launch has few tiles (SplitK in ns_gemm.h; the scratch must then have been
// sized with split_k): a matrix's result then depends, in the order of its fp32 additions, on how
// many matrices share the call, which is why only the functional entry point asks for it — the
// optimizer step and the entry points that promise its arithmetic never do.
int ns_run_with_scratch(const void* src, int dtype, int64_t rows, int64_t cols, int64_t ld_src,
                        int64_t src_bs, __nv_bfloat16* out, int64_t ldo, int64_t o_bs,
                        unsigned char* scratch, int batch, int mode, int steps, const float* coeffs,
                        float eps, bool replay, cudaStream_t stream, bool split_k = false);

// Argument checks shared by both entry points: fills in the default step count.
int ns_check_mode(int mode, int* steps, const float* coeffs);

}  // namespace mb
