// Internal interface between the NS GEMM kernels and the C-ABI layer.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace mb {

enum GemmMode : int {
  MODE_SYRK = 0,   // out = opA · opAᵀ                       (lower tiles + mirror)
  MODE_AXPBY = 1,  // out = alpha · opA · opAᵀ + beta · opA   (lower tiles + mirror)
  MODE_BX = 2,     // out = opA · opB + alpha · opB           (full)
};

// How line 2 obtains the addend beta * A for the mirrored (upper-triangle) element.
enum AddendMode : int {
  ADD_GENERIC = 0,     // A arbitrary: the mirrored element reads A[col, row] from memory
  ADD_SYMMETRIC = 1,   // A == A^T bit for bit: the finished value is mirrored
  ADD_ROW_SCALED = 2,  // A = S / s with S symmetric: both addends are rebuilt from S and s
};

// Kernel variants beyond mode and addend: 8-bit floating point (e4m3) in the two symmetric
// products (see Fp8Spec), and the parameter update fused into the last line 3 (see UpdateSpec).
enum Variant : int {
  F8_NONE = 0,
  F8_OPERANDS = 1,   // the product's operands are e4m3 (lines 1 and 2)
  F8_EXTRA_OUT = 2,  // bf16 product that also writes an e4m3 copy of its output (line 3)
  V_UPD_BF16 = 3,    // line 3 applies its output to bf16 parameters of the tile's orientation
  V_UPD_BF16_T = 4,  // ... to bf16 parameters stored as the transpose of the tile (tall parameters)
  V_UPD_F32 = 5,     // ... to fp32 parameters of the tile's orientation
  V_BATCH_SCALE = 6, // lines 1 and 3: the output of matrix b is multiplied by batch_scale[b] (a
                     // scalar in device memory) before it is rounded: the Frobenius normalisation
                     // of the classic iteration folded into its first two products
};

constexpr int kMaxUpdateTensors = 64;  // parameters one fused-update launch can address

// The update epilogue (reference muon.py:14 and :66-67) done by the last line 3 itself:
//   p = T(T(p * decay) + neg_lr * bf16(U * scale))
// param[b] is the parameter of matrix b of the batch, contiguous [rows, cols]; the iteration ran
// on its transpose when rows > cols.
struct UpdateSpec {
  void* const* param = nullptr;
  int dtype = 0;  // a DType
  int64_t rows = 0, cols = 0;
  float scale = 1.f, decay = 1.f, neg_lr = 0.f;
};
// Whether launch_ns_gemm can fuse this update (fp32 tall parameters, batches beyond
// kMaxUpdateTensors and rows that are not 16-byte multiples are left to the epilogue kernel).
bool update_fusable(const UpdateSpec& u, int batch);

// The e4m3 variant of the iteration keeps, beside the bf16 matrices, X8 = e4m3(X * sx) and
// E8 = e4m3((A - I) * se), both with power-of-two scales:
//   line 1 (F8_OPERANDS): A = (X8 · X8ᵀ) * acc_scale, acc_scale = 1 / sx²; writes A in bf16 and E8.
//   line 2 (F8_OPERANDS): with E = A - I, alpha·A·A + beta·A = alpha·E·E + (beta + 2·alpha)·A - alpha·I,
//                         so only the small matrix E goes through e4m3: out = (E8 · E8ᵀ) * alpha'
//                         + beta' * A + diag * I with alpha' = alpha / se², beta' = beta + 2·alpha,
//                         diag = -alpha (the caller passes alpha', beta', diag).
//   line 3 (F8_EXTRA_OUT): bf16 as always, and writes X8 for the next line 1.
struct Fp8Spec {
  int kind = F8_NONE;
  const uint8_t* op8 = nullptr;  // F8_OPERANDS: the e4m3 operand [batch, M, K], pitch ld8 bytes
  int64_t ld8 = 0, bs8 = 0;
  uint8_t* out8 = nullptr;       // e4m3 copy of the output (line 1: E8, line 3: X8), or null
  int64_t ldo8 = 0, out8_bs = 0;
  float out8_scale = 1.f;        // se or sx
  float acc_scale = 1.f;         // line 1: 1 / sx²
  float diag = 0.f;              // line 2: added to the diagonal of the output
};

struct GemmParams {
  int M, N, K;  // output rows, output cols, contraction length
  int batch;
  int tiles_m, tiles_n;
  int tiles_per_batch;
  int triangular;
  int sym_add;  // line 2: an AddendMode
  const float* row_scale;  // ADD_ROW_SCALED: s, one float per matrix row
  long long scale_bs;      // batch pitch of row_scale in floats
  float alpha, beta;
  __nv_bfloat16* out;
  long long ldo, out_bs;
  const __nv_bfloat16* add;
  long long ldadd, add_bs;
  // e4m3 variants (see Fp8Spec)
  uint8_t* out8;
  long long ldo8, out8_bs;
  float out8_scale, acc_scale, diag;
  // fused parameter update (see UpdateSpec)
  void* upd_param[kMaxUpdateTensors];
  float upd_scale, upd_decay, upd_neg_lr;
  // V_BATCH_SCALE: one factor per matrix of the batch
  const float* batch_scale;
  // Split-K of line 1 (see SplitK): 0 = none; 1 = every work item is one of split_k K-slices
  // (split_kb k-blocks each) of a tile and leaves fp32 partial sums in `partial`.
  int split_phase, split_k, split_kb;
  float* partial;
};

// Scratch for split-K: a launch of line 1 whose tiles would occupy less than a third of the SMs
// (one or a few small matrices with a long K) is cut along K into slices that run on different
// SMs; a second, small kernel adds the slices of every 32 x 32 block in slice order (so the
// result does not depend on scheduling) and stores the block and its mirror image.
struct SplitK {
  float* partial = nullptr;  // 256-byte aligned
  int64_t bytes = 0;
};
// Slices launch_ns_gemm would use for line 1 of `batch` m x m products with contraction length k
// (1 = no split), and the scratch bytes that takes; both functions of the sizes only (sized for
// the 148 SMs of a B200, so that layouts can be computed without a device).
int splitk_slices(int batch, int64_t m, int64_t k);
int64_t splitk_scratch_bytes(int batch, int64_t m, int64_t k);

int device_sm_count(int* sm_count_out);
// Whether kernels that support it are launched with programmatic stream serialization.
bool dependent_launch_enabled();
void set_reserved_sms(int n);
int get_reserved_sms();

int launch_ns_gemm(int mode, const __nv_bfloat16* opa, int64_t lda, int64_t a_bs,
                   const __nv_bfloat16* opb, int64_t ldb, int64_t b_bs, __nv_bfloat16* out,
                   int64_t ldo, int64_t out_bs, int batch, int64_t M, int64_t N, int64_t K,
                   float alpha, float beta, int sym_add, cudaStream_t stream,
                   const __nv_bfloat16* addend = nullptr, const float* row_scale = nullptr,
                   int64_t scale_bs = 0, const Fp8Spec* f8 = nullptr, const UpdateSpec* upd = nullptr,
                   const float* batch_scale = nullptr, const SplitK* split = nullptr);

}  // namespace mb
