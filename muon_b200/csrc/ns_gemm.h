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
};

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
                   int64_t scale_bs = 0);

}  // namespace mb
