// Internal interface between the elementwise kernels and the C-ABI layer.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace mb {

// DT_F64 is accepted by the cast kernel only (inputs of the functional Newton-Schulz); parameters,
// gradients and optimizer state are DT_F32, DT_BF16 or DT_F16.
enum DType : int { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2, DT_F64 = 3 };

constexpr int kMaxTensors = 32;  // tensors per multi-tensor launch

struct PrologueArgs {
  void* grad[kMaxTensors];
  void* mom[kMaxTensors];
  __nv_bfloat16* x;   // X of tensor i starts at x + i * x_bs
  long long x_bs;
  long long ldx;      // pitch of X in elements
  int count;
  int rows, cols;     // 2-D view of each parameter
  int nesterov;
  int vec_ok;         // all grad/mom pointers 16-byte aligned and cols % vector == 0
  float w_mom;        // float(1 - beta)
  float beta;         // float(beta)
  float* sumsq;       // or null: per-tile sums of squares of X, tensor i at sumsq + i * sumsq_bs
  long long sumsq_bs;
};

struct EpilogueArgs {
  void* param[kMaxTensors];
  const __nv_bfloat16* u;  // NS output of tensor i at u + i * u_bs
  long long u_bs;
  long long ldu;
  int count;
  int rows, cols;
  int vec_ok;
  float scale;   // max(1, rows/cols)^0.5 as the reference evaluates it
  float decay;   // float(1 - lr*wd)
  float neg_lr;  // float(-lr)
};

// Copies of the same parameters in other GPUs' memory (mapped on this device): the epilogue
// kernel stores every updated element there as well, with plain stores over NVLink.
constexpr int kMaxPeers = 7;
struct EpiloguePeers {
  void* param[kMaxPeers][kMaxTensors];
  int n_peers;
};

struct AdamArgs {
  void* param[kMaxTensors];
  void* grad[kMaxTensors];
  void* exp_avg[kMaxTensors];
  void* exp_avg_sq[kMaxTensors];
  long long numel[kMaxTensors];
  float bc1[kMaxTensors];  // 1 - beta1^step
  float bc2[kMaxTensors];  // 1 - beta2^step
  int block_start[kMaxTensors + 1];
  unsigned char vec_ok[kMaxTensors];
  int count;
  float w1, w2;  // float(1 - beta1), float(1 - beta2)
  float eps;
  float decay;
  float neg_lr;
};

int adam_elems_per_block(int dtype);
int launch_prologue(const PrologueArgs& a, int dtype, int transpose, cudaStream_t stream);
int launch_epilogue(const EpilogueArgs& a, int dtype, int transpose, cudaStream_t stream,
                    const EpiloguePeers* peers = nullptr);
int launch_aol_rescale(__nv_bfloat16* X, long long ldx, long long x_bs, const __nv_bfloat16* A,
                       __nv_bfloat16* A_out, long long lda, long long a_bs, float* svec,
                       long long s_bs, int m, int n, int batch, float eps, cudaStream_t stream);
// Tiles (= partial sums) per tensor of the prologue kernel for parameters of this 2-D view.
int prologue_tiles(int rows, int cols, int dtype);
// scales[b] = 1 / (||X_b||_F + eps) and scales[batch + b] = its square, for the classic iteration.
// With tile_sumsq (per-tile sums the prologue kernel left: tile_count per matrix, matrix b at
// tile_sumsq + b * tile_bs) X is not read; otherwise one pass over X writes `chunks` partial sums
// per matrix into `partials` first.
int launch_fro_scales(const __nv_bfloat16* X, long long ldx, long long x_bs, int m, int n, int batch,
                      float eps, float* partials, int chunks, const float* tile_sumsq, long long tile_bs,
                      int tile_count, float* scales, cudaStream_t stream);
int launch_adam(const AdamArgs& a, int dtype, cudaStream_t stream);
// dst[b][r][c] (or dst[b][c][r] when transpose) = bf16(float(src[b][r][c]) * scale); src has
// element type `dtype`, pitches in elements. src and dst may be the same buffer when the types
// and pitches agree and transpose == 0.
int launch_cast_bf16(const void* src, int dtype, long long ld_src, long long src_bs, __nv_bfloat16* dst,
                     long long ld_dst, long long dst_bs, int rows, int cols, int batch, int transpose,
                     float scale, cudaStream_t stream);

}  // namespace mb
