// HBM-bound kernels of the Muon step: momentum prologue, AOL / Frobenius rescale,
// update epilogue and the fused Adam step. All of them move 128 bits per thread per
// access where alignment allows, are grid-stride over tiles, and take up to
// kMaxTensors same-shape tensors per launch so that a group of parameters costs one
// launch instead of one per parameter.
#include "common.cuh"
#include "elementwise.h"

#include <cuda_fp16.h>
#include "ns_gemm.h"
#include "profiling.h"

namespace mb {

namespace {

constexpr int kThreads = 256;
constexpr int kTileRows = 64;
constexpr int kRowsInFlight = 2;  // rows of a tile whose loads a thread issues back to back

template <typename T>
constexpr bool kIsBf16 = false;
template <>
constexpr bool kIsBf16<__nv_bfloat16> = true;

template <typename T>
struct Vec;
template <>
struct Vec<float> {
  static constexpr int N = 4;
  using Raw = float4;
  // (streaming loads and stores: the data is touched once and must not push the operands of GEMMs
  // that run beside these kernels out of L2)
  __device__ static Raw load_raw(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
  __device__ static void store_stream(float* p, const float (&v)[4]) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
  }
  __device__ static void unpack(const Raw& r, float (&v)[4]) {
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  }
  __device__ static void load(const float* p, float (&v)[4]) {
    float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  }
  __device__ static void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  using Raw = uint4;
  __device__ static Raw load_raw(const __nv_bfloat16* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
  __device__ static void store_stream(__nv_bfloat16* p, const float (&v)[8]) {
    __stcs(reinterpret_cast<uint4*>(p), make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                                   pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7])));
  }
  __device__ static void unpack(const Raw& r, float (&v)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = bf16_bits_to_float(w[j] & 0xffffu);
      v[2 * j + 1] = bf16_bits_to_float(w[j] >> 16);
    }
  }
  __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 r = *reinterpret_cast<const uint4*>(p);
    uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = bf16_bits_to_float(w[j] & 0xffffu);
      v[2 * j + 1] = bf16_bits_to_float(w[j] >> 16);
    }
  }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[8]) {
    *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                              pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
  }
};

template <>
struct Vec<__half> {
  static constexpr int N = 8;
  using Raw = uint4;
  __device__ static Raw load_raw(const __half* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
  __device__ static void unpack(const Raw& r, float (&v)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
    }
  }
  __device__ static void load(const __half* p, float (&v)[8]) {
    unpack(*reinterpret_cast<const uint4*>(p), v);
  }
  __device__ static uint4 pack(const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
      w[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ static void store(__half* p, const float (&v)[8]) { *reinterpret_cast<uint4*>(p) = pack(v); }
  __device__ static void store_stream(__half* p, const float (&v)[8]) { __stcs(reinterpret_cast<uint4*>(p), pack(v)); }
};

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// Round an fp32 intermediate to the storage type and back, i.e. what an eager
// elementwise op leaves in a tensor of type T.
template <typename T>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<float>(float v) { return v; }
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
template <>
__device__ __forceinline__ float round_to<__half>(float v) { return __half2float(__float2half_rn(v)); }
// Same for two values at once: for bf16 one packed conversion instead of two scalar ones.
template <typename T>
__device__ __forceinline__ void round_pair_to(float& a, float& b);
template <>
__device__ __forceinline__ void round_pair_to<float>(float&, float&) {}
template <>
__device__ __forceinline__ void round_pair_to<__nv_bfloat16>(float& a, float& b) {
  const uint32_t w = pack_bf16x2(a, b);
  a = bf16_bits_to_float(w & 0xffffu);
  b = bf16_bits_to_float(w >> 16);
}
template <>
__device__ __forceinline__ void round_pair_to<__half>(float& a, float& b) {
  const float2 f = __half22float2(__floats2half2_rn(a, b));
  a = f.x;
  b = f.y;
}
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// torch.lerp(self, end, weight) in opmath precision: two algebraically equal forms,
// picked by |weight| < 0.5 (ATen/native/Lerp.h).
__device__ __forceinline__ float torch_lerp(float self, float end, float w) {
  const float d = end - self;
  return (fabsf(w) < 0.5f) ? fmaf(w, d, self) : fmaf(-d, 1.0f - w, end);
}

// ---------------------------------------------------------------------------
// Prologue (reference muon_update, muon.py:9-12 and the cast/transposition of
// zeropower_via_newtonschulz5, muon.py:760-764):
//   mom  <- lerp(mom, grad, 1 - beta)
//   grad <- lerp(grad, mom, beta)            (Nesterov; written back like lerp_ does)
//   X    <- bf16(nesterov ? grad : mom), stored [rows, cols] or transposed [cols, rows]
// A tile is kTileRows x (16 * Vec<T>::N) elements.
// With a.sumsq the kernel also leaves, per tile, the sum of the squares of the bf16 values it
// stored (the Frobenius norm of the classic iteration, muon.py:282, taken while X is produced):
// one float per (tensor, tile), added later in index order, so the norm does not depend on which
// CTA handled which tile.
// ---------------------------------------------------------------------------
template <typename T, bool TRANSPOSE>
__global__ void __launch_bounds__(kThreads)
prologue_kernel(const PrologueArgs a) {
  constexpr int V = Vec<T>::N;
  constexpr int kTileCols = 16 * V;
  // Transposition staging: [col][row] with one pad column of 2 bf16 to skew banks.
  __shared__ __nv_bfloat16 tile[TRANSPOSE ? kTileCols : 1][TRANSPOSE ? kTileRows + 2 : 1];
  __shared__ float warp_ss[2][kThreads / 32];  // two sets taking turns: one barrier per tile

  const int tiles_c = (a.cols + kTileCols - 1) / kTileCols;
  const int tiles_r = (a.rows + kTileRows - 1) / kTileRows;
  const long long tiles_per = (long long)tiles_c * tiles_r;
  const long long total = tiles_per * a.count;
  const int tx = threadIdx.x & 15;
  const int ty = threadIdx.x >> 4;
  int turn = 0;
  griddep_launch_dependents();  // line 1 may set itself up while this kernel drains
  const float w1 = a.w_mom;  // float(1 - beta)
  const float w2 = a.beta;   // float(beta)

  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    const int ti = (int)(t / tiles_per);
    const long long rem = t - (long long)ti * tiles_per;
    const int tr = (int)(rem / tiles_c);
    const int tcn = (int)(rem - (long long)tr * tiles_c);
    T* g = static_cast<T*>(a.grad[ti]);
    T* m = static_cast<T*>(a.mom[ti]);
    __nv_bfloat16* x = a.x + (long long)ti * a.x_bs;
    const int c0 = tcn * kTileCols + tx * V;
    float ss = 0.f;  // this thread's share of the tile's sum of squares

    const bool full = a.vec_ok && (c0 + V <= a.cols);
#pragma unroll
    for (int it0 = 0; it0 < kTileRows / 16; it0 += kRowsInFlight) {
     // The 128-bit loads of kRowsInFlight rows are issued together and kept as raw words, so
     // each thread has 2 * kRowsInFlight requests in flight at little register cost.
     typename Vec<T>::Raw rg[kRowsInFlight], rm[kRowsInFlight];
#pragma unroll
     for (int u = 0; u < kRowsInFlight; ++u) {
       const int r = tr * kTileRows + (it0 + u) * 16 + ty;
       if (full && r < a.rows) {
         const long long off = (long long)r * a.cols + c0;
         rg[u] = Vec<T>::load_raw(g + off);
         rm[u] = Vec<T>::load_raw(m + off);
       }
     }
#pragma unroll
     for (int u = 0; u < kRowsInFlight; ++u) {
      const int it = it0 + u;
      const int rl = it * 16 + ty;
      const int r = tr * kTileRows + rl;
      float xv[V];
#pragma unroll
      for (int j = 0; j < V; ++j) xv[j] = 0.f;
      if (r < a.rows && c0 < a.cols) {
        const long long off = (long long)r * a.cols + c0;
        float gv[V], mv[V];
        if (full) {
          Vec<T>::unpack(rg[u], gv);
          Vec<T>::unpack(rm[u], mv);
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) {
            const bool in = c0 + j < a.cols;
            gv[j] = in ? to_f<T>(g[off + j]) : 0.f;
            mv[j] = in ? to_f<T>(m[off + j]) : 0.f;
          }
        }
        // Two elements at a time: rounding to bf16 is one packed conversion per pair.
#pragma unroll
        for (int j = 0; j < V; j += 2) {
          mv[j] = torch_lerp(mv[j], gv[j], w1);
          mv[j + 1] = torch_lerp(mv[j + 1], gv[j + 1], w1);
          round_pair_to<T>(mv[j], mv[j + 1]);
          if (a.nesterov) {
            gv[j] = torch_lerp(gv[j], mv[j], w2);
            gv[j + 1] = torch_lerp(gv[j + 1], mv[j + 1], w2);
            round_pair_to<T>(gv[j], gv[j + 1]);
            xv[j] = gv[j];
            xv[j + 1] = gv[j + 1];
          } else {
            xv[j] = mv[j];
            xv[j + 1] = mv[j + 1];
          }
          if (!kIsBf16<T>) round_pair_to<__nv_bfloat16>(xv[j], xv[j + 1]);  // fp32 / fp16 state -> bf16 X
          ss = fmaf(xv[j], xv[j], ss);  // elements outside the matrix are zero
          ss = fmaf(xv[j + 1], xv[j + 1], ss);
        }
        if (full) {
          Vec<T>::store_stream(m + off, mv);
          if (a.nesterov) Vec<T>::store_stream(g + off, gv);
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j)
            if (c0 + j < a.cols) {
              m[off + j] = from_f<T>(mv[j]);
              if (a.nesterov) g[off + j] = from_f<T>(gv[j]);
            }
        }
        if (!TRANSPOSE) {
          __nv_bfloat16* xr = x + (long long)r * a.ldx + c0;
          if (c0 + V <= a.cols) {
            if (V == 8) {
              *reinterpret_cast<uint4*>(xr) =
                  make_uint4(pack_bf16x2(xv[0], xv[1]), pack_bf16x2(xv[2], xv[3]),
                             pack_bf16x2(xv[V - 4], xv[V - 3]), pack_bf16x2(xv[V - 2], xv[V - 1]));
            } else {
              *reinterpret_cast<uint2*>(xr) =
                  make_uint2(pack_bf16x2(xv[0], xv[1]), pack_bf16x2(xv[2], xv[3]));
            }
          } else {
#pragma unroll
            for (int j = 0; j < V; ++j)
              if (c0 + j < a.cols) xr[j] = __float2bfloat16_rn(xv[j]);
          }
        }
      }
      if (TRANSPOSE) {
#pragma unroll
        for (int j = 0; j < V; ++j) tile[tx * V + j][rl] = __float2bfloat16_rn(xv[j]);
      }
     }
    }
    if (TRANSPOSE) {
      __syncthreads();
      // Output rows are input columns. 8 threads cover one output row of 64 elements.
      const int seg = threadIdx.x & 7;
      for (int cl = threadIdx.x >> 3; cl < kTileCols; cl += kThreads / 8) {
        const int c = tcn * kTileCols + cl;
        const int r0 = tr * kTileRows + seg * 8;
        if (c < a.cols && r0 < a.rows) {
          __nv_bfloat16* xr = x + (long long)c * a.ldx + r0;
          if (r0 + 8 <= a.rows) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              w[j] = *reinterpret_cast<const uint32_t*>(&tile[cl][seg * 8 + 2 * j]);
            *reinterpret_cast<uint4*>(xr) = make_uint4(w[0], w[1], w[2], w[3]);
          } else {
            for (int j = 0; j < 8 && r0 + j < a.rows; ++j) xr[j] = tile[cl][seg * 8 + j];
          }
        }
      }
      __syncthreads();
    }
    if (a.sumsq) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((threadIdx.x & 31) == 0) warp_ss[turn][threadIdx.x >> 5] = ss;
      __syncthreads();
      if (threadIdx.x == 0) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) s += warp_ss[turn][w];
        a.sumsq[(long long)ti * a.sumsq_bs + rem] = s;
      }
      turn ^= 1;
    }
  }
}

// ---------------------------------------------------------------------------
// Epilogue (reference muon.py:14 and :66-67): with U the bf16 NS output
//   U' = bf16(U * scale)            (update *= max(1, rows/cols)**0.5)
//   p  = T(p * (1 - lr*wd))         (p.mul_)
//   p  = T(p - lr * U')             (p.add_(update, alpha=-lr))
// U is [rows, cols] or, for tall parameters, stored transposed as [cols, rows].
// With PUSH the new value also goes to the same element of every peer copy (the exchange of
// the distributed step, reference dist.all_gather at muon.py:68, done by the producing kernel).
// ---------------------------------------------------------------------------
template <typename T, bool TRANSPOSE, bool PUSH>
__global__ void __launch_bounds__(kThreads)
epilogue_kernel(const EpilogueArgs a, const EpiloguePeers peers) {
  constexpr int V = Vec<T>::N;
  constexpr int kTileCols = 16 * V;
  __shared__ __nv_bfloat16 tile[TRANSPOSE ? kTileCols : 1][TRANSPOSE ? kTileRows + 2 : 1];

  const int tiles_c = (a.cols + kTileCols - 1) / kTileCols;
  const int tiles_r = (a.rows + kTileRows - 1) / kTileRows;
  const long long tiles_per = (long long)tiles_c * tiles_r;
  const long long total = tiles_per * a.count;
  const int tx = threadIdx.x & 15;
  const int ty = threadIdx.x >> 4;

  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    const int ti = (int)(t / tiles_per);
    const long long rem = t - (long long)ti * tiles_per;
    const int tr = (int)(rem / tiles_c);
    const int tcn = (int)(rem - (long long)tr * tiles_c);
    T* p = static_cast<T*>(a.param[ti]);
    const __nv_bfloat16* u = a.u + (long long)ti * a.u_bs;

    if (TRANSPOSE) {
      // Stage U[c, r0..r0+63] rows into tile[c][r].
      const int seg = threadIdx.x & 7;
      for (int cl = threadIdx.x >> 3; cl < kTileCols; cl += kThreads / 8) {
        const int c = tcn * kTileCols + cl;
        const int r0 = tr * kTileRows + seg * 8;
        if (c < a.cols && r0 < a.rows) {
          const __nv_bfloat16* ur = u + (long long)c * a.ldu + r0;
          if (r0 + 8 <= a.rows) {
            uint4 q = *reinterpret_cast<const uint4*>(ur);
            uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint32_t*>(&tile[cl][seg * 8 + 2 * j]) = w[j];
          } else {
            for (int j = 0; j < 8 && r0 + j < a.rows; ++j) tile[cl][seg * 8 + j] = ur[j];
          }
        }
      }
      __syncthreads();
    }

    const int c0 = tcn * kTileCols + tx * V;
    const bool full = a.vec_ok && (c0 + V <= a.cols);
    // One row per pass here: batching the loads of two rows, which helps the prologue, made
    // this kernel a third slower (fewer resident warps, nothing gained on its two streams).
#pragma unroll
    for (int it = 0; it < kTileRows / 16; ++it) {
     {
      const int rl = it * 16 + ty;
      const int r = tr * kTileRows + rl;
      if (r < a.rows && c0 < a.cols) {
        const long long off = (long long)r * a.cols + c0;
        float pv[V], uv[V];
        if (full) {
          Vec<T>::load(p + off, pv);
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) pv[j] = (c0 + j < a.cols) ? to_f<T>(p[off + j]) : 0.f;
        }
        if (TRANSPOSE) {
#pragma unroll
          for (int j = 0; j < V; ++j) uv[j] = __bfloat162float(tile[tx * V + j][rl]);
        } else {
          const __nv_bfloat16* ur = u + (long long)r * a.ldu + c0;
          if (c0 + V <= a.cols) {
            if (V == 8) {
              float tmp[8];
              Vec<__nv_bfloat16>::load(ur, tmp);
#pragma unroll
              for (int j = 0; j < V; ++j) uv[j] = tmp[j];
            } else {
              uint2 q = *reinterpret_cast<const uint2*>(ur);
              uv[0] = bf16_bits_to_float(q.x & 0xffffu);
              uv[1] = bf16_bits_to_float(q.x >> 16);
              uv[2] = bf16_bits_to_float(q.y & 0xffffu);
              uv[3] = bf16_bits_to_float(q.y >> 16);
            }
          } else {
#pragma unroll
            for (int j = 0; j < V; ++j) uv[j] = (c0 + j < a.cols) ? __bfloat162float(ur[j]) : 0.f;
          }
        }
#pragma unroll
        for (int j = 0; j < V; j += 2) {
          float u0 = uv[j] * a.scale, u1 = uv[j + 1] * a.scale;
          round_pair_to<__nv_bfloat16>(u0, u1);
          float p0 = pv[j] * a.decay, p1 = pv[j + 1] * a.decay;
          round_pair_to<T>(p0, p1);
          pv[j] = fmaf(a.neg_lr, u0, p0);
          pv[j + 1] = fmaf(a.neg_lr, u1, p1);
          round_pair_to<T>(pv[j], pv[j + 1]);
        }
        if (full) {
          Vec<T>::store(p + off, pv);
          if (PUSH) {
            for (int r = 0; r < peers.n_peers; ++r) Vec<T>::store(static_cast<T*>(peers.param[r][ti]) + off, pv);
          }
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j)
            if (c0 + j < a.cols) {
              p[off + j] = from_f<T>(pv[j]);
              if (PUSH) {
                for (int r = 0; r < peers.n_peers; ++r)
                  static_cast<T*>(peers.param[r][ti])[off + j] = from_f<T>(pv[j]);
              }
            }
        }
      }
     }
    }
    if (TRANSPOSE) __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// AOL rescale (reference muon.py:779-785), one CTA per matrix row i, with the rounding points of
// the reference's compiled graph (one reduction kernel that also divides, one pointwise kernel
// that reads the stored sums):
//   s_i  = sum_j |A_ij|                         (fp32)
//   A_i: = bf16( A_i: * (1 / max(s_i, eps)) )   (rows only, exactly as the reference does; the
//                                                quotient uses the unrounded fp32 sum and is formed
//                                                with the correctly rounded reciprocal, so that
//                                                other kernels can rebuild it bit for bit)
//   X_i: = bf16( X_i: * rsqrt(max(bf16(s_i), eps)) )   (the sums are materialised in bf16)
// The scaled A goes to A_out (same pitches; may be A itself) so that the symmetric,
// unscaled A stays available; 1/max(s_i, eps) goes to svec (one float per row) when given.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
aol_rescale_kernel(__nv_bfloat16* X, long long ldx, long long x_bs, const __nv_bfloat16* A,
                   __nv_bfloat16* A_out, long long lda, long long a_bs, float* svec, long long s_bs,
                   int m, int n, int batch, float eps) {
  __shared__ float warp_sums[kThreads / 32];
  __shared__ float s_bcast;
  // Launched as a programmatic dependent of line 1 and followed by line 2 (see common.cuh).
  griddep_launch_dependents();
  griddep_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long rows_total = (long long)m * batch;
  for (long long row = blockIdx.x; row < rows_total; row += gridDim.x) {
    const int b = (int)(row / m);
    const int i = (int)(row - (long long)b * m);
    const __nv_bfloat16* arow = A + (long long)b * a_bs + (long long)i * lda;
    __nv_bfloat16* orow = A_out + (long long)b * a_bs + (long long)i * lda;
    __nv_bfloat16* xrow = X + (long long)b * x_bs + (long long)i * ldx;
    float acc = 0.f;
    const int mv = m & ~7;
    for (int j = threadIdx.x * 8; j < mv; j += kThreads * 8) {
      float v[8];
      Vec<__nv_bfloat16>::load(arow + j, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc += fabsf(v[k]);
    }
    for (int j = mv + threadIdx.x; j < m; j += kThreads) acc += fabsf(__bfloat162float(arow[j]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) warp_sums[warp] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int w = 0; w < kThreads / 32; ++w) s += warp_sums[w];
      s_bcast = s;
      if (svec) svec[(long long)b * s_bs + i] = __frcp_rn(fmaxf(s, eps));
    }
    __syncthreads();
    const float s = s_bcast;
    const float rs = rsqrtf(fmaxf(bf16_round(s), eps));
    const float w = __frcp_rn(fmaxf(s, eps));  // A / s is evaluated as A * (1/s), one rounding each
    for (int j = threadIdx.x * 8; j < mv; j += kThreads * 8) {
      float v[8];
      Vec<__nv_bfloat16>::load(arow + j, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] *= w;
      Vec<__nv_bfloat16>::store(orow + j, v);
    }
    for (int j = mv + threadIdx.x; j < m; j += kThreads)
      orow[j] = __float2bfloat16_rn(__bfloat162float(arow[j]) * w);
    const int nv = n & ~7;
    for (int j = threadIdx.x * 8; j < nv; j += kThreads * 8) {
      float v[8];
      Vec<__nv_bfloat16>::load(xrow + j, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] *= rs;
      Vec<__nv_bfloat16>::store(xrow + j, v);
    }
    for (int j = nv + threadIdx.x; j < n; j += kThreads)
      xrow[j] = __float2bfloat16_rn(__bfloat162float(xrow[j]) * rs);
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// Frobenius normalisation of the classic iteration (commented block, muon.py:282):
//   X = X / (||X||_F + 1e-7), bf16 eager semantics for the denominator: the norm and the sum are
//   each rounded to bf16.
// X itself is not rewritten: the factor 1 / (||X|| + eps) of every matrix goes to device memory
// and the first Gram product and the first line 3 multiply their outputs by its square and by it
// (V_BATCH_SCALE in the GEMM kernel). The sum of squares comes as partial sums, one per tile from
// the prologue kernel or one per chunk of rows from sumsq_partial_kernel, and fro_finish_kernel
// adds them in a fixed order, so the result does not depend on scheduling.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
sumsq_partial_kernel(const __nv_bfloat16* X, long long ldx, long long x_bs, int m, int n, int chunks,
                     float* partials) {
  __shared__ float warp_sums[kThreads / 32];
  const int b = blockIdx.y, ch = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float acc = 0.f;
  for (int i = ch; i < m; i += chunks) {
    const __nv_bfloat16* xrow = X + (long long)b * x_bs + (long long)i * ldx;
    const int nv = n & ~7;
    for (int j = threadIdx.x * 8; j < nv; j += kThreads * 8) {
      float v[8];
      Vec<__nv_bfloat16>::load(xrow + j, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc = fmaf(v[k], v[k], acc);
    }
    for (int j = nv + threadIdx.x; j < n; j += kThreads) {
      float v = __bfloat162float(xrow[j]);
      acc = fmaf(v, v, acc);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) warp_sums[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < kThreads / 32; ++w) s += warp_sums[w];
    partials[(long long)b * chunks + ch] = s;
  }
}

// One block per matrix: partials[b * stride + i], i < count  ->  scales[b] = 1 / (||X_b|| + eps),
// scales[batch + b] = its square. Thread t adds the partials t, t + 256, ... in that order, then the
// 256 sums are added pairwise in a fixed tree.
__global__ void __launch_bounds__(kThreads)
fro_finish_kernel(const float* partials, long long stride, int count, float eps, float* scales, int batch) {
  __shared__ float tree[kThreads];
  const int b = blockIdx.x;
  float acc = 0.f;
  for (int i = threadIdx.x; i < count; i += kThreads) acc += partials[(long long)b * stride + i];
  tree[threadIdx.x] = acc;
  __syncthreads();
  for (int half = kThreads / 2; half > 0; half >>= 1) {
    if (threadIdx.x < half) tree[threadIdx.x] += tree[threadIdx.x + half];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float den = bf16_round(bf16_round(sqrtf(tree[0])) + eps);
    const float c = __frcp_rn(den);
    scales[b] = c;
    scales[batch + b] = c * c;
  }
}

// ---------------------------------------------------------------------------
// Fused Adam step (reference adam_update + the two in-place parameter ops,
// muon.py:104-109 and :196-197), every intermediate rounded to the tensor dtype as
// the eager ops do:
//   m  = lerp(m, g, 1-b1) ; v = lerp(v, g*g, 1-b2)
//   u  = (m / bc1) / (sqrt(v / bc2) + eps)
//   p  = p * (1 - lr*wd) ; p = p - lr * u
// Blocks are assigned to tensors through block_start (prefix sums of per-tensor
// block counts), so tensors of different sizes share a launch.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
adam_kernel(const AdamArgs a) {
  constexpr int V = Vec<T>::N;
  constexpr int kPerBlock = kThreads * V * 4;
  int ti = 0;
  while (ti + 1 < a.count && (int)blockIdx.x >= a.block_start[ti + 1]) ++ti;
  const long long base = (long long)((int)blockIdx.x - a.block_start[ti]) * kPerBlock;
  T* p = static_cast<T*>(a.param[ti]);
  const T* g = static_cast<const T*>(a.grad[ti]);
  T* m = static_cast<T*>(a.exp_avg[ti]);
  T* v = static_cast<T*>(a.exp_avg_sq[ti]);
  const long long numel = a.numel[ti];
  const float bc1 = a.bc1[ti], bc2 = a.bc2[ti];
  const bool vec_ok = a.vec_ok[ti] != 0;

#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const long long off = base + ((long long)it * kThreads + threadIdx.x) * V;
    if (off >= numel) break;
    const bool full = vec_ok && (off + V <= numel);
    float pv[V], gv[V], mv[V], vv[V];
    if (full) {
      Vec<T>::load(p + off, pv);
      Vec<T>::load(g + off, gv);
      Vec<T>::load(m + off, mv);
      Vec<T>::load(v + off, vv);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const bool in = off + j < numel;
        pv[j] = in ? to_f<T>(p[off + j]) : 0.f;
        gv[j] = in ? to_f<T>(g[off + j]) : 0.f;
        mv[j] = in ? to_f<T>(m[off + j]) : 0.f;
        vv[j] = in ? to_f<T>(v[off + j]) : 1.f;
      }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
      mv[j] = round_to<T>(torch_lerp(mv[j], gv[j], a.w1));
      const float g2 = round_to<T>(gv[j] * gv[j]);
      vv[j] = round_to<T>(torch_lerp(vv[j], g2, a.w2));
      const float mh = round_to<T>(__fdiv_rn(mv[j], bc1));
      const float vh = round_to<T>(__fdiv_rn(vv[j], bc2));
      const float den = round_to<T>(round_to<T>(__fsqrt_rn(vh)) + a.eps);
      const float u = round_to<T>(__fdiv_rn(mh, den));
      const float p1 = round_to<T>(pv[j] * a.decay);
      pv[j] = round_to<T>(fmaf(a.neg_lr, u, p1));
    }
    if (full) {
      Vec<T>::store(p + off, pv);
      Vec<T>::store(m + off, mv);
      Vec<T>::store(v + off, vv);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j)
        if (off + j < numel) {
          p[off + j] = from_f<T>(pv[j]);
          m[off + j] = from_f<T>(mv[j]);
          v[off + j] = from_f<T>(vv[j]);
        }
    }
  }
}

// ---------------------------------------------------------------------------
// Cast (+ transposition, + scale) into bf16: the entry of zeropower_via_newtonschulz5
// (X = G.to(bfloat16), X.mT for tall inputs, .contiguous(); muon.py:760-764) and the aspect
// scale of muon_update (muon.py:14). 32 x 32 tiles through shared memory when transposing.
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p) { return __half2float(*p); }
template <>
__device__ __forceinline__ float load_as_float<double>(const double* p) {
  // double -> bf16 in one rounding would need a 64-bit path; going through float first rounds
  // twice, which differs from the direct conversion only on exact ties of the float rounding.
  return static_cast<float>(*p);
}

template <typename T, bool TRANSPOSE>
__global__ void __launch_bounds__(kThreads)
cast_bf16_kernel(const T* src, long long ld_src, long long src_bs, __nv_bfloat16* dst, long long ld_dst,
                 long long dst_bs, int rows, int cols, int batch, float scale) {
  __shared__ __nv_bfloat16 tile[TRANSPOSE ? 32 : 1][TRANSPOSE ? 34 : 1];
  const int tiles_c = (cols + 31) / 32, tiles_r = (rows + 31) / 32;
  const long long per = (long long)tiles_c * tiles_r, total = per * batch;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8 threads
  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    const int b = (int)(t / per);
    const long long rem = t - (long long)b * per;
    const int tr = (int)(rem / tiles_c), tcn = (int)(rem - (long long)tr * tiles_c);
    const T* s = src + (long long)b * src_bs;
    __nv_bfloat16* d = dst + (long long)b * dst_bs;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int r = tr * 32 + ty + 8 * k, c = tcn * 32 + tx;
      if (r < rows && c < cols) {
        const __nv_bfloat16 v = __float2bfloat16_rn(load_as_float<T>(s + (long long)r * ld_src + c) * scale);
        if (TRANSPOSE) tile[tx][ty + 8 * k] = v;
        else d[(long long)r * ld_dst + c] = v;
      }
    }
    if (TRANSPOSE) {
      __syncthreads();
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = tcn * 32 + ty + 8 * k, r = tr * 32 + tx;  // output row c, output column r
        if (r < rows && c < cols) d[(long long)c * ld_dst + r] = tile[ty + 8 * k][tx];
      }
      __syncthreads();
    }
  }
}

int grid_for(long long work_items, int per_sm) {
  int sms = 0;
  if (device_sm_count(&sms) != OK) return -1;
  long long cap = (long long)sms * per_sm;
  long long g = work_items < cap ? work_items : cap;
  return (int)(g < 1 ? 1 : g);
}

}  // namespace

int adam_elems_per_block(int dtype) {
  return kThreads * (dtype == DT_F32 ? 4 : 8) * 4;
}

int prologue_tiles(int rows, int cols, int dtype) {
  const int tile_cols = 16 * (dtype == DT_F32 ? 4 : 8);
  return ((cols + tile_cols - 1) / tile_cols) * ((rows + kTileRows - 1) / kTileRows);
}

int launch_prologue(const PrologueArgs& a, int dtype, int transpose, cudaStream_t stream) {
  const int tile_cols = 16 * (dtype == DT_F32 ? 4 : 8);
  long long tiles = (long long)((a.cols + tile_cols - 1) / tile_cols) *
                    ((a.rows + kTileRows - 1) / kTileRows) * a.count;
  int grid = grid_for(tiles, 8);
  if (grid < 0) return ERR_UNSUPPORTED;
  const double b = dtype == DT_F32 ? 4 : 2;  // read g, m; write m (+ g with Nesterov); write bf16 X
  LaunchScope scope(K_PROLOGUE, (double)a.rows * a.cols * a.count * (3 * b + 2 + (a.nesterov ? b : 0)),
                    stream);
  if (dtype == DT_F32) {
    if (transpose) prologue_kernel<float, true><<<grid, kThreads, 0, stream>>>(a);
    else prologue_kernel<float, false><<<grid, kThreads, 0, stream>>>(a);
  } else if (dtype == DT_F16) {
    if (transpose) prologue_kernel<__half, true><<<grid, kThreads, 0, stream>>>(a);
    else prologue_kernel<__half, false><<<grid, kThreads, 0, stream>>>(a);
  } else {
    if (transpose) prologue_kernel<__nv_bfloat16, true><<<grid, kThreads, 0, stream>>>(a);
    else prologue_kernel<__nv_bfloat16, false><<<grid, kThreads, 0, stream>>>(a);
  }
  MB_CUDA_CHECK(cudaGetLastError());
  return OK;
}

template <typename T, bool TRANSPOSE>
void launch_epilogue_variant(int grid, const EpilogueArgs& a, const EpiloguePeers* peers, cudaStream_t stream) {
  if (peers && peers->n_peers > 0) {
    epilogue_kernel<T, TRANSPOSE, true><<<grid, kThreads, 0, stream>>>(a, *peers);
  } else {
    EpiloguePeers none;
    none.n_peers = 0;
    epilogue_kernel<T, TRANSPOSE, false><<<grid, kThreads, 0, stream>>>(a, none);
  }
}

int launch_epilogue(const EpilogueArgs& a, int dtype, int transpose, cudaStream_t stream,
                    const EpiloguePeers* peers) {
  const int tile_cols = 16 * (dtype == DT_F32 ? 4 : 8);
  long long tiles = (long long)((a.cols + tile_cols - 1) / tile_cols) *
                    ((a.rows + kTileRows - 1) / kTileRows) * a.count;
  int grid = grid_for(tiles, 8);
  if (grid < 0) return ERR_UNSUPPORTED;
  const double b = dtype == DT_F32 ? 4 : 2;  // read bf16 U; read and write p (peer copies not counted)
  LaunchScope scope(K_EPILOGUE, (double)a.rows * a.cols * a.count * (2 * b + 2), stream);
  if (dtype == DT_F32) {
    if (transpose) launch_epilogue_variant<float, true>(grid, a, peers, stream);
    else launch_epilogue_variant<float, false>(grid, a, peers, stream);
  } else if (dtype == DT_F16) {
    if (transpose) launch_epilogue_variant<__half, true>(grid, a, peers, stream);
    else launch_epilogue_variant<__half, false>(grid, a, peers, stream);
  } else {
    if (transpose) launch_epilogue_variant<__nv_bfloat16, true>(grid, a, peers, stream);
    else launch_epilogue_variant<__nv_bfloat16, false>(grid, a, peers, stream);
  }
  MB_CUDA_CHECK(cudaGetLastError());
  return OK;
}

int launch_aol_rescale(__nv_bfloat16* X, long long ldx, long long x_bs, const __nv_bfloat16* A,
                       __nv_bfloat16* A_out, long long lda, long long a_bs, float* svec,
                       long long s_bs, int m, int n, int batch, float eps, cudaStream_t stream) {
  int grid = grid_for((long long)m * batch, 16);
  if (grid < 0) return ERR_UNSUPPORTED;
  // read + write A (m x m) and X (m x n), bf16
  LaunchScope scope(K_AOL_RESCALE, 4.0 * m * ((double)m + n) * batch, stream);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent_launch_enabled() ? 1 : 0;
  MB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, aol_rescale_kernel, X, ldx, x_bs, A, A_out, lda, a_bs, svec, s_bs,
                                   m, n, batch, eps));
  MB_CUDA_CHECK(cudaGetLastError());
  return OK;
}

int launch_fro_scales(const __nv_bfloat16* X, long long ldx, long long x_bs, int m, int n, int batch,
                      float eps, float* partials, int chunks, const float* tile_sumsq, long long tile_bs,
                      int tile_count, float* scales, cudaStream_t stream) {
  if (!tile_sumsq) {
    // nobody summed while X was produced: one pass over X (bf16)
    LaunchScope scope(K_FRO_NORMALIZE, 2.0 * m * (double)n * batch, stream);
    sumsq_partial_kernel<<<dim3(chunks, batch), kThreads, 0, stream>>>(X, ldx, x_bs, m, n, chunks, partials);
    MB_CUDA_CHECK(cudaGetLastError());
  }
  LaunchScope scope(K_FRO_NORMALIZE, 4.0 * (tile_sumsq ? tile_count : chunks) * batch, stream);
  if (tile_sumsq) fro_finish_kernel<<<batch, kThreads, 0, stream>>>(tile_sumsq, tile_bs, tile_count, eps, scales, batch);
  else fro_finish_kernel<<<batch, kThreads, 0, stream>>>(partials, chunks, chunks, eps, scales, batch);
  MB_CUDA_CHECK(cudaGetLastError());
  return OK;
}

int launch_cast_bf16(const void* src, int dtype, long long ld_src, long long src_bs, __nv_bfloat16* dst,
                     long long ld_dst, long long dst_bs, int rows, int cols, int batch, int transpose,
                     float scale, cudaStream_t stream) {
  const long long tiles = (long long)((cols + 31) / 32) * ((rows + 31) / 32) * batch;
  int grid = grid_for(tiles, 8);
  if (grid < 0) return ERR_UNSUPPORTED;
#define MB_CAST(T)                                                                                      \
  do {                                                                                                  \
    if (transpose)                                                                                      \
      cast_bf16_kernel<T, true><<<grid, kThreads, 0, stream>>>(static_cast<const T*>(src), ld_src, src_bs, \
                                                               dst, ld_dst, dst_bs, rows, cols, batch, scale); \
    else                                                                                                \
      cast_bf16_kernel<T, false><<<grid, kThreads, 0, stream>>>(static_cast<const T*>(src), ld_src, src_bs, \
                                                                dst, ld_dst, dst_bs, rows, cols, batch, scale); \
  } while (0)
  switch (dtype) {
    case DT_F32: MB_CAST(float); break;
    case DT_BF16: MB_CAST(__nv_bfloat16); break;
    case DT_F16: MB_CAST(__half); break;
    case DT_F64: MB_CAST(double); break;
    default: return set_error(ERR_INVALID_ARG, "cast: unknown element type %d", dtype);
  }
#undef MB_CAST
  MB_CUDA_CHECK(cudaGetLastError());
  return OK;
}

int launch_adam(const AdamArgs& a, int dtype, cudaStream_t stream) {
  int blocks = a.block_start[a.count];
  if (blocks <= 0) return OK;
  double elems = 0;
  for (int i = 0; i < a.count; ++i) elems += (double)a.numel[i];
  LaunchScope scope(K_ADAM, elems * 7 * (dtype == DT_F32 ? 4 : 2), stream);  // read p,g,m,v; write p,m,v
  if (dtype == DT_F32) adam_kernel<float><<<blocks, kThreads, 0, stream>>>(a);
  else if (dtype == DT_F16) adam_kernel<__half><<<blocks, kThreads, 0, stream>>>(a);
  else adam_kernel<__nv_bfloat16><<<blocks, kThreads, 0, stream>>>(a);
  MB_CUDA_CHECK(cudaGetLastError());
  return OK;
}

}  // namespace mb
