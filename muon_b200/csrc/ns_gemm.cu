// Newton-Schulz GEMMs for sm_100a: one persistent, warp-specialised tcgen05 kernel
// family covering the three products of an iteration.
//
//   line 1  A  = X · Xᵀ                       (reference ns_line_1_kernel, muon.py:349-417)
//   line 2  B  = alpha · A · Aᵀ + beta · A     (reference ns_line_2_kernel, muon.py:464-544)
//   line 3  X' = a · X + B · X                 (reference ns_line_3_kernel, muon.py:639-702)
//
// All operands are bf16, accumulation is fp32 in tensor memory, and every output
// element is rounded to bf16 exactly once, after the fused epilogue arithmetic
// (muon.py:404-405, :528-532, :696-697).
//
// Lines 1 and 2 only visit output tiles that touch the lower triangle. Inside such a
// tile the values with row >= col are computed once, stored at (row, col) and
// mirrored to (col, row); nothing above the diagonal is stored from its own position,
// so the result is deterministic.
// Line 2 with a non-symmetric A (first iteration: A/s scales rows only, muon.py:785):
// the reference stores every computed tile and then its transpose (muon.py:534-544), so
// outside the tiles on the diagonal its output is the finished lower-triangle value,
// addend beta*A[row, col] included, mirrored; on a diagonal tile the transposed store
// lands last and the tile ends up holding its own transpose. With the 64 x 64 tiles its
// autotuner picks on a B200 for every m <= 1024 that result is deterministic, and it is
// what this kernel reproduces: finished values mirrored everywhere, the two addends
// swapped inside the 64 x 64 blocks of the diagonal.
//
// Roles inside a CTA (64 + 32 * EW threads, EW = 4 or 8 epilogue warps):
//   warp 0      TMA producer: fills a ring of {A tile, B tile} stages in shared memory
//   warp 1      MMA issuer: tcgen05.mma, K = 16 per instruction, accumulators double-buffered
//               in TMEM (2 x 256 columns)
//   warps 2..   epilogue: tcgen05.ld -> fp32 epilogue -> bf16 stores (+ mirrored stores)
// The grid is persistent: each CTA (or CTA pair) walks tiles w, w + stride, ...
#include "common.cuh"
#include "elementwise.h"
#include "ns_gemm.h"
#include "profiling.h"

#include <cuda.h>
#include <cuda_fp8.h>
#include <atomic>
#include <cstdlib>
#include <mutex>

namespace mb {

__device__ int g_device_status = 0;

int read_device_status(int* status_out) {
  MB_CUDA_CHECK(cudaDeviceSynchronize());
  MB_CUDA_CHECK(cudaMemcpyFromSymbol(status_out, g_device_status, sizeof(int)));
  return OK;
}
int clear_device_status() {
  int zero = 0;
  MB_CUDA_CHECK(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
  return OK;
}

namespace {

constexpr int BM = 128;  // rows of the output tile each CTA owns (TMEM lanes)
constexpr int BN = 256;  // UMMA N
constexpr int BK = 64;   // one 128-byte swizzle span of bf16
constexpr int UMMA_K = 16;
constexpr int TMEM_COLS = 512;  // two 256-column fp32 accumulators
// Threads of a CTA with EW epilogue warps (warp 0 = TMA producer, warp 1 = MMA issuer).
__host__ __device__ constexpr int num_threads(int epi_warps) { return 64 + 32 * epi_warps; }
constexpr int SMEM_BARRIER_BYTES = 256;

// CTAS = 1: one CTA computes a 128 x 256 tile (tcgen05.mma.cta_group::1, M = 128).
// CTAS = 2: a cluster of two CTAs computes a 256 x 256 tile with one cta_group::2 MMA
//           (M = 256): each CTA stages its 128 rows of the A tile and its 128 of the 256
//           rows of the B tile, so per FLOP a third less operand traffic leaves L2 and
//           each SM's shared memory is read half as often for B.
template <int CTAS>
struct Cfg {
  static constexpr int TILE_M = BM * CTAS;
  static constexpr int B_ROWS = BN / CTAS;               // B-operand rows this CTA stages
  static constexpr int STAGES = CTAS == 1 ? 4 : 6;
  static constexpr int A_STAGE_BYTES = BM * BK * 2;       // 16 KiB
  static constexpr int B_STAGE_BYTES = B_ROWS * BK * 2;   // 32 / 16 KiB
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  // operand ring + barriers + one epilogue staging buffer per epilogue warp + alignment slack
  static constexpr int smem_total(int epi_warps) {
    return STAGES * STAGE_BYTES + SMEM_BARRIER_BYTES + epi_warps * 32 * 64 + 1024;
  }
};

struct TileCoord {
  int batch, tm, tn;
};

// Linear tile index -> (batch, tile row, tile col). For the triangular schedule row
// tile i (tile_m rows) owns the column tiles j with j*BN <= i*tile_m + tile_m - 1.
__host__ __device__ __forceinline__ int tri_row_count(int i, int tiles_n, int tile_m) {
  int c = (i * tile_m + tile_m - 1) / BN + 1;
  return c < tiles_n ? c : tiles_n;
}

template <int TILE_M>
__device__ __forceinline__ TileCoord decode_tile(int t, const GemmParams& p) {
  TileCoord tc;
  tc.batch = t / p.tiles_per_batch;
  int r = t - tc.batch * p.tiles_per_batch;
  if (!p.triangular) {
    // Row tiles vary fastest: the CTAs of one wave share a few 256-column slabs of the wide
    // operand X, which is then streamed from HBM once, while the small square operand
    // (every row tile reads a different part of it) stays resident in L2.
    tc.tn = r / p.tiles_m;
    tc.tm = r - tc.tn * p.tiles_m;
    return tc;
  }
  int i = 0;
  for (; i < p.tiles_m; ++i) {
    int c = tri_row_count(i, p.tiles_n, TILE_M);
    if (r < c) break;
    r -= c;
  }
  tc.tm = i;
  tc.tn = r;
  return tc;
}

// Instruction descriptor: bf16 x bf16 (kind::f16) or e4m3 x e4m3 (kind::f8f6f4) -> fp32, N = 256,
// A K-major, B K- or MN-major.
__host__ __device__ constexpr uint32_t make_idesc(bool b_mn_major, int mma_m, bool e4m3) {
  return (1u << 4)                         // D format: f32
         | ((e4m3 ? 0u : 1u) << 7)         // A format: kind::f16 1 = bf16; kind::f8f6f4 0 = e4m3
         | ((e4m3 ? 0u : 1u) << 10)        // B format
         | ((b_mn_major ? 1u : 0u) << 16)  // B major: 0 = K, 1 = MN
         | (uint32_t(BN >> 3) << 17)       // N
         | (uint32_t(mma_m >> 4) << 24);   // M
}

// ---------------------------------------------------------------------------
// Epilogue helpers. Thread owns one output row `r` and 32 consecutive columns.
// ---------------------------------------------------------------------------
// 32 columns of the row `src` points at, as packed bf16 pairs, not yet converted: issued one chunk
// ahead so that the global-memory latency passes while the previous chunk is converted and
// stored. Vector path when the whole span is in range (16-byte aligned because leading
// dimensions and col0 are multiples of 8).
__device__ __forceinline__ void load_row32_raw(const __nv_bfloat16* src, int col0, int ncols,
                                               uint32_t (&raw)[16]) {
  if (col0 + 32 <= ncols) {
    const uint4* v = reinterpret_cast<const uint4*>(src + col0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 q = __ldg(v + i);
      raw[4 * i] = q.x; raw[4 * i + 1] = q.y; raw[4 * i + 2] = q.z; raw[4 * i + 3] = q.w;
    }
  } else {
    const unsigned short* s = reinterpret_cast<const unsigned short*>(src);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int c = col0 + 2 * j;
      const uint32_t lo = (c < ncols) ? __ldg(s + c) : 0u;
      const uint32_t hi = (c + 1 < ncols) ? __ldg(s + c + 1) : 0u;
      raw[j] = lo | (hi << 16);
    }
  }
}
__device__ __forceinline__ void unpack_row32(const uint32_t (&raw)[16], float (&dst)[32]) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    dst[2 * j] = bf16_bits_to_float(raw[j] & 0xffffu);
    dst[2 * j + 1] = bf16_bits_to_float(raw[j] >> 16);
  }
}

__device__ __forceinline__ void store_row32(__nv_bfloat16* dst, int col0, int col_end,
                                            const uint32_t (&packed)[16]) {
  // Stores columns [col0, min(col0+32, col_end)) of one row.
  if (col0 + 32 <= col_end) {
    uint4* v = reinterpret_cast<uint4*>(dst + col0);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      v[i] = make_uint4(packed[i * 4], packed[i * 4 + 1], packed[i * 4 + 2], packed[i * 4 + 3]);
  } else {
    unsigned short* s = reinterpret_cast<unsigned short*>(dst);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      int c = col0 + j;
      if (c < col_end) {
        uint32_t w = packed[j >> 1];
        s[c] = static_cast<unsigned short>((j & 1) ? (w >> 16) : (w & 0xffffu));
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Per-warp staging buffer: 32 rows x 64 bytes of shared memory, the four 16-byte pieces of a
// row XOR-swizzled by the row pair. The accumulator arrives with one row per thread, so a
// thread's 64 bytes of a row are contiguous but the rows of a warp are a pitch apart: stored
// straight from registers, every 16-byte store instruction touches 32 different lines. Passing
// the block through this buffer changes the mapping to four lanes per row, eight rows per
// instruction (8 x 64 contiguous bytes), for the stores and for the addend loads alike.
//   "row"  pattern: lane l owns row l, pieces 0..3
//   "coal" pattern: instruction i, lane l -> row 8i + l/4, piece l%4
// Both patterns are free of bank conflicts with this swizzle.
// ---------------------------------------------------------------------------
constexpr int STAGING_BYTES_PER_WARP = 32 * 64;

__device__ __forceinline__ uint32_t stage_addr(uint32_t base, int row, int piece) {
  return base + row * 64 + ((piece ^ ((row >> 1) & 3)) << 4);
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}
__device__ __forceinline__ void lds128(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr)
               : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void stage_put_row(uint32_t base, int lane, const uint32_t (&w)[16]) {
#pragma unroll
  for (int k = 0; k < 4; ++k)
    sts128(stage_addr(base, lane, k), w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
}
__device__ __forceinline__ void stage_get_row(uint32_t base, int lane, uint32_t (&w)[16]) {
#pragma unroll
  for (int k = 0; k < 4; ++k)
    lds128(stage_addr(base, lane, k), w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
}
__device__ __forceinline__ void stage_put_coal(uint32_t base, int lane, const uint32_t (&w)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
    sts128(stage_addr(base, 8 * i + (lane >> 2), lane & 3), w[4 * i], w[4 * i + 1], w[4 * i + 2],
           w[4 * i + 3]);
}
__device__ __forceinline__ void stage_get_coal(uint32_t base, int lane, uint32_t (&w)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
    lds128(stage_addr(base, 8 * i + (lane >> 2), lane & 3), w[4 * i], w[4 * i + 1], w[4 * i + 2],
           w[4 * i + 3]);
}
// A 32 x 32 bf16 block at (row0, col0) of a matrix with pitch ld, in the "coal" pattern. The
// block must lie inside the matrix; col0 is a multiple of 32 and ld of 8, so every access is
// 16-byte aligned.
__device__ __forceinline__ void block_load_coal(const __nv_bfloat16* base, long long ld, int row0,
                                                int col0, int lane, uint32_t (&w)[16]) {
  const __nv_bfloat16* ptr = base + (row0 + (lane >> 2)) * ld + col0 + (lane & 3) * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(ptr + 8 * i * ld));
    w[4 * i] = q.x; w[4 * i + 1] = q.y; w[4 * i + 2] = q.z; w[4 * i + 3] = q.w;
  }
}
__device__ __forceinline__ void block_store_coal(__nv_bfloat16* base, long long ld, int row0, int col0,
                                                 int lane, const uint32_t (&w)[16]) {
  __nv_bfloat16* ptr = base + (row0 + (lane >> 2)) * ld + col0 + (lane & 3) * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<uint4*>(ptr + 8 * i * ld) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
}

// The same two for data that is touched exactly once by the launch (the parameters a fused update
// reads and rewrites): streaming accesses, so that they do not push the operand matrices, which
// every tile re-reads, out of L2.
__device__ __forceinline__ void block_load_stream(const __nv_bfloat16* base, long long ld, int row0,
                                                  int col0, int lane, uint32_t (&w)[16]) {
  const __nv_bfloat16* ptr = base + (row0 + (lane >> 2)) * ld + col0 + (lane & 3) * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 q = __ldcs(reinterpret_cast<const uint4*>(ptr + 8 * i * ld));
    w[4 * i] = q.x; w[4 * i + 1] = q.y; w[4 * i + 2] = q.z; w[4 * i + 3] = q.w;
  }
}
__device__ __forceinline__ void block_store_stream(__nv_bfloat16* base, long long ld, int row0, int col0,
                                                   int lane, const uint32_t (&w)[16]) {
  __nv_bfloat16* ptr = base + (row0 + (lane >> 2)) * ld + col0 + (lane & 3) * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    __stcs(reinterpret_cast<uint4*>(ptr + 8 * i * ld), make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]));
}

// ---------------------------------------------------------------------------
// e4m3 copies of an output block (see Fp8Spec in ns_gemm.h).
// ---------------------------------------------------------------------------
// Eight bf16 values (four packed words) times a power-of-two scale -> eight e4m3 bytes.
__device__ __forceinline__ uint2 bf16x8_to_e4m3x8(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3,
                                                  float scale) {
  const uint32_t w[4] = {w0, w1, w2, w3};
  uint32_t h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = make_float2(bf16_bits_to_float(w[i] & 0xffffu) * scale, bf16_bits_to_float(w[i] >> 16) * scale);
    h[i] = __nv_cvt_float2_to_fp8x2(v, __NV_SATFINITE, __NV_E4M3);
  }
  return make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
}
__device__ __forceinline__ uint8_t bf16_to_e4m3(uint32_t bits16, float scale, float minus) {
  return static_cast<uint8_t>(
      __nv_cvt_float_to_fp8((bf16_bits_to_float(bits16) - minus) * scale, __NV_SATFINITE, __NV_E4M3));
}
// A 32 x 32 block held in the "coal" pattern (instruction i, lane l: row 8i + l/4, eight columns
// from 8 * (l%4)) -> e4m3 at (row0, col0) of a byte matrix with pitch ld: 32 contiguous bytes per row.
__device__ __forceinline__ void block_store_coal_e4m3(uint8_t* base, long long ld, int row0, int col0,
                                                      int lane, const uint32_t (&w)[16], float scale) {
  uint8_t* ptr = base + (row0 + (lane >> 2)) * ld + col0 + (lane & 3) * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<uint2*>(ptr + 8 * i * ld) =
        bf16x8_to_e4m3x8(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3], scale);
}

// ---------------------------------------------------------------------------
// Fused parameter update (reference muon.py:14 and :66-67, see UpdateSpec in ns_gemm.h): the
// last line 3 of an orthogonalisation applies its output to the parameter instead of storing it.
//   u' = bf16(U * scale);  p1 = T(p * decay);  p = T(p1 - lr * u')        (T = parameter dtype)
// The same operations, in the same order and with the same roundings, as epilogue_kernel.
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float upd_round(float v);
template <>
__device__ __forceinline__ float upd_round<float>(float v) { return v; }
template <>
__device__ __forceinline__ float upd_round<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <typename T>
__device__ __forceinline__ float upd_apply(float pv, float u_bf16, float scale, float decay, float neg_lr) {
  const float us = __bfloat162float(__float2bfloat16_rn(u_bf16 * scale));
  const float p1 = upd_round<T>(pv * decay);
  return upd_round<T>(fmaf(neg_lr, us, p1));
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr) : "memory");
  return v;
}
// A 32-row x 16-float block (64 bytes per row, like a 32 x 32 bf16 block) in the "coal" pattern.
__device__ __forceinline__ void block_load_coal_f32(const float* base, long long ld, int row0, int col0,
                                                    int lane, uint32_t (&w)[16]) {
  const float* ptr = base + (row0 + (lane >> 2)) * ld + col0 + (lane & 3) * 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 q = __ldcs(reinterpret_cast<const uint4*>(ptr + 8 * i * ld));
    w[4 * i] = q.x; w[4 * i + 1] = q.y; w[4 * i + 2] = q.z; w[4 * i + 3] = q.w;
  }
}
__device__ __forceinline__ void block_store_coal_f32(float* base, long long ld, int row0, int col0, int lane,
                                                     const uint32_t (&w)[16]) {
  float* ptr = base + (row0 + (lane >> 2)) * ld + col0 + (lane & 3) * 4;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    __stcs(reinterpret_cast<uint4*>(ptr + 8 * i * ld), make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]));
}

// ADD: how line 2's addend is formed (AddendMode); the other two lines pass ADD_SYMMETRIC.
// VAR: a Variant (e4m3 operands / extra e4m3 output / fused parameter update).
template <int MODE, bool B_MN, int CTAS, int EW, int ADD, int VAR>
__global__ void __launch_bounds__(num_threads(EW), 1)
ns_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ GemmParams p) {
  using C = Cfg<CTAS>;
  constexpr int STAGES = C::STAGES;
  constexpr int TILE_M = C::TILE_M;
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_abort;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * C::STAGE_BYTES;
  // barrier layout (8 bytes each): full[STAGES], empty[STAGES], tfull[2], tempty[2], tmem slot
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
  const uint32_t stage_area = bar_base + SMEM_BARRIER_BYTES;  // EW staging buffers of the epilogue
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(
      smem_gen + STAGES * C::STAGE_BYTES + 8 * (2 * STAGES + 4));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // In a pair, CTA 0 issues the MMAs and owns the barriers the pair shares (full, tempty).
  const uint32_t cta_rank = CTAS == 2 ? cluster_cta_rank() : 0u;
  const bool leader = cta_rank == 0;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), EW * CTAS);  // one arrival per epilogue warp of every CTA
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    if (CTAS == 2) {
      tmem_alloc_pair(tmem_slot, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();  // the peer's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  // Everything above (barriers, tensor memory, descriptor prefetch) touches no memory that an
  // earlier kernel writes, so with a programmatic dependent launch it overlaps the tail of the
  // kernel before this one in the stream; all global-memory traffic comes after the wait. The
  // kernel after this one may start its own set-up on every SM this grid leaves.
  griddep_launch_dependents();
  griddep_wait();

  // One shared-memory stage holds 128 bytes of K per row: 64 bf16 or 128 e4m3 elements.
  constexpr int KSTEP = VAR == F8_OPERANDS ? 2 * BK : BK;
  const int k_blocks = (p.K + KSTEP - 1) / KSTEP;
  // Split-K (line 1 of launches with far fewer tiles than SMs, see launch_ns_gemm): a work item is
  // then one K-slice of a tile and its fp32 partial sums go to p.partial, where
  // splitk_reduce_kernel finds them. Otherwise a work item is a tile.
  constexpr bool kCanSplit = MODE == MODE_SYRK && VAR == F8_NONE;
  const int split_phase = kCanSplit ? p.split_phase : 0;
  const int work_per_tile = split_phase == 1 ? p.split_k : 1;
  const int total_tiles = p.tiles_per_batch * p.batch * work_per_tile;
  const int work0 = blockIdx.x / CTAS;
  const int work_stride = gridDim.x / CTAS;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = work0; t < total_tiles && ok; t += work_stride) {
        const TileCoord tc = decode_tile<TILE_M>(t / work_per_tile, p);
        const int a_row = tc.tm * TILE_M + (int)cta_rank * BM;
        const int b_row = tc.tn * BN + (int)cta_rank * C::B_ROWS;
        const int kb_first = split_phase == 1 ? (t % work_per_tile) * p.split_kb : 0;
        const int kb_last = split_phase == 1 && kb_first + p.split_kb < k_blocks ? kb_first + p.split_kb : k_blocks;
        for (int kb = kb_first; kb < kb_last; ++kb) {
          const bool freed = CTAS == 2 ? mbar_wait_bounded_cluster(empty_bar(stage), phase ^ 1u, &s_abort)
                                       : mbar_wait_bounded(empty_bar(stage), phase ^ 1u, &s_abort);
          if (!freed) {
            atomicCAS(&g_device_status, 0, 1);
            s_abort = 1;
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * C::STAGE_BYTES;
          const uint32_t sb = sa + C::A_STAGE_BYTES;
          if (CTAS == 2) {
            // Both CTAs' copies complete on the leader's barrier, which expects both halves.
            const uint32_t full = map_to_cta(full_bar(stage), 0);
            if (leader) mbar_expect_tx(full_bar(stage), 2 * C::STAGE_BYTES);
            tma_load_3d_pair(sa, &tmap_a, full, kb * KSTEP, a_row, tc.batch);
            if (!B_MN) {
              tma_load_3d_pair(sb, &tmap_b, full, kb * KSTEP, b_row, tc.batch);
            } else {
#pragma unroll
              for (int c = 0; c < C::B_ROWS / 64; ++c)
                tma_load_3d_pair(sb + c * (BK * 128), &tmap_b, full, b_row + c * 64, kb * BK, tc.batch);
            }
          } else {
            mbar_expect_tx(full_bar(stage), C::STAGE_BYTES);
            tma_load_3d(sa, &tmap_a, full_bar(stage), kb * KSTEP, a_row, tc.batch);
            if (!B_MN) {
              // B operand rows are output columns; K contiguous.
              tma_load_3d(sb, &tmap_b, full_bar(stage), kb * KSTEP, b_row, tc.batch);
            } else {
              // B operand is [K, N] with N contiguous: 64-column slabs of 64 k-rows.
#pragma unroll
              for (int c = 0; c < C::B_ROWS / 64; ++c)
                tma_load_3d(sb + c * (BK * 128), &tmap_b, full_bar(stage), b_row + c * 64, kb * BK,
                            tc.batch);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Let copies that are still in flight land before shared memory goes away.
        for (int i = 0; i < 100; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc(B_MN, TILE_M, VAR == F8_OPERANDS);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int t = work0; t < total_tiles && ok; t += work_stride, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        const int kb_first = split_phase == 1 ? (t % work_per_tile) * p.split_kb : 0;
        const int kb_last = split_phase == 1 && kb_first + p.split_kb < k_blocks ? kb_first + p.split_kb : k_blocks;
        const bool drained = CTAS == 2
                                 ? mbar_wait_bounded_cluster(tempty_bar(acc), acc_phase ^ 1u, &s_abort)
                                 : mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1u, &s_abort);
        if (!drained) {
          atomicCAS(&g_device_status, 0, 3);
          s_abort = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb_first; kb < kb_last; ++kb) {
          const bool filled = CTAS == 2 ? mbar_wait_bounded_cluster(full_bar(stage), phase, &s_abort)
                                        : mbar_wait_bounded(full_bar(stage), phase, &s_abort);
          if (!filled) {
            atomicCAS(&g_device_status, 0, 2);
            s_abort = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * C::STAGE_BYTES;
          const uint32_t sb = sa + C::A_STAGE_BYTES;
          // K-major tiles: rows of 128 bytes, 8-row groups 1024 bytes apart.
          const uint64_t a_desc = make_smem_desc_sw128(sa, 16, 1024);
          // MN-major B: 64-column slabs BK*128 bytes apart, 8-k groups 1024 bytes apart.
          const uint64_t b_desc =
              B_MN ? make_smem_desc_sw128(sb, BK * 128, 1024) : make_smem_desc_sw128(sb, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t a_adv = static_cast<uint64_t>((kk * UMMA_K * 2) >> 4);
            const uint64_t b_adv = B_MN ? static_cast<uint64_t>((kk * UMMA_K * 128) >> 4)
                                        : static_cast<uint64_t>((kk * UMMA_K * 2) >> 4);
            const uint32_t accumulate = (kb != kb_first || kk != 0) ? 1u : 0u;
            // 32 bytes of K per instruction either way: 16 bf16 or 32 e4m3 elements.
            if constexpr (VAR == F8_OPERANDS) {
              if (CTAS == 2) umma_f8_ss_pair(d_tmem, a_desc + a_adv, b_desc + b_adv, idesc, accumulate);
              else umma_f8_ss(d_tmem, a_desc + a_adv, b_desc + b_adv, idesc, accumulate);
            } else {
              if (CTAS == 2) umma_bf16_ss_pair(d_tmem, a_desc + a_adv, b_desc + b_adv, idesc, accumulate);
              else umma_bf16_ss(d_tmem, a_desc + a_adv, b_desc + b_adv, idesc, accumulate);
            }
          }
          // Frees the stage (in both CTAs of a pair) once these MMAs have read it.
          if (CTAS == 2) umma_commit_pair(empty_bar(stage), 0x3);
          else umma_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {  // accumulator complete: wake the epilogue warps (of both CTAs)
          if (CTAS == 2) umma_commit_pair(tfull_bar(acc), 0x3);
          else umma_commit(tfull_bar(acc));
        }
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    // A warp may only read the TMEM lanes of quarter (warp id % 4). With EW = 4 * PARTS epilogue
    // warps every quarter is served by PARTS warps, each taking a share of the tile's columns.
    // Each scheduler of the SM then interleaves PARTS epilogue warps: with a single one, the
    // dependent-instruction latency of the conversion and store code is fully exposed and a
    // short-K tile's epilogue takes several times longer than its MMAs.
    constexpr int PARTS = EW / 4;
    constexpr int CHUNKS = (BN / 32) / PARTS;  // 32-column chunks per warp and tile
    const int q = warp & 3;
    const int c_begin = ((warp - 2) >> 2) * CHUNKS;
    int local = 0;
    for (int t = work0; t < total_tiles; t += work_stride, ++local) {
      const TileCoord tc = decode_tile<TILE_M>(t / work_per_tile, p);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      const int row_base = tc.tm * TILE_M + (int)cta_rank * BM + q * 32;
      const int r = row_base + lane;  // output row of this thread
      const int r_warp_max = row_base + 31;
      const bool row_ok = r < p.M;
      __nv_bfloat16* out_b = p.out + static_cast<long long>(tc.batch) * p.out_bs;
      const __nv_bfloat16* add_b =
          (MODE == MODE_SYRK) ? nullptr : p.add + static_cast<long long>(tc.batch) * p.add_bs;
      __nv_bfloat16* out_row = out_b + static_cast<long long>(r) * p.ldo;
      // e4m3 copy of the output (null when this launch keeps none)
      uint8_t* out8_b = ((VAR == F8_OPERANDS || VAR == F8_EXTRA_OUT) && p.out8) ? p.out8 + static_cast<long long>(tc.batch) * p.out8_bs : nullptr;
      const __nv_bfloat16* add_row =
          (MODE == MODE_SYRK) ? nullptr : add_b + static_cast<long long>(r) * p.ldadd;

      // A chunk is worked on when it is inside the matrix and, for the triangular products, not
      // strictly above the diagonal for every row of this warp (both tests are warp-uniform).
      auto chunk_live = [&](int c) {
        const int col0 = tc.tn * BN + c * 32;
        return col0 < p.N && (MODE == MODE_BX || col0 <= r_warp_max);
      };
      // Global memory is accessed through the staging buffer when the chunk's whole 32 x 32 block
      // lies inside the matrix (warp-uniform); ragged edges use one row per thread.
      const bool rows_full = r_warp_max < p.M;
      auto chunk_full = [&](int c) { return rows_full && tc.tn * BN + c * 32 + 32 <= p.N; };
      const uint32_t stage = stage_area + (warp - 2) * STAGING_BYTES_PER_WARP;

      // Addend of the chunk about to be processed, fetched one chunk ahead ("coal" pattern for
      // a full chunk, this thread's own row otherwise); the first one before the accumulator is
      // waited for, so that its latency passes under the tile's last MMAs. (Two buffers taking
      // turns instead of the copy below were measured: no faster, and 25 registers more.)
      uint32_t add_raw[MODE == MODE_SYRK ? 1 : 16] = {};
      if constexpr (MODE != MODE_SYRK) {
        if (chunk_live(c_begin)) {
          const int col0 = tc.tn * BN + c_begin * 32;
          if (chunk_full(c_begin)) block_load_coal(add_b, p.ldadd, row_base, col0, lane, add_raw);
          else if (row_ok) load_row32_raw(add_row, col0, p.N, add_raw);
        }
      }

      int ok = (CTAS == 2 ? mbar_wait_bounded_cluster(tfull_bar(acc), acc_phase, &s_abort)
                          : mbar_wait_bounded(tfull_bar(acc), acc_phase, &s_abort))
                   ? 1
                   : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) {
          atomicCAS(&g_device_status, 0, 4);
          s_abort = 1;
        }
        break;
      }
      tc_fence_after();

#pragma unroll 1
      for (int c = c_begin; c < c_begin + CHUNKS; ++c) {
        if (!chunk_live(c)) break;
        const int col0 = tc.tn * BN + c * 32;
        const bool full = chunk_full(c);
        uint32_t v[32];
        __syncwarp();  // tcgen05.ld is warp-collective: reconverge after the predicated stores
        tmem_ld_x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32, v);
        uint32_t add_next[MODE == MODE_SYRK ? 1 : 16] = {};
        const bool more = MODE != MODE_SYRK && c + 1 < c_begin + CHUNKS && chunk_live(c + 1);
        if constexpr (MODE != MODE_SYRK) {
          if (more) {
            if (chunk_full(c + 1)) block_load_coal(add_b, p.ldadd, row_base, col0 + 32, lane, add_next);
            else if (row_ok) load_row32_raw(add_row, col0 + 32, p.N, add_next);
          }
        }
        tmem_ld_wait();

        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
        if constexpr (kCanSplit) {
          if (split_phase == 1) {
            // this slice's share of the chunk, as it is: splitk_reduce_kernel adds the slices
            float* dst = p.partial +
                (((static_cast<long long>(t) * CTAS + cta_rank) * 4 + q) * (BN / 32) + c) * 1024 + lane;
#pragma unroll
            for (int j = 0; j < 32; ++j) dst[j * 32] = f[j];
            continue;
          }
        }
        float a[MODE == MODE_SYRK ? 1 : 32];
        if constexpr (MODE != MODE_SYRK) {
          if (full) {
            uint32_t own[16];
            stage_put_coal(stage, lane, add_raw);
            __syncwarp();
            stage_get_row(stage, lane, own);
            __syncwarp();
            unpack_row32(own, a);
          } else {
            unpack_row32(add_raw, a);
          }
          if (more) {
#pragma unroll
            for (int j = 0; j < 16; ++j) add_raw[j] = add_next[j];
          }
        }

        // f keeps the product term (alpha * acc for line 2) so that the mirrored element can be
        // formed from it at store time; `packed` receives the value of position (r, col).
        uint32_t packed[16];
        float w_r = 0.f;                 // ADD_ROW_SCALED: 1/s of this thread's row
        const float* wv = nullptr;       // ADD_ROW_SCALED: the 1/s vector of this matrix
        if constexpr (MODE == MODE_AXPBY) {
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] *= p.alpha;
          if constexpr (VAR == F8_OPERANDS) {
            // The operand was E = A - I: the identity's share, diag * I, lands on the diagonal
            // (block on the diagonal: this thread's row is column `lane` of the chunk).
            if (col0 == row_base) {
#pragma unroll
              for (int j = 0; j < 32; ++j) f[j] += (j == lane) ? p.diag : 0.f;
            }
          }
          if constexpr (ADD == ADD_ROW_SCALED) {
            // The addend is S * w (rows scaled by w = 1/s), S symmetric and given unscaled:
            // bf16(S[r,col] * w[r]) is bit for bit what the materialised scaled matrix holds at
            // (r, col), bf16(S[r,col] * w[col]) what it holds at (col, r).
            wv = p.row_scale + static_cast<long long>(tc.batch) * p.scale_bs;
            w_r = row_ok ? wv[r] : 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float d0 = __bfloat162float(__float2bfloat16_rn(a[2 * j] * w_r));
              const float d1 = __bfloat162float(__float2bfloat16_rn(a[2 * j + 1] * w_r));
              packed[j] = pack_bf16x2(fmaf(d0, p.beta, f[2 * j]), fmaf(d1, p.beta, f[2 * j + 1]));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              packed[j] = pack_bf16x2(fmaf(a[2 * j], p.beta, f[2 * j]), fmaf(a[2 * j + 1], p.beta, f[2 * j + 1]));
          }
        } else if constexpr (MODE == MODE_BX) {
          if constexpr (VAR == V_BATCH_SCALE) {
            // X was not normalised: (alpha * X + B X) / (||X|| + eps), one rounding
            const float s = __ldg(p.batch_scale + tc.batch);
#pragma unroll
            for (int j = 0; j < 16; ++j)
              packed[j] = pack_bf16x2(fmaf(a[2 * j], p.alpha, f[2 * j]) * s, fmaf(a[2 * j + 1], p.alpha, f[2 * j + 1]) * s);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              packed[j] = pack_bf16x2(fmaf(a[2 * j], p.alpha, f[2 * j]), fmaf(a[2 * j + 1], p.alpha, f[2 * j + 1]));
          }
        } else {
          if constexpr (VAR == V_BATCH_SCALE) {
            const float s = __ldg(p.batch_scale + tc.batch);
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] *= s;
          }
          if constexpr (VAR == F8_OPERANDS) {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] *= p.acc_scale;  // the operands carried a power-of-two scale
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) packed[j] = pack_bf16x2(f[2 * j], f[2 * j + 1]);
        }

        if constexpr (MODE == MODE_BX && VAR >= V_UPD_BF16 && VAR <= V_UPD_F32) {
          // Last line 3 of the run: `packed` holds the bf16 Newton-Schulz output of row r, columns
          // col0 .. col0+31; it goes into the parameter instead of into the workspace.
          if constexpr (VAR == V_UPD_BF16) {
            // bf16 parameter [M, N] in the tile's orientation
            __nv_bfloat16* pb = static_cast<__nv_bfloat16*>(p.upd_param[tc.batch]);
            if (full) {
              uint32_t pw[16], own[16];
              block_load_stream(pb, p.N, row_base, col0, lane, pw);
              stage_put_coal(stage, lane, pw);
              __syncwarp();
              stage_get_row(stage, lane, own);
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float n0 = upd_apply<__nv_bfloat16>(bf16_bits_to_float(own[j] & 0xffffu),
                                                          bf16_bits_to_float(packed[j] & 0xffffu), p.upd_scale,
                                                          p.upd_decay, p.upd_neg_lr);
                const float n1 = upd_apply<__nv_bfloat16>(bf16_bits_to_float(own[j] >> 16),
                                                          bf16_bits_to_float(packed[j] >> 16), p.upd_scale,
                                                          p.upd_decay, p.upd_neg_lr);
                own[j] = pack_bf16x2(n0, n1);
              }
              stage_put_row(stage, lane, own);
              __syncwarp();
              stage_get_coal(stage, lane, pw);
              __syncwarp();
              block_store_stream(pb, p.N, row_base, col0, lane, pw);
            } else if (row_ok) {
              __nv_bfloat16* prow = pb + static_cast<long long>(r) * p.N;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int col = col0 + j;
                if (col < p.N) {
                  const uint32_t u = (j & 1) ? (packed[j >> 1] >> 16) : (packed[j >> 1] & 0xffffu);
                  prow[col] = __float2bfloat16_rn(upd_apply<__nv_bfloat16>(
                      __bfloat162float(prow[col]), bf16_bits_to_float(u), p.upd_scale, p.upd_decay, p.upd_neg_lr));
                }
              }
            }
          } else if constexpr (VAR == V_UPD_BF16_T) {
            // bf16 parameter [N, M]: the tile is its transpose; block (col0.., row_base..) of it
            __nv_bfloat16* pb = static_cast<__nv_bfloat16*>(p.upd_param[tc.batch]);
            if (full) {
              uint32_t pw[16], np[16];
              block_load_stream(pb, p.M, col0, row_base, lane, pw);
              stage_put_coal(stage, lane, pw);
              __syncwarp();
              // this thread's tile row r is column `lane` of the staged block: read it down the rows
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float o0 = bf16_bits_to_float(lds_u16(stage_addr(stage, 2 * j, lane >> 3) + (lane & 7) * 2));
                const float o1 = bf16_bits_to_float(lds_u16(stage_addr(stage, 2 * j + 1, lane >> 3) + (lane & 7) * 2));
                const float n0 = upd_apply<__nv_bfloat16>(o0, bf16_bits_to_float(packed[j] & 0xffffu), p.upd_scale,
                                                          p.upd_decay, p.upd_neg_lr);
                const float n1 = upd_apply<__nv_bfloat16>(o1, bf16_bits_to_float(packed[j] >> 16), p.upd_scale,
                                                          p.upd_decay, p.upd_neg_lr);
                np[j] = pack_bf16x2(n0, n1);
              }
              __syncwarp();
              // transposed store, as for the mirrored blocks of lines 1 and 2
              const int odd = lane & 1;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const uint32_t other = __shfl_xor_sync(0xffffffffu, np[j], 1);
                const uint32_t word = odd ? __byte_perm(other, np[j], 0x7632) : __byte_perm(np[j], other, 0x5410);
                sts32(stage_addr(stage, 2 * j + odd, lane >> 3) + ((lane & 6) << 1), word);
              }
              __syncwarp();
              stage_get_coal(stage, lane, pw);
              __syncwarp();
              block_store_stream(pb, p.M, col0, row_base, lane, pw);
            } else if (row_ok) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int col = col0 + j;
                if (col < p.N) {
                  __nv_bfloat16* pe = pb + static_cast<long long>(col) * p.M + r;
                  const uint32_t u = (j & 1) ? (packed[j >> 1] >> 16) : (packed[j >> 1] & 0xffffu);
                  *pe = __float2bfloat16_rn(upd_apply<__nv_bfloat16>(__bfloat162float(*pe), bf16_bits_to_float(u),
                                                                     p.upd_scale, p.upd_decay, p.upd_neg_lr));
                }
              }
            }
          } else {
            // fp32 parameter [M, N] in the tile's orientation: two halves of 16 columns, each a
            // 32-row x 64-byte block like a bf16 one
            float* pf = static_cast<float*>(p.upd_param[tc.batch]);
            if (full) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                uint32_t pw[16], own[16];
                block_load_coal_f32(pf, p.N, row_base, col0 + 16 * h, lane, pw);
                stage_put_coal(stage, lane, pw);
                __syncwarp();
                stage_get_row(stage, lane, own);
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const int jj = 16 * h + j;
                  const uint32_t u = (jj & 1) ? (packed[jj >> 1] >> 16) : (packed[jj >> 1] & 0xffffu);
                  own[j] = __float_as_uint(upd_apply<float>(__uint_as_float(own[j]), bf16_bits_to_float(u), p.upd_scale,
                                                            p.upd_decay, p.upd_neg_lr));
                }
                stage_put_row(stage, lane, own);
                __syncwarp();
                stage_get_coal(stage, lane, pw);
                __syncwarp();
                block_store_coal_f32(pf, p.N, row_base, col0 + 16 * h, lane, pw);
              }
            } else if (row_ok) {
              float* prow = pf + static_cast<long long>(r) * p.N;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int col = col0 + j;
                if (col < p.N) {
                  const uint32_t u = (j & 1) ? (packed[j >> 1] >> 16) : (packed[j >> 1] & 0xffffu);
                  prow[col] = upd_apply<float>(prow[col], bf16_bits_to_float(u), p.upd_scale, p.upd_decay, p.upd_neg_lr);
                }
              }
            }
          }
        } else if constexpr (MODE == MODE_BX) {
          if (full) {
            uint32_t w[16];
            stage_put_row(stage, lane, packed);
            __syncwarp();
            stage_get_coal(stage, lane, w);
            __syncwarp();
            block_store_coal(out_b, p.ldo, row_base, col0, lane, w);
            if constexpr (VAR == F8_EXTRA_OUT) {
              if (out8_b) block_store_coal_e4m3(out8_b, p.ldo8, row_base, col0, lane, w, p.out8_scale);
            }
          } else if (row_ok) {
            store_row32(out_row, col0, p.N, packed);
            if constexpr (VAR == F8_EXTRA_OUT) {
              if (out8_b) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const int col = col0 + j;
                  if (col < p.N) {
                    const uint32_t wv2 = packed[j >> 1];
                    out8_b[static_cast<long long>(r) * p.ldo8 + col] =
                        bf16_to_e4m3((j & 1) ? (wv2 >> 16) : (wv2 & 0xffffu), p.out8_scale, 0.f);
                  }
                }
              }
            }
          }
        } else {
          // Mirror: element (r, col) with col < r also lands at (col, r), with the same finished
          // value (addend included), which is what the reference's transposed store of every
          // off-diagonal tile leaves (muon.py:541-544). `mp` holds the values for the mirrored
          // positions.
          uint32_t mp[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) mp[j] = packed[j];
          if constexpr (MODE == MODE_AXPBY && ADD != ADD_SYMMETRIC) {
            // A not symmetric (first iteration, A / s). On a 64 x 64 tile of the diagonal the
            // reference stores the tile and then its transpose over it, so position (r, col)
            // ends up with the value computed for (col, r), i.e. with the addend beta * A[col, r],
            // and (col, r) with the one computed for (r, col). Both 32 x 32 blocks of this chunk
            // lie in one such tile or outside all of them: the test is the same for every lane.
            if ((row_base >> 6) == (col0 >> 6)) {
              if constexpr (ADD == ADD_ROW_SCALED) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  // A[col, r] = S[r, col] * w[col]; w[col] is one broadcast load for the warp.
                  const int col = col0 + 2 * j;
                  const float w0 = col < p.N ? __ldg(wv + col) : 0.f;
                  const float w1 = col + 1 < p.N ? __ldg(wv + col + 1) : 0.f;
                  const float m0 = __bfloat162float(__float2bfloat16_rn(a[2 * j] * w0));
                  const float m1 = __bfloat162float(__float2bfloat16_rn(a[2 * j + 1] * w1));
                  packed[j] = pack_bf16x2(fmaf(m0, p.beta, f[2 * j]), fmaf(m1, p.beta, f[2 * j + 1]));
                }
              } else {
                const unsigned short* add_s = reinterpret_cast<const unsigned short*>(add_b);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const int col = col0 + 2 * j;
                  float t0 = a[2 * j], t1 = a[2 * j + 1];
                  if (row_ok && col < r && col < p.N)
                    t0 = bf16_bits_to_float(__ldg(add_s + static_cast<long long>(col) * p.ldadd + r));
                  if (row_ok && col + 1 < r && col + 1 < p.N)
                    t1 = bf16_bits_to_float(__ldg(add_s + static_cast<long long>(col + 1) * p.ldadd + r));
                  packed[j] = pack_bf16x2(fmaf(t0, p.beta, f[2 * j]), fmaf(t1, p.beta, f[2 * j + 1]));
                }
              }
            }
          }

          if (full && col0 + 32 <= row_base) {
            // The whole block is strictly below the diagonal (the same for every lane): it is
            // stored as it is, and its transpose goes to (col0, row_base). For the transpose
            // neighbouring lanes, which hold neighbouring rows, swap one packed word per column
            // pair, so that the even lane holds rows (r, r+1) of column col0+2j and the odd lane
            // those of column col0+2j+1; these words are written into the buffer as rows col0+2j
            // and col0+2j+1 of the transposed block.
            uint32_t w[16];
            stage_put_row(stage, lane, packed);
            __syncwarp();
            stage_get_coal(stage, lane, w);
            __syncwarp();
            block_store_coal(out_b, p.ldo, row_base, col0, lane, w);
            if constexpr (VAR == F8_OPERANDS && MODE == MODE_SYRK) {
              // strictly below the diagonal: (A - I) = A here
              if (out8_b) block_store_coal_e4m3(out8_b, p.ldo8, row_base, col0, lane, w, p.out8_scale);
            }
            const int odd = lane & 1;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const uint32_t other = __shfl_xor_sync(0xffffffffu, mp[j], 1);
              const uint32_t word = odd ? __byte_perm(other, mp[j], 0x7632) : __byte_perm(mp[j], other, 0x5410);
              sts32(stage_addr(stage, 2 * j + odd, lane >> 3) + ((lane & 6) << 1), word);
            }
            __syncwarp();
            stage_get_coal(stage, lane, w);
            __syncwarp();
            block_store_coal(out_b, p.ldo, col0, row_base, lane, w);
            if constexpr (VAR == F8_OPERANDS && MODE == MODE_SYRK) {
              if (out8_b) block_store_coal_e4m3(out8_b, p.ldo8, col0, row_base, lane, w, p.out8_scale);
            }
          } else if (row_ok) {
            // Blocks on the diagonal and ragged edges: one row per thread, the lower triangle
            // (col <= r) from its own position, the elements with col < r also to (col, r).
            int col_end = r + 1 < p.N ? r + 1 : p.N;
            store_row32(out_row, col0, col_end, packed);
            unsigned short* out_s = reinterpret_cast<unsigned short*>(out_b);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int col = col0 + j;
              if (col < r && col < p.N) {
                const uint32_t w = mp[j >> 1];
                out_s[static_cast<long long>(col) * p.ldo + r] =
                    static_cast<unsigned short>((j & 1) ? (w >> 16) : (w & 0xffffu));
              }
            }
            if constexpr (VAR == F8_OPERANDS && MODE == MODE_SYRK) {
              if (out8_b) {
                // E8 = e4m3((A - I) * se), from the bf16 values just stored: own position for
                // col <= r (the diagonal loses its 1), mirrored position for col < r.
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const int col = col0 + j;
                  if (col <= r && col < p.N) {
                    const uint32_t w = packed[j >> 1];
                    const uint8_t e = bf16_to_e4m3((j & 1) ? (w >> 16) : (w & 0xffffu), p.out8_scale,
                                                   col == r ? 1.f : 0.f);
                    out8_b[static_cast<long long>(r) * p.ldo8 + col] = e;
                    if (col < r) out8_b[static_cast<long long>(col) * p.ldo8 + r] = e;
                  }
                }
              }
            }
          }
        }
      }
      // Accumulator drained: hand it back to the MMA warp (of the pair's leader).
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CTAS == 2) mbar_arrive_remote(map_to_cta(tempty_bar(acc), 0));
        else mbar_arrive(tempty_bar(acc));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  // A CTA of a pair must outlive every access its peer makes to its shared memory,
  // barriers and tensor memory.
  if (CTAS == 2) cluster_sync_all();
  tc_fence_after();
  if (warp == 1) {
    if (CTAS == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// Second launch of a line 1 that was split along K: one warp per 32-row x 8-column piece of the
// output adds the piece's K-slices in slice order (lane = row, so every load and every mirrored
// store is contiguous across the warp), rounds once and stores the piece and its mirror image
// with the rules of the GEMM epilogue: positions with col <= row from their own value, positions
// above the diagonal from the mirrored one. Pieces this narrow because the launches that are
// split have few tiles: four warps per 32 x 32 block put enough loads in flight on the few SMs
// that get work.
// ---------------------------------------------------------------------------
template <int CTAS>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const GemmParams p) {
  constexpr int TILE_M = BM * CTAS;
  constexpr int PIECES_PER_TILE = CTAS * 4 * (BN / 32) * 4;
  griddep_launch_dependents();
  griddep_wait();  // the partial sums come from the launch before this one
  const int lane = threadIdx.x & 31;
  const long long warp_global = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long total = static_cast<long long>(p.tiles_per_batch) * p.batch * PIECES_PER_TILE;
  if (warp_global >= total) return;
  const int tile = static_cast<int>(warp_global / PIECES_PER_TILE);
  int within = static_cast<int>(warp_global - static_cast<long long>(tile) * PIECES_PER_TILE);
  const int j0 = (within & 3) * 8;  // first of the piece's 8 columns inside its 32-column chunk
  within >>= 2;
  const int c = within % (BN / 32);
  const int q = (within / (BN / 32)) & 3;
  const int rank = within / (4 * (BN / 32));
  const TileCoord tc = decode_tile<TILE_M>(tile, p);
  const int row_base = tc.tm * TILE_M + rank * BM + q * 32;
  const int col0 = tc.tn * BN + c * 32 + j0;
  if (col0 >= p.N || col0 > row_base + 31 || row_base >= p.M) return;  // outside, or above the diagonal

  // Two slices per round: their 16 loads are in flight together, the additions keep slice order.
  const long long slice_pitch = static_cast<long long>(CTAS) * 4 * (BN / 32) * 1024;
  const float* src = p.partial +
      (((static_cast<long long>(tile) * p.split_k * CTAS + rank) * 4 + q) * (BN / 32) + c) * 1024 + j0 * 32 + lane;
  float sum[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) sum[j] = 0.f;
  int sl = 0;
  for (; sl + 1 < p.split_k; sl += 2) {
    float first[8], second[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) first[j] = __ldcg(src + j * 32);
#pragma unroll
    for (int j = 0; j < 8; ++j) second[j] = __ldcg(src + slice_pitch + j * 32);
#pragma unroll
    for (int j = 0; j < 8; ++j) sum[j] = (sum[j] + first[j]) + second[j];
    src += 2 * slice_pitch;
  }
  if (sl < p.split_k) {
#pragma unroll
    for (int j = 0; j < 8; ++j) sum[j] += __ldcg(src + j * 32);
  }

  const int r = row_base + lane;
  if (r >= p.M) return;
  unsigned short* out_s = reinterpret_cast<unsigned short*>(p.out + static_cast<long long>(tc.batch) * p.out_bs);
  uint32_t packed[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) packed[j] = pack_bf16x2(sum[2 * j], sum[2 * j + 1]);
  if (col0 + 8 <= row_base && col0 + 8 <= p.N) {
    // strictly below the diagonal and inside the matrix: the row's 16 bytes in one piece
    *reinterpret_cast<uint4*>(out_s + static_cast<long long>(r) * p.ldo + col0) =
        make_uint4(packed[0], packed[1], packed[2], packed[3]);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int col = col0 + j;
      if (col <= r && col < p.N)
        out_s[static_cast<long long>(r) * p.ldo + col] =
            static_cast<unsigned short>((j & 1) ? (packed[j >> 1] >> 16) : (packed[j >> 1] & 0xffffu));
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int col = col0 + j;
    if (col < r && col < p.N)
      out_s[static_cast<long long>(col) * p.ldo + r] =
          static_cast<unsigned short>((j & 1) ? (packed[j >> 1] >> 16) : (packed[j >> 1] & 0xffffu));
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// bf16 (elem_bytes 2) or e4m3 (elem_bytes 1) tensor [batch, rows, cols] with row pitch `ld` and
// batch pitch `bs` (elements). Box = box_rows x 128 bytes of columns, 128-byte swizzle, zero fill
// outside the tensor.
int encode_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld,
               int64_t bs, int batch, int box_rows, int elem_bytes = 2) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return set_error(ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
    return set_error(ERR_ALIGNMENT, "GEMM operand base %p is not 16-byte aligned", base);
  if ((ld * elem_bytes) % 16 != 0 || (batch > 1 && (bs * elem_bytes) % 16 != 0))
    return set_error(ERR_ALIGNMENT,
                     "GEMM operand pitch must be a multiple of 16 bytes (ld=%lld bs=%lld elements of %d bytes)",
                     (long long)ld, (long long)bs, elem_bytes);
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * elem_bytes, (cuuint64_t)(batch > 1 ? bs : rows * ld) * elem_bytes};
  cuuint32_t box[3] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                  const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return OK;
}

constexpr int kKernelSlots = 3 * 2 * 2 * 3 * 7;  // mode x CTAs per tile x epilogue warps x addend mode x variant
struct DeviceInfo {
  int sm_count = 0;
  int cc_major = 0;
  bool attr_set[kKernelSlots] = {};
  int max_clusters[kKernelSlots] = {};
};
DeviceInfo g_dev[64];
std::mutex g_dev_mu;

// 0 = pick per shape, 1 / 2 = force the one- or two-CTA kernel (environment variable
// MUON_B200_NS_CTAS, read once; meant for A/B measurements).
int forced_ctas() {
  static int v = [] {
    const char* e = std::getenv("MUON_B200_NS_CTAS");
    int x = e ? std::atoi(e) : 0;
    return (x == 1 || x == 2) ? x : 0;
  }();
  return v;
}

// Programmatic dependent launch of the GEMMs (MUON_B200_PDL=0 switches it off; read once; meant
// for A/B measurements).
}  // namespace
bool dependent_launch_enabled() {
  static bool v = [] {
    const char* e = std::getenv("MUON_B200_PDL");
    return !(e && (e[0] == '0' || e[0] == 'n' || e[0] == 'f'));
  }();
  return v;
}
namespace {

// SMs the persistent GEMM grids leave free, for kernels of other streams that must make
// progress while a GEMM runs (a collective's copy kernels in the distributed step).
std::atomic<int> g_reserved_sms{0};

// Epilogue warps forced by the environment variable MUON_B200_NS_EPI_WARPS (4 or 8; read
// once; meant for A/B measurements), 0 = pick per launch.
int forced_epi_warps() {
  static int v = [] {
    const char* e = std::getenv("MUON_B200_NS_EPI_WARPS");
    int x = e ? std::atoi(e) : 0;
    return (x == 4 || x == 8) ? x : 0;
  }();
  return v;
}

template <int MODE, bool B_MN, int CTAS, int EW, int ADD, int F8 = F8_NONE>
int launch_instance(int dev, int sms, const CUtensorMap& ta, const CUtensorMap& tb,
                    const GemmParams& p, cudaStream_t stream) {
  using C = Cfg<CTAS>;
  auto kern = ns_gemm_kernel<MODE, B_MN, CTAS, EW, ADD, F8>;
  const int slot = (((MODE * 2 + (CTAS - 1)) * 2 + (EW == 4 ? 0 : 1)) * 3 + ADD) * 7 + F8;
  const long long total = (long long)p.tiles_per_batch * p.batch * (p.split_phase == 1 ? p.split_k : 1);

  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(num_threads(EW));
  cfg.dynamicSmemBytes = C::smem_total(EW);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent_launch_enabled() ? 2 : 1;

  int max_units;  // co-resident CTAs (CTAS = 1) or clusters (CTAS = 2)
  {
    std::lock_guard<std::mutex> lk(g_dev_mu);
    if (!g_dev[dev].attr_set[slot]) {
      MB_CUDA_CHECK(
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::smem_total(EW)));
      if (CTAS == 2) {
        cfg.gridDim = dim3(sms / 2 * 2);
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
        if (e != cudaSuccess || n < 1) {
          (void)cudaGetLastError();
          n = sms / 2;
        }
        g_dev[dev].max_clusters[slot] = n;
      }
      g_dev[dev].attr_set[slot] = true;
    }
    max_units = CTAS == 2 ? g_dev[dev].max_clusters[slot] : sms;
  }
  const int reserved = g_reserved_sms.load(std::memory_order_relaxed);
  if (reserved > 0) {
    max_units -= (reserved + CTAS - 1) / CTAS;
    if (max_units < 1) max_units = 1;
  }
  const int units = (int)(total < max_units ? total : max_units);
  cfg.gridDim = dim3(units * CTAS);
  {
    const double m = p.M, n = p.N, k = p.K, b = p.batch;
    const double flops = MODE == MODE_BX ? 2.0 * m * k * n * b : m * (m + 1.0) * k * b;
    const int64_t tag = ((int64_t)p.M << 40) | ((int64_t)(MODE == MODE_BX ? p.N : p.K) << 16) | ((int64_t)(p.batch & 0xfff) << 4) |
                        (p.sym_add == ADD_SYMMETRIC ? 1 : 0) | (CTAS == 2 ? 2 : 0) |
                        (p.sym_add == ADD_ROW_SCALED ? 4 : 0) | (EW >= 8 ? 8 : 0);
    LaunchScope scope(MODE == MODE_SYRK ? K_NS_LINE1 : MODE == MODE_AXPBY ? K_NS_LINE2 : K_NS_LINE3,
                      flops, stream, tag);
    MB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, ta, tb, p));
  }
  MB_CUDA_CHECK(cudaGetLastError());
  return OK;
}

constexpr int kLongK = 2048;  // from this K on, four epilogue warps (see launch_ns_gemm)

template <int MODE, bool B_MN, int CTAS>
int launch_epi(int ew, int f8, int dev, int sms, const CUtensorMap& ta, const CUtensorMap& tb,
               const GemmParams& p, cudaStream_t stream) {
  if constexpr (MODE == MODE_BX) {
    // line 3 with the parameter update fused into its epilogue
    switch (f8) {
      case V_UPD_BF16:
        return ew == 4 ? launch_instance<MODE, B_MN, CTAS, 4, ADD_SYMMETRIC, V_UPD_BF16>(dev, sms, ta, tb, p, stream)
                       : launch_instance<MODE, B_MN, CTAS, 8, ADD_SYMMETRIC, V_UPD_BF16>(dev, sms, ta, tb, p, stream);
      case V_UPD_BF16_T:
        return ew == 4 ? launch_instance<MODE, B_MN, CTAS, 4, ADD_SYMMETRIC, V_UPD_BF16_T>(dev, sms, ta, tb, p, stream)
                       : launch_instance<MODE, B_MN, CTAS, 8, ADD_SYMMETRIC, V_UPD_BF16_T>(dev, sms, ta, tb, p, stream);
      case V_UPD_F32:
        return ew == 4 ? launch_instance<MODE, B_MN, CTAS, 4, ADD_SYMMETRIC, V_UPD_F32>(dev, sms, ta, tb, p, stream)
                       : launch_instance<MODE, B_MN, CTAS, 8, ADD_SYMMETRIC, V_UPD_F32>(dev, sms, ta, tb, p, stream);
      default: break;
    }
  }
  if (f8 == V_BATCH_SCALE) {
    if constexpr (MODE != MODE_AXPBY) {
      return ew == 4 ? launch_instance<MODE, B_MN, CTAS, 4, ADD_SYMMETRIC, V_BATCH_SCALE>(dev, sms, ta, tb, p, stream)
                     : launch_instance<MODE, B_MN, CTAS, 8, ADD_SYMMETRIC, V_BATCH_SCALE>(dev, sms, ta, tb, p, stream);
    } else {
      return set_error(ERR_INVALID_ARG, "line 2 has no per-matrix scale");
    }
  }
  if (f8 != F8_NONE) {
    // e4m3 variants exist for the symmetric-addend forms only (iterations after the first).
    constexpr int KIND = MODE == MODE_BX ? F8_EXTRA_OUT : F8_OPERANDS;
    if (ew == 4) return launch_instance<MODE, B_MN, CTAS, 4, ADD_SYMMETRIC, KIND>(dev, sms, ta, tb, p, stream);
    return launch_instance<MODE, B_MN, CTAS, 8, ADD_SYMMETRIC, KIND>(dev, sms, ta, tb, p, stream);
  }
  if constexpr (MODE == MODE_AXPBY) {
    if (p.sym_add == ADD_ROW_SCALED)
      return ew == 4 ? launch_instance<MODE, B_MN, CTAS, 4, ADD_ROW_SCALED>(dev, sms, ta, tb, p, stream)
                     : launch_instance<MODE, B_MN, CTAS, 8, ADD_ROW_SCALED>(dev, sms, ta, tb, p, stream);
    if (p.sym_add == ADD_GENERIC)
      return ew == 4 ? launch_instance<MODE, B_MN, CTAS, 4, ADD_GENERIC>(dev, sms, ta, tb, p, stream)
                     : launch_instance<MODE, B_MN, CTAS, 8, ADD_GENERIC>(dev, sms, ta, tb, p, stream);
    return ew == 4 ? launch_instance<MODE, B_MN, CTAS, 4, ADD_SYMMETRIC>(dev, sms, ta, tb, p, stream)
                   : launch_instance<MODE, B_MN, CTAS, 8, ADD_SYMMETRIC>(dev, sms, ta, tb, p, stream);
  } else {
    if (ew == 4) return launch_instance<MODE, B_MN, CTAS, 4, ADD_SYMMETRIC>(dev, sms, ta, tb, p, stream);
    return launch_instance<MODE, B_MN, CTAS, 8, ADD_SYMMETRIC>(dev, sms, ta, tb, p, stream);
  }
}

}  // namespace

namespace {
// Lower-triangle tile count of an m x m product and the tile geometry launch_ns_gemm picks.
int tri_tile_count(int64_t m, int* ctas_out) {
  int ctas = forced_ctas();
  if (ctas == 0) ctas = m > BM ? 2 : 1;
  const int tile_m = BM * ctas;
  const int tiles_m = (int)((m + tile_m - 1) / tile_m), tiles_n = (int)((m + BN - 1) / BN);
  int cnt = 0;
  for (int i = 0; i < tiles_m; ++i) cnt += tri_row_count(i, tiles_n, tile_m);
  if (ctas_out) *ctas_out = ctas;
  return cnt;
}
constexpr int kSplitSms = 148;       // SMs of the GPU the split is sized for (a B200)
constexpr int kSplitMinSlices = 3;   // below that a split does not pay for its second launch
constexpr int kSplitMaxSlices = 16;
constexpr int kSplitMinBlocks = 4;   // k-blocks (of 64) per slice at least
}  // namespace

int splitk_slices(int batch, int64_t m, int64_t k) {
  static const bool off = [] {
    const char* e = std::getenv("MUON_B200_SPLITK");
    return e && (e[0] == '0' || e[0] == 'n' || e[0] == 'f');
  }();
  if (off || batch < 1 || m < 1 || k < 1) return 1;
  int ctas = 1;
  const long long tiles = (long long)tri_tile_count(m, &ctas) * batch;
  const int units = kSplitSms / ctas;
  const int k_blocks = (int)((k + BK - 1) / BK);
  long long want = units / tiles;
  if (want > k_blocks / kSplitMinBlocks) want = k_blocks / kSplitMinBlocks;
  if (want > kSplitMaxSlices) want = kSplitMaxSlices;
  if (want < kSplitMinSlices) return 1;
  const int per = (k_blocks + (int)want - 1) / (int)want;
  return (k_blocks + per - 1) / per;  // every slice has at least one k-block
}

int64_t splitk_scratch_bytes(int batch, int64_t m, int64_t k) {
  const int s = splitk_slices(batch, m, k);
  if (s <= 1) return 0;
  int ctas = 1;
  const long long tiles = (long long)tri_tile_count(m, &ctas) * batch;
  return tiles * s * ctas * (int64_t)(BM * BN * 4);
}

bool update_fusable(const UpdateSpec& u, int batch) {
  if (!u.param || batch < 1 || batch > kMaxUpdateTensors || u.rows < 1 || u.cols < 1) return false;
  const bool tall = u.rows > u.cols;
  if (u.dtype == DT_F32) {
    if (tall || u.cols % 4 != 0) return false;  // tall fp32 parameters: left to the epilogue kernel
  } else if (u.dtype == DT_BF16) {
    if (u.cols % 8 != 0) return false;          // rows of the parameter must be 16-byte multiples
  } else {
    return false;
  }
  for (int b = 0; b < batch; ++b)
    if (!u.param[b] || (reinterpret_cast<uintptr_t>(u.param[b]) & 15)) return false;
  return true;
}

void set_reserved_sms(int n) { g_reserved_sms.store(n < 0 ? 0 : n); }
int get_reserved_sms() { return g_reserved_sms.load(); }

int device_sm_count(int* sm_count_out) {
  int dev = 0;
  MB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(ERR_UNSUPPORTED, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_dev_mu);
  if (g_dev[dev].sm_count == 0) {
    int major = 0, sms = 0;
    MB_CUDA_CHECK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    MB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    g_dev[dev].cc_major = major;
    g_dev[dev].sm_count = sms;
  }
  if (g_dev[dev].cc_major != 10)
    return set_error(ERR_UNSUPPORTED, "muon_b200 kernels need an sm_100 device (found sm_%d0)",
                     g_dev[dev].cc_major);
  *sm_count_out = g_dev[dev].sm_count;
  return OK;
}

// out[batch, M, N] = epilogue( opA[batch, M, K] · opB ), see GemmMode.
//   MODE_SYRK / MODE_AXPBY: opB = opA (K contiguous), N = M, triangular schedule + mirror.
//   MODE_BX: opA = Bmat [M, M], opB = X [M(K), N] with N contiguous, add = X.
int launch_ns_gemm(int mode, const __nv_bfloat16* opa, int64_t lda, int64_t a_bs,
                   const __nv_bfloat16* opb, int64_t ldb, int64_t b_bs, __nv_bfloat16* out,
                   int64_t ldo, int64_t out_bs, int batch, int64_t M, int64_t N, int64_t K,
                   float alpha, float beta, int sym_add, cudaStream_t stream, const __nv_bfloat16* addend,
                   const float* row_scale, int64_t scale_bs, const Fp8Spec* f8, const UpdateSpec* upd,
                   const float* batch_scale, const SplitK* split) {
  if (!opa || !opb || !out) return set_error(ERR_INVALID_ARG, "null pointer passed to NS GEMM");
  if (batch < 1 || M < 1 || N < 1 || K < 1)
    return set_error(ERR_INVALID_ARG, "NS GEMM needs batch, M, N, K >= 1 (got %d, %lld, %lld, %lld)",
                     batch, (long long)M, (long long)N, (long long)K);
  if (M > (1 << 24) || N > (1 << 24) || K > (1 << 24))
    return set_error(ERR_UNSUPPORTED, "NS GEMM dimension beyond 2^24");
  if ((reinterpret_cast<uintptr_t>(out) & 15) != 0 || (ldo % 8) != 0 || (out_bs % 8) != 0)
    return set_error(ERR_ALIGNMENT, "NS GEMM output must be 16-byte aligned with pitch %% 8 == 0");
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != OK) return rc;
  int dev = 0;
  MB_CUDA_CHECK(cudaGetDevice(&dev));

  // A pair wastes half its rows on a matrix of at most 128 rows: those stay on one CTA.
  int ctas = forced_ctas();
  if (ctas == 0) ctas = M > BM ? 2 : 1;
  const int tile_m = BM * ctas;
  const int b_rows = BN / ctas;

  GemmParams p{};
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.batch = batch;
  p.tiles_m = (int)((M + tile_m - 1) / tile_m);
  p.tiles_n = (int)((N + BN - 1) / BN);
  p.alpha = alpha;
  p.beta = beta;
  p.out = out;
  p.ldo = ldo;
  p.out_bs = out_bs;
  int f8_kind = f8 ? f8->kind : F8_NONE;
  p.acc_scale = 1.f;
  if (upd) {
    if (mode != MODE_BX || f8_kind != F8_NONE || !update_fusable(*upd, batch))
      return set_error(ERR_INVALID_ARG, "this parameter update cannot be fused into the launch");
    const bool tall = upd->rows > upd->cols;
    if ((tall ? upd->cols : upd->rows) != M || (tall ? upd->rows : upd->cols) != N)
      return set_error(ERR_INVALID_ARG, "fused update: parameter shape does not match the product");
    for (int b = 0; b < batch; ++b) p.upd_param[b] = upd->param[b];
    p.upd_scale = upd->scale;
    p.upd_decay = upd->decay;
    p.upd_neg_lr = upd->neg_lr;
    f8_kind = upd->dtype == DT_F32 ? V_UPD_F32 : (tall ? V_UPD_BF16_T : V_UPD_BF16);
  }
  if (batch_scale) {
    if (f8_kind != F8_NONE || mode == MODE_AXPBY)
      return set_error(ERR_INVALID_ARG, "a per-matrix scale goes with plain bf16 lines 1 and 3 only");
    p.batch_scale = batch_scale;
    f8_kind = V_BATCH_SCALE;
  }
  if (f8 && f8->kind != F8_NONE) {
    if ((f8_kind == F8_OPERANDS) != (mode != MODE_BX))
      return set_error(ERR_INVALID_ARG, "e4m3 operands go with lines 1 and 2, the extra e4m3 output with line 3");
    if (f8_kind == F8_OPERANDS && (!f8->op8 || sym_add != ADD_SYMMETRIC))
      return set_error(ERR_INVALID_ARG, "e4m3 products need the e4m3 operand and a symmetric addend");
    if (f8->out8 && ((reinterpret_cast<uintptr_t>(f8->out8) & 15) || (f8->ldo8 % 16) || (f8->out8_bs % 16) ||
                     f8->ldo8 < N))
      return set_error(ERR_ALIGNMENT, "e4m3 output must be 16-byte aligned with pitches %% 16 == 0 and >= N");
    p.out8 = f8->out8;
    p.ldo8 = f8->ldo8;
    p.out8_bs = f8->out8_bs;
    p.out8_scale = f8->out8_scale;
    p.acc_scale = f8->acc_scale;
    p.diag = f8->diag;
  }

  CUtensorMap ta, tb;
  if (mode == MODE_SYRK || mode == MODE_AXPBY) {
    if (M != N) return set_error(ERR_INVALID_ARG, "symmetric product needs a square output");
    p.triangular = 1;
    int cnt = 0;
    for (int i = 0; i < p.tiles_m; ++i) cnt += tri_row_count(i, p.tiles_n, tile_m);
    p.tiles_per_batch = cnt;
    p.sym_add = sym_add;
    // Line 2 adds beta * A. Normally A is the operand itself; in row-scaled mode the operand is
    // the materialised S / s while the addend is rebuilt from the unscaled S and s.
    p.add = (sym_add == ADD_ROW_SCALED) ? addend : opa;
    p.ldadd = lda;
    p.add_bs = a_bs;
    p.row_scale = row_scale;
    p.scale_bs = scale_bs;
    if (sym_add == ADD_ROW_SCALED && (!addend || !row_scale))
      return set_error(ERR_INVALID_ARG, "row-scaled line 2 needs the unscaled matrix and the scale vector");
    if (mode == MODE_AXPBY && K != M)
      return set_error(ERR_INVALID_ARG, "line 2 needs a square operand (got %lld x %lld)",
                       (long long)M, (long long)K);
    if (f8_kind == F8_OPERANDS) {
      // Both operands are the e4m3 matrix; the bf16 one (opa) is only line 2's addend.
      if ((rc = encode_map(&ta, f8->op8, M, K, f8->ld8, f8->bs8, batch, BM, 1)) != OK) return rc;
      if ((rc = encode_map(&tb, f8->op8, M, K, f8->ld8, f8->bs8, batch, b_rows, 1)) != OK) return rc;
    } else {
      if ((rc = encode_map(&ta, opa, M, K, lda, a_bs, batch, BM)) != OK) return rc;
      if ((rc = encode_map(&tb, opb, M, K, ldb, b_bs, batch, b_rows)) != OK) return rc;
    }
  } else if (mode == MODE_BX) {
    if (K != M) return set_error(ERR_INVALID_ARG, "line 3 needs a square left operand");
    p.triangular = 0;
    p.tiles_per_batch = p.tiles_m * p.tiles_n;
    p.add = opb;  // a * X
    p.ldadd = ldb;
    p.add_bs = b_bs;
    if ((rc = encode_map(&ta, opa, M, K, lda, a_bs, batch, BM)) != OK) return rc;
    if ((rc = encode_map(&tb, opb, K, N, ldb, b_bs, batch, BK)) != OK) return rc;
  } else {
    return set_error(ERR_INVALID_ARG, "unknown NS GEMM mode %d", mode);
  }
  if ((reinterpret_cast<uintptr_t>(p.add) & 15) != 0 || (p.ldadd % 8) != 0)
    return set_error(ERR_ALIGNMENT, "NS GEMM addend must be 16-byte aligned with pitch %% 8 == 0");
  if ((long long)p.tiles_per_batch * batch > (1ll << 30))
    return set_error(ERR_UNSUPPORTED, "too many output tiles");

  int ew = forced_epi_warps();
  // With a long K the MMAs of the next tile hide the epilogue even with four warps, and the
  // smaller CTA leaves room on the SM (registers, 8 KiB of shared memory) for the HBM-bound
  // kernels that the engine runs beside the GEMMs. With a short K the epilogue is what a tile
  // waits for: eight warps.
  // (with e4m3 operands a tile's main loop takes half as long: the threshold doubles)
  if (ew == 0) ew = K >= (f8_kind == F8_OPERANDS ? 2 * kLongK : kLongK) ? 4 : 8;
  if (split && split->partial && mode == MODE_SYRK && f8_kind == F8_NONE) {
    const int slices = splitk_slices(batch, M, K);
    if (slices > 1 && split->bytes >= splitk_scratch_bytes(batch, M, K) &&
        (reinterpret_cast<uintptr_t>(split->partial) & 15) == 0) {
      const int k_blocks = (int)((K + BK - 1) / BK);
      p.split_k = slices;
      p.split_kb = (k_blocks + slices - 1) / slices;
      p.partial = split->partial;
      p.split_phase = 1;  // slices -> partial sums; a slice is short: eight epilogue warps
      rc = ctas == 2 ? launch_epi<MODE_SYRK, false, 2>(8, f8_kind, dev, sms, ta, tb, p, stream)
                     : launch_epi<MODE_SYRK, false, 1>(8, f8_kind, dev, sms, ta, tb, p, stream);
      if (rc != OK) return rc;
      // partial sums -> bf16 pieces and their mirror images, one warp per 32 rows x 8 columns
      const long long warps = (long long)p.tiles_per_batch * batch * ctas * 4 * (BN / 32) * 4;
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)((warps + 7) / 8));
      cfg.blockDim = dim3(256);
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = dependent_launch_enabled() ? 1 : 0;
      LaunchScope scope(K_NS_LINE1, 0.0, stream);
      if (ctas == 2) MB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, splitk_reduce_kernel<2>, p));
      else MB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, splitk_reduce_kernel<1>, p));
      MB_CUDA_CHECK(cudaGetLastError());
      return OK;
    }
  }
  if (ctas == 2) {
    switch (mode) {
      case MODE_SYRK: return launch_epi<MODE_SYRK, false, 2>(ew, f8_kind, dev, sms, ta, tb, p, stream);
      case MODE_AXPBY: return launch_epi<MODE_AXPBY, false, 2>(ew, f8_kind, dev, sms, ta, tb, p, stream);
      default: return launch_epi<MODE_BX, true, 2>(ew, f8_kind, dev, sms, ta, tb, p, stream);
    }
  }
  switch (mode) {
    case MODE_SYRK: return launch_epi<MODE_SYRK, false, 1>(ew, f8_kind, dev, sms, ta, tb, p, stream);
    case MODE_AXPBY: return launch_epi<MODE_AXPBY, false, 1>(ew, f8_kind, dev, sms, ta, tb, p, stream);
    default: return launch_epi<MODE_BX, true, 1>(ew, f8_kind, dev, sms, ta, tb, p, stream);
  }
}

}  // namespace mb
