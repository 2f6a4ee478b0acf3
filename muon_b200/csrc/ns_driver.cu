// Launch sequence of one Newton-Schulz orthogonalisation (reference
// zeropower_via_newtonschulz5, muon.py:778-795, and the classic iteration of its commented
// block, muon.py:282-289).
#include "../../include/muon_b200.h"

#include "common.cuh"
#include "elementwise.h"
#include "ns_driver.h"
#include "ns_gemm.h"

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

}  // namespace mb
