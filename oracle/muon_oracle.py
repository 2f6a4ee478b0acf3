"""CPU oracle for the Muon optimizer step.  TEST INFRASTRUCTURE ONLY.

This module restates, with plain torch CPU ops, the algorithm of thib-s/Muon's
``muon.py`` for the one path this repository accelerates.  Only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import
it; the product (``muon_b200``) never does and has no CPU fallback.

Pinning status
--------------
The reference ships no tests, golden vectors or fixtures, and its Newton-Schulz
kernels are Triton kernels that need a GPU.  What pins this restatement:

* ``adam_update``, ``muon_update``'s momentum/scale arithmetic and all optimizer-class
  host logic are checked against the *real* reference code imported on CPU
  (``tests/golden/make_golden.py``), bit for bit;
* the three GEMM lines are checked against the *real* reference Triton kernels run
  under Triton's CPU interpreter in fp32 (the interpreter cannot run them in bf16);
* the bf16 Newton-Schulz driver is checked against the *real* reference driver
  (``zeropower_via_newtonschulz5``, run uncompiled on CPU) calling its real Triton kernels
  under the interpreter, with the bf16 operands of every kernel call handed over as fp32 and
  the fp32 result rounded to bf16 once: bit for bit on single-tile cases, call by call (12
  kernel calls, at most one bf16 step apart on <0.1% of the elements, where fp32 sums taken
  in another order round the other way) on a multi-tile case, with ``glue="eager"`` and
  ``mirror="ref_square_tiles"``.  The defaults of this module (``glue="fused"``,
  ``mirror="product"``: what the CUDA kernels implement) differ from that run by the two
  documented choices; at 768x768 / 768x3072 by 8.0e-3 / 6.6e-3 relative Frobenius norm,
  while the reference itself moves by 5.1e-3 / 4.1e-3 between 64- and 128-wide tiles.
  What no CPU run can pin is the reference as a GPU executes it: compiled glue, autotuned
  tile shapes and two racing stores on diagonal tiles;
* ``muon_param_step`` end to end: three steps of the real ``SingleDeviceMuon`` with the real
  Newton-Schulz driver and kernels (executed as above) on one fp32 768x3072 parameter; the
  defaults of this module give the same parameters to 2e-4 relative;
* the distributed class against the real ``Muon`` run on two gloo CPU ranks.

Every function cites the reference lines (``muon.py:<line>``) it follows.
"""
from __future__ import annotations

import torch
from torch import Tensor

# muon.py:754-759 — (a, b, c) per iteration of the live (AOL) algorithm.
AOL4_COEFFS = (
    (4.0098, -7.0585, 2.4635),
    (3.4585, -5.5479, 2.5959),
    (2.7573, -3.2939, 1.4254),
    (2.7215, -3.0494, 1.3169),
)
# muon.py:276 — the classic quintic iteration's fixed coefficients.
CLASSIC_COEFFS = (3.4445, -4.7750, 2.0315)


# --------------------------------------------------------------------------------------
# GEMM lines.  Inputs of any float dtype; arithmetic in fp32 ("tl.dot" accumulates in
# fp32, muon.py:394/:510/:681-686); one rounding to the input dtype at the end
# (muon.py:404-405, :531-532, :696-697).
# --------------------------------------------------------------------------------------
def _mirror(P: Tensor, policy: str, tile: int) -> Tensor:
    """Resolve which of P[i,j] / P[j,i] an output element takes.

    ``lower``: element (i,j) with i >= j is authoritative and mirrored — the rule the
    CUDA kernels implement.  ``ref_square_tiles``: what the reference's kernels leave
    when run with square ``tile`` x ``tile`` blocks and stores applied in program order
    (muon.py:378-381 skips tiles strictly above the diagonal; :408-417 stores each
    computed tile, then its transpose): off-diagonal tiles are lower-authoritative,
    diagonal tiles end up holding their own transpose.
    """
    low = torch.tril(P)
    out = low + torch.tril(P, -1).mT
    if policy == "lower":
        return out
    if policy == "ref_square_tiles":
        M = P.shape[-1]
        for s in range(0, M, tile):
            e = min(s + tile, M)
            out[..., s:e, s:e] = P[..., s:e, s:e].mT
        return out
    if policy == "none":
        return P
    raise ValueError(f"unknown mirror policy {policy!r}")


def ns_line_1(X: Tensor, *, mirror: str = "lower", tile: int = 64) -> Tensor:
    """A = X · Xᵀ (muon.py:349-417)."""
    Xf = X.float()
    P = Xf @ Xf.mT
    return _mirror(P, mirror, tile).to(X.dtype)


def ns_line_2(A: Tensor, alpha: float, beta: float, *, mirror: str = "ref_square_tiles", tile: int = 64) -> Tensor:
    """B = alpha · A · Aᵀ + beta · A (muon.py:464-544).  Note Aᵀ: the kernel reads its
    second operand through swapped strides (muon.py:507-508).

    ``mirror="ref_square_tiles"`` with 64-wide tiles (default, and the rule of the CUDA
    kernel): what the reference's two stores per tile (muon.py:534-544) leave with the
    64 x 64 tiles its autotuner picks on a B200 for every m <= 1024 — finished values,
    addend included, mirrored from below the diagonal; diagonal tiles hold their own
    transpose.  Measured on a B200 (``tests/golden/make_reference_b200.py`` records the
    pattern the reference leaves for a non-symmetric input).  ``mirror="product"`` mirrors
    only the product A·Aᵀ and takes the addend beta·A at each position, i.e. the documented
    formula (muon.py:483-486) evaluated for any A.  The policies differ only when A is not
    symmetric (first iteration, muon.py:785).
    """
    Af = A.float()
    if mirror == "product":
        P = _mirror(Af @ Af.mT, "lower", tile) * alpha + Af * beta
        return P.to(A.dtype)
    P = (Af @ Af.mT) * alpha + Af * beta  # muon.py:528-529
    return _mirror(P, mirror, tile).to(A.dtype)


def ns_line_3(B: Tensor, X: Tensor, a: float) -> Tensor:
    """C = a · X + B · X (muon.py:639-702); a·X is formed in fp32 (muon.py:681-686)."""
    Xf = X.float()
    return (Xf * a + B.float() @ Xf).to(X.dtype)


# --------------------------------------------------------------------------------------
# Newton-Schulz drivers
# --------------------------------------------------------------------------------------
def zeropower_via_newtonschulz5(G: Tensor, epsilon: float = 1e-7, *, mirror: str = "ref_square_tiles",
                                dtype: torch.dtype = torch.bfloat16, glue: str = "fused") -> Tensor:
    """The live algorithm, muon.py:748-799: AOL rescale + 4 iterations.

    Rounding points (each ``.to(dtype)``): the cast (:760), every GEMM line's output,
    X·rsqrt(s) (:782), A/s (:785) and, depending on ``glue``, the row sums s (:779-781):

    * ``glue="compiled"``: the graph torch.compile generates for the reference on a B200 (read from
      its generated code): one reduction kernel sums |A| per row in fp32, divides A by the
      unrounded clamped sum and stores the sum as bf16; one pointwise kernel multiplies the
      *uncast* input G (fp32 when the caller passes fp32) by rsqrt(max(stored sum, eps)).  With the
      default mirror rule this is within accumulation-order noise (about 3e-3) of the reference's
      output on a B200 (``tests/golden/reference_b200.pt``).
    * ``glue="fused"`` (default, what the CUDA kernels implement): the same, except that X·rsqrt(s)
      starts from the bf16 cast of G, like every uncompiled run of the reference does; the only
      copy of G the kernels keep is the bf16 one.  A/s is formed as A·(1/s) with a correctly
      rounded reciprocal (the CUDA kernels rebuild it bit for bit in two places).
    * ``glue="eager"`` rounds after every torch op (abs, sum, clamp, rsqrt, multiply, divide),
      which is what the reference does when it runs uncompiled; with
      ``mirror="ref_square_tiles"`` that variant reproduces the real reference driver executed on
      CPU (its Triton kernels under the interpreter) bit for bit.
    """
    assert G.ndim in (2, 3)
    assert glue in ("fused", "eager", "compiled")
    X = G.to(dtype)
    tall = G.size(-2) > G.size(-1)
    if tall:
        X = X.mT  # :761-762
    X = X.contiguous()
    m1 = "lower" if mirror == "product" else mirror  # line 1's output is symmetric either way
    A = ns_line_1(X, mirror=m1)  # :778
    if glue == "eager":
        s = torch.clamp_min(A.abs().sum(dim=-1, keepdim=True), epsilon)  # :779-781, every op in dtype
        X = X * torch.rsqrt(s)  # :782
        A = A / s  # :785
    else:
        s32 = A.float().abs().sum(dim=-1, keepdim=True)  # :779-780, kept in fp32 by the reduction kernel
        s_stored = torch.clamp_min(s32.to(dtype).float(), epsilon)  # what the pointwise kernel reads back
        if glue == "compiled":
            src = (G.mT if tall else G).float()  # the cast of :760 is fused away: G itself is read
            X = (src * torch.rsqrt(s_stored)).to(dtype)  # :782
            A = (A.float() / torch.clamp_min(s32, epsilon)).to(dtype)  # :785 (rows only)
        else:
            X = (X.float() * torch.rsqrt(s_stored)).to(dtype)  # :782
            A = (A.float() * (1.0 / torch.clamp_min(s32, epsilon))).to(dtype)  # :785 (rows only)
    for k, (a, b, c) in enumerate(AOL4_COEFFS):
        if k > 0:
            A = ns_line_1(X, mirror=m1)  # :792
        B = ns_line_2(A, alpha=c, beta=b, mirror=mirror)  # :786 / :793
        X = ns_line_3(B, X, a)  # :787 / :794
    if tall:
        X = X.mT  # :797-798
    return X


def _e4m3(T: Tensor, scale: float) -> Tensor:
    """fp32 values of e4m3(T * scale) / scale: round to nearest even, saturating at +-448."""
    return (T.float() * scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float() / scale


def zeropower_aol4_fp8(G: Tensor, epsilon: float = 1e-7) -> Tensor:
    """Restatement of the library's ``aol4_fp8`` variant (no counterpart in the reference): the
    live algorithm (muon.py:748-799) with the two symmetric products of iterations 2..4 taken on
    e4m3 operands with power-of-two scales and fp32 accumulation.  Line 1 multiplies
    e4m3(X * sx); line 2, rewritten as c·E·E + (b + 2c)·A − c·I with E = A − I, multiplies
    e4m3(E * 64).  The first iteration and every line 3 are those of ``zeropower_via_newtonschulz5``."""
    assert G.ndim in (2, 3)
    if max(G.size(-2), G.size(-1)) < 1024:  # the library iterates narrow matrices in bf16 in this mode too
        return zeropower_via_newtonschulz5(G, epsilon)
    dtype = torch.bfloat16
    X = G.to(dtype)
    tall = G.size(-2) > G.size(-1)
    if tall:
        X = X.mT
    X = X.contiguous()
    m, n = X.shape[-2], X.shape[-1]
    sx = 1.0
    while sx < 256.0 and sx * sx * 2.0 <= n:
        sx *= 2.0
    se = 64.0
    eye = torch.eye(m)
    A = ns_line_1(X, mirror="ref_square_tiles")
    s32 = A.float().abs().sum(dim=-1, keepdim=True)
    s_stored = torch.clamp_min(s32.to(dtype).float(), epsilon)
    X = (X.float() * torch.rsqrt(s_stored)).to(dtype)
    A = (A.float() * (1.0 / torch.clamp_min(s32, epsilon))).to(dtype)
    for k, (a, b, c) in enumerate(AOL4_COEFFS):
        if k == 0:
            B = ns_line_2(A, alpha=c, beta=b)
        else:
            X8 = _e4m3(X, sx)
            A = _mirror(X8 @ X8.mT, "lower", 64).to(dtype)
            E8 = _e4m3(A.float() - eye, se)
            B = (_mirror(E8 @ E8.mT, "lower", 64) * c + A.float() * (b + 2.0 * c) - c * eye).to(dtype)
        X = ns_line_3(B, X, a)
    if tall:
        X = X.mT
    return X


def zeropower_classic5(G: Tensor, steps: int = 5, *, fused: bool = False, folded: bool = False) -> Tensor:
    """The commented reference block, muon.py:265-291 (Frobenius normalisation, fixed
    coefficients).  ``fused=False`` executes it literally with eager bf16 tensors (every
    op rounds); ``fused=True`` rounds once per GEMM line like the kernels do.

    ``folded=True`` (implies the single rounding per line) is the arithmetic of the CUDA path:
    X is not divided by its norm in memory; with c = 1 / bf16(bf16(||X||) + 1e-7) in fp32 the
    first Gram product is rounded once from c^2 · (X · Xᵀ) and the first line 3 once from
    c · (a · X + B · X).  It differs from ``fused=True`` only by the rounding of X / (||X|| + eps)
    to bf16 that it leaves out."""
    assert G.ndim >= 2
    a, b, c = CLASSIC_COEFFS
    X = G.bfloat16()
    if G.size(-2) > G.size(-1):
        X = X.mT
    if folded:
        den = (X.norm(dim=(-2, -1), keepdim=True) + 1e-7).float()  # bf16 norm, bf16 sum (eager)
        inv = 1.0 / den
        for k in range(steps):
            if k == 0:
                Xf = X.float()
                A = _mirror((Xf @ Xf.mT) * (inv * inv), "lower", 64).to(X.dtype)
                B = ns_line_2(A, alpha=c, beta=b)
                X = ((Xf * a + B.float() @ Xf) * inv).to(X.dtype)
            else:
                A = ns_line_1(X)
                B = ns_line_2(A, alpha=c, beta=b)
                X = ns_line_3(B, X, a)
        if G.size(-2) > G.size(-1):
            X = X.mT
        return X
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        if fused:
            A = ns_line_1(X)
            B = ns_line_2(A, alpha=c, beta=b)
            X = ns_line_3(B, X, a)
        else:
            A = X @ X.mT
            B = b * A + c * A @ A
            X = a * X + B @ X
    if G.size(-2) > G.size(-1):
        X = X.mT
    return X


# --------------------------------------------------------------------------------------
# Functional updates
# --------------------------------------------------------------------------------------
def muon_update(grad: Tensor, momentum: Tensor, beta: float = 0.95, nesterov: bool = True,
                ns=zeropower_via_newtonschulz5) -> Tensor:
    """muon.py:8-15.  In place on ``momentum`` and (with Nesterov) on ``grad``."""
    momentum.lerp_(grad, 1 - beta)  # :9
    update = grad.lerp_(momentum, beta) if nesterov else momentum  # :10
    if update.ndim == 4:
        update = update.view(len(update), -1)  # :11-12
    update = ns(update)  # :13
    update = update * max(1, grad.size(-2) / grad.size(-1)) ** 0.5  # :14 (out of place: ns may alias)
    return update


def adam_update(grad: Tensor, buf1: Tensor, buf2: Tensor, step: int, betas, eps: float) -> Tensor:
    """muon.py:104-109."""
    buf1.lerp_(grad, 1 - betas[0])
    buf2.lerp_(grad.square(), 1 - betas[1])
    buf1c = buf1 / (1 - betas[0] ** step)
    buf2c = buf2 / (1 - betas[1] ** step)
    return buf1c / (buf2c.sqrt() + eps)


def muon_param_step(p: Tensor, grad: Tensor, momentum: Tensor, lr: float, weight_decay: float,
                    beta: float, ns=zeropower_via_newtonschulz5) -> None:
    """One parameter's update inside ``*.step`` (muon.py:65-67 / :97-99)."""
    update = muon_update(grad, momentum, beta=beta, ns=ns)
    p.mul_(1 - lr * weight_decay)
    p.add_(update.reshape(p.shape), alpha=-lr)


def adam_param_step(p: Tensor, grad: Tensor, exp_avg: Tensor, exp_avg_sq: Tensor, step: int,
                    lr: float, weight_decay: float, betas, eps: float) -> None:
    """One parameter's Adam update inside ``*.step`` (muon.py:194-197)."""
    update = adam_update(grad, exp_avg, exp_avg_sq, step, betas, eps)
    p.mul_(1 - lr * weight_decay)
    p.add_(update, alpha=-lr)


# --------------------------------------------------------------------------------------
# Ownership rule of the distributed optimizer
# --------------------------------------------------------------------------------------
def sorted_param_order(shapes) -> list[int]:
    """Indices that sort shapes descending, lexicographically on the size tuple, stable
    (muon.py:42 / :143: ``sorted(params, key=lambda x: x.size(), reverse=True)``)."""
    return [i for i, _ in sorted(enumerate(shapes), key=lambda t: tuple(t[1]), reverse=True)]


def owner_of(sorted_index: int, world_size: int) -> int:
    """Rank that updates the parameter at ``sorted_index`` (muon.py:56-58)."""
    return sorted_index % world_size


def padded_length(n_params: int, world_size: int) -> int:
    """Length of ``params_pad`` (muon.py:55): always adds ``W - n % W`` entries."""
    return n_params + (world_size - n_params % world_size)


# --------------------------------------------------------------------------------------
# Tolerance helpers shared by the tests
# --------------------------------------------------------------------------------------
def rel_fro(x: Tensor, ref: Tensor) -> float:
    x, ref = x.double(), ref.double()
    return float((x - ref).norm() / ref.norm().clamp_min(1e-30))


def singular_value_band(U: Tensor) -> tuple[float, float]:
    s = torch.linalg.svdvals(U.float())
    return float(s.min()), float(s.max())
