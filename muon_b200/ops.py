"""Functional API with the reference's names and signatures (muon.py:8, :104, :420, :547,
:705, :749), executed by the sm_100a library."""
from __future__ import annotations

import ctypes

import torch
from torch import Tensor

from . import _lib
from ._lib import check, lib
from .engine import (_NS_MODES, _require_cuda, _stream_ptr, aspect_scale, dtype_code, get_backend,
                     get_ns_mode, view_2d)


def _as_bf16_3d(t: Tensor, name: str) -> tuple[Tensor, int]:
    """Contiguous bf16 [batch, r, c] alias (or copy) of a 2-D/3-D tensor."""
    if t.ndim > 3 or t.ndim < 2:
        raise ValueError(f"Input tensor must be 2D or 3D, but got {t.ndim}D tensor.")
    _require_cuda(t, name)
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bfloat16 (the tensor-core path is bf16 only), got {t.dtype}")
    batch = t.shape[0] if t.ndim == 3 else 1
    t3 = t.reshape(batch, t.shape[-2], t.shape[-1])
    ok = t3.stride(-1) == 1 and t3.stride(-2) % 8 == 0 and t3.data_ptr() % 16 == 0 and \
        (batch == 1 or t3.stride(0) % 8 == 0)
    if not ok:
        r, c = t3.shape[-2:]
        ld = (c + 7) // 8 * 8
        buf = torch.empty(batch, r, ld, dtype=torch.bfloat16, device=t.device)
        buf[:, :, :c].copy_(t3)
        t3 = buf[:, :, :c]
    return t3, batch


def _out_3d(out: Tensor | None, like: Tensor, shape: tuple[int, ...]) -> tuple[Tensor, Tensor | None]:
    """(kernel output buffer, user tensor to copy back into or None)."""
    batch, r, c = shape
    if out is not None and out.dtype == torch.bfloat16 and out.is_contiguous() and c % 8 == 0 \
            and out.data_ptr() % 16 == 0 and out.numel() == batch * r * c:
        return out.view(batch, r, c), None  # the kernel can write the user's tensor directly
    ld = (c + 7) // 8 * 8
    buf = torch.empty(batch, r, ld, dtype=torch.bfloat16, device=like.device)[:, :, :c]
    return buf, out


def ns_line_1(A: Tensor, *, out: Tensor = None) -> Tensor:
    """C = A @ A.T for bf16 A of shape [M, K] or [B, M, K] (muon.py:420-456)."""
    A3, batch = _as_bf16_3d(A, "A")
    M, K = A3.shape[-2:]
    if out is not None:
        assert out.size(-2) == M, "Output matrix has incorrect shape"
        assert out.size(-1) == M, "Output matrix has incorrect shape"
    buf, user = _out_3d(out, A, (batch, M, M))
    with torch.cuda.device(A.device):
        # a product with few output tiles and a long K is split along K: room for its partial sums
        need = lib.muon_b200_ns_line1_scratch_bytes(batch, M, K)
        backend = get_backend()
        scratch = backend._aligned_ptr(backend.workspace(A.device, need, slot=4)) if need > 0 else None
        check(lib.muon_b200_ns_line1_scratch(A3.data_ptr(), A3.stride(-2), A3.stride(0), buf.data_ptr(),
                                             buf.stride(-2), buf.stride(0), batch, M, K, scratch, need,
                                             _stream_ptr(A.device)))
    return _finish(buf, user, A.ndim, (M, M))


def ns_line_2(A: Tensor, alpha: float, beta: float, *, out: Tensor = None, symmetric: bool = False) -> Tensor:
    """C = alpha * A @ A.T + beta * A for square bf16 A (muon.py:547-588). ``symmetric=True``
    (not in the reference's signature) promises that A equals its transpose bit for bit, as the
    output of ``ns_line_1`` does: the kernel then mirrors finished values instead of reading
    A[col, row] for the mirrored element (same result for such an A, less traffic)."""
    if A.ndim > 3 or A.ndim < 2:
        raise ValueError(f"Input tensor must be 2D or 3D, but got {A.ndim}D tensor.")
    M, K = A.shape[-2:]
    if M != K:
        raise ValueError(f"Input must be symmetric square matrix, but got shape {A.shape}")
    A3, batch = _as_bf16_3d(A, "A")
    if out is not None:
        assert out.size(-2) == M, "Output matrix has incorrect shape"
        assert out.size(-1) == M, "Output matrix has incorrect shape"
    buf, user = _out_3d(out, A, (batch, M, M))
    if buf.data_ptr() == A3.data_ptr():
        buf, user = _out_3d(None, A, (batch, M, M))[0], out
    with torch.cuda.device(A.device):
        # The reference's kernel takes any square A (muon.py:483-486); unless the caller says that
        # this one is symmetric bit for bit, the general addend path is used (for such an A it
        # gives the same result as the symmetric one).
        check(lib.muon_b200_ns_line2(A3.data_ptr(), A3.stride(-2), A3.stride(0), buf.data_ptr(),
                                     buf.stride(-2), buf.stride(0), batch, M, float(alpha), float(beta),
                                     1 if symmetric else 0, _stream_ptr(A.device)))
    return _finish(buf, user, A.ndim, (M, M))


def ns_line_3(B: Tensor, X: Tensor, a: float, *, out: Tensor = None) -> Tensor:
    """C = a * X + B @ X for square bf16 B and bf16 X with the same row count (muon.py:705-746)."""
    if B.shape[-2] != B.shape[-1]:
        raise ValueError("B must be square")
    if B.shape[-2] != X.shape[-2]:
        raise ValueError("B and X must have the same number of rows")
    B3, bb = _as_bf16_3d(B, "B")
    X3, batch = _as_bf16_3d(X, "X")
    if bb != batch:
        raise ValueError("B and X must have the same batch size")
    M, N = X3.shape[-2:]
    buf, user = _out_3d(out, X, (batch, M, N))
    if buf.data_ptr() == X3.data_ptr():
        buf, user = _out_3d(None, X, (batch, M, N))[0], out
    with torch.cuda.device(X.device):
        check(lib.muon_b200_ns_line3(B3.data_ptr(), B3.stride(-2), B3.stride(0), X3.data_ptr(),
                                     X3.stride(-2), X3.stride(0), buf.data_ptr(), buf.stride(-2),
                                     buf.stride(0), batch, M, N, float(a), _stream_ptr(X.device)))
    return _finish(buf, user, X.ndim, (M, N))


def _finish(buf: Tensor, user: Tensor | None, ndim: int, mat_shape: tuple[int, int]) -> Tensor:
    res = buf if ndim == 3 else buf[0]
    if user is not None:
        user.copy_(res.reshape(user.shape))
        return user
    return res


def zeropower_via_newtonschulz5(G: Tensor, epsilon: float = 1e-7) -> Tensor:
    """Newton-Schulz orthogonalisation of G (muon.py:749): bf16 result of G's shape.
    The variant (AOL / classic) is the module-level setting of ``set_ns_mode``."""
    return get_backend().newton_schulz(G, epsilon)


def muon_update(grad: Tensor, momentum: Tensor, beta: float = 0.95, nesterov: bool = True) -> Tensor:
    """muon.py:8-15: momentum update in place, Nesterov blend written back into ``grad``,
    then the orthogonalised, aspect-scaled bf16 update of the (collapsed) 2-D shape. Three library
    calls (prologue, Newton-Schulz, scale); the result is a fresh tensor, scratch is cached."""
    _require_cuda(grad, "grad")
    if grad.shape != momentum.shape or grad.dtype != momentum.dtype:
        raise ValueError("grad and momentum must have the same shape and dtype")
    if not (grad.is_contiguous() and momentum.is_contiguous()):
        raise ValueError("muon_update needs contiguous grad and momentum")
    rows, cols = view_2d(grad.shape)
    tall = rows > cols
    m_, n_ = (cols, rows) if tall else (rows, cols)
    ldn = (n_ + 7) // 8 * 8
    dev = grad.device
    backend = get_backend()
    with torch.cuda.device(dev):
        stage_bytes = (m_ * ldn * 2 + 255) // 256 * 256  # bf16 X as the prologue leaves it
        mode, steps = get_ns_mode()
        need = lib.muon_b200_zeropower_scratch_bytes(1, m_, n_, _NS_MODES[mode])
        ws = backend.workspace(dev, stage_bytes + need, slot=3)
        stage = backend._aligned_ptr(ws)
        stream = _stream_ptr(dev)
        check(lib.muon_b200_prologue(_lib.ptr_array([grad.data_ptr()]), _lib.ptr_array([momentum.data_ptr()]),
                                     1, rows, cols, dtype_code(grad), beta, 1 if nesterov else 0,
                                     stage, ldn, m_ * ldn, 1 if tall else 0, stream))
        out = torch.empty(m_, ldn, dtype=torch.bfloat16, device=dev)
        check(lib.muon_b200_zeropower(stage, _lib.BF16, m_, n_, ldn, m_ * ldn, 1, out.data_ptr(), ldn, m_ * ldn,
                                      stage + stage_bytes, need, _NS_MODES[mode], steps, None, 1e-7, stream))
        scale = aspect_scale(grad.shape)
        if scale != 1:  # update *= max(1, rows/cols)**0.5, rounded to bf16 like the reference's multiply
            check(lib.muon_b200_cast_bf16(out.data_ptr(), _lib.BF16, m_, n_, ldn, m_ * ldn, out.data_ptr(), ldn,
                                          m_ * ldn, 1, 0, scale, stream))
    out = out[:, :n_]
    return out.mT if tall else out


def adam_update(grad: Tensor, buf1: Tensor, buf2: Tensor, step: int, betas, eps: float) -> Tensor:
    """muon.py:104-109: updates ``buf1``/``buf2`` in place and returns the Adam direction.
    Runs the fused kernel on a zero parameter with lr = -1, which leaves exactly u."""
    _require_cuda(grad, "grad")
    u = torch.zeros_like(grad)
    get_backend().adam_step([u], [grad.contiguous()], [buf1], [buf2], [int(step)], -1.0, 0.0,
                            (betas[0], betas[1]), eps)
    return u
