"""The allocation-free Newton-Schulz entry point (muon_b200_ns_run_static).

It exists for callers that may not allocate device memory when the step runs (a frozen
allocator inside a memory-planned region, a plugin that only receives buffers). This test calls
it through the C ABI, twice in a row, and checks each result against muon_b200_ns_run on a caller
workspace: the two run the same kernels in the same order, so the outputs must be identical. The
file name makes pytest collect it last, so a run that stops at the first failure has already
executed every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _workspace_result(L, X, mode=0, steps=0, coeffs=None):
    """muon_b200_ns_run on a caller workspace: the existing entry point."""
    batch, m, n = X.shape
    lay = L.ns_layout(batch, m, n)
    ws = torch.empty(lay.total_bytes + 256, dtype=torch.uint8, device=X.device)
    base = (ws.data_ptr() + 255) & ~255
    off = base - ws.data_ptr()

    def slot(o):
        return ws[off + o: off + o + batch * lay.x_bs * 2].view(torch.bfloat16).view(batch, m, lay.ldn)[:, :, :n]

    slot(lay.x_offset_bytes).copy_(X)
    which = ctypes.c_int(0)
    L.check(L.lib.muon_b200_ns_run(base, batch, m, n, mode, steps, _floats(coeffs), 1e-7, ctypes.byref(which),
                                   torch.cuda.current_stream().cuda_stream))
    return slot(lay.x_offset_bytes if which.value == 0 else lay.c_offset_bytes).clone()


def _floats(values):
    return None if values is None else (ctypes.c_float * len(values))(*values)


def _static_result(L, X, mode=0, steps=0, coeffs=None, out=None):
    batch, m, n = X.shape
    if out is None:
        out = torch.full_like(X, float("nan"))  # the caller owns input and output
    L.check(L.lib.muon_b200_ns_run_static(X.data_ptr(), X.stride(1), X.stride(0), out.data_ptr(),
                                          out.stride(1), out.stride(0), batch, m, n, mode, steps,
                                          _floats(coeffs), 1e-7, torch.cuda.current_stream().cuda_stream))
    return out


@pytest.mark.parametrize("shape", [(2, 256, 640), (1, 768, 3072)])
def test_static_scratch_variant_matches_workspace_variant(shape):
    import muon_b200._lib as L
    g = torch.Generator().manual_seed(41)
    X1 = torch.randn(shape, generator=g).bfloat16().cuda()
    X2 = torch.randn(shape, generator=g).bfloat16().cuda()
    x1_before = X1.clone()
    # two calls in a row share the built-in scratch: the second must not see the first's leftovers
    got1 = _static_result(L, X1)
    got2 = _static_result(L, X2)
    ref1 = _workspace_result(L, X1)
    ref2 = _workspace_result(L, X2)
    torch.cuda.synchronize()
    assert torch.equal(X1, x1_before), "the input must not be modified"
    assert torch.equal(got1, ref1)
    assert torch.equal(got2, ref2)
    assert not torch.equal(got1, got2)
    assert L.device_status() == 0


def test_static_scratch_variant_odd_iteration_count_and_limits():
    import muon_b200._lib as L
    g = torch.Generator().manual_seed(42)
    X = torch.randn(1, 128, 384, generator=g).bfloat16().cuda()
    # classic mode runs five iterations: the result still has to land in `out`, and it is the
    # workspace variant's result bit for bit (same kernels, same order)
    out = _static_result(L, X, mode=L.NS_CLASSIC5)
    assert torch.equal(out, _workspace_result(L, X, mode=L.NS_CLASSIC5))
    s = torch.linalg.svdvals(out[0].float())
    assert torch.isfinite(out.float()).all() and 0.3 < float(s.min()) and float(s.max()) < 1.3
    # three iterations given through `coeffs`, input and output as views with padded pitches
    coeffs = [3.0, -4.0, 1.5, 2.9, -3.5, 1.4, 2.7, -3.0, 1.3]
    Xp = torch.zeros(2, 128, 400, dtype=torch.bfloat16, device="cuda")
    Xp[:, :, :384] = torch.randn(2, 128, 384, generator=g).bfloat16().cuda()
    Xv = Xp[:, :, :384]
    Op = torch.full((2, 136, 392), float("nan"), dtype=torch.bfloat16, device="cuda")
    Ov = Op[:, :128, :384]
    _static_result(L, Xv, steps=3, coeffs=coeffs, out=Ov)
    assert torch.equal(Ov, _workspace_result(L, Xv.contiguous(), steps=3, coeffs=coeffs))
    assert torch.isnan(Op[:, 128:, :].float()).all() and torch.isnan(Op[:, :, 384:].float()).all()
    # neighbouring views of one buffer: out starts inside x's range
    both = torch.zeros(2 * 128 * 384 + 64, dtype=torch.bfloat16, device="cuda")
    rc = L.lib.muon_b200_ns_run_static(both.data_ptr(), 384, 0, both.data_ptr() + 128, 384, 0, 1, 128, 384,
                                       0, 0, None, 1e-7, None)
    assert rc == -1 and b"overlap" in L.lib.muon_b200_last_error()
    cap = L.lib.muon_b200_ns_static_scratch_bytes()
    assert cap == 64 << 20
    assert L.lib.muon_b200_ns_static_required_bytes(1, 768, 3072) <= cap
    assert L.lib.muon_b200_ns_static_required_bytes(1, 4096, 14336) > cap
    big = torch.empty(1, 8, 8, dtype=torch.bfloat16, device="cuda")
    rc = L.lib.muon_b200_ns_run_static(big.data_ptr(), 14336, 0, big.data_ptr() + 4096, 14336, 0, 1, 4096,
                                       14336, 0, 0, None, 1e-7, None)
    assert rc == -4 and b"scratch" in L.lib.muon_b200_last_error()
