"""The benchmark configurations as parity cases: GPT-2-small-shaped hidden weights with aux Adam
(reduced to 2 of 12 layers so that the CPU oracle finishes in seconds), batched conv filters
(8 + 8 of the 64 + 64), and the Llama-3-8B / 70B matrix shapes: against the CPU oracle matrix by
matrix (a few seconds each on the host cores), as one grouped launch, as a whole layer through the
optimizer, and through size-independent properties of the orthogonalised update.

Tolerances: Newton-Schulz output rel-Fro <= 2e-2 against the oracle with singular values in the
same band; updated fp32 parameters <= 1e-3; the accumulated update alone (p - p0, which is ~3% of
the parameter) <= 2e-2; bf16 parameters <= 4e-3 (they carry 2^-9 rounding themselves, and one step's
update is about one bf16 ulp of the parameter, so "the update alone" is only meaningful in fp32)."""
import pytest
import torch

from oracle import muon_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def mb():
    import muon_b200
    yield muon_b200
    assert muon_b200.device_status() == 0


def _step_both(mb, opt, params, ref_p, ref_m, grads, lr, wd, beta=0.95):
    for p, g in zip(params, grads):
        p.grad = g.clone().to(DEV)
    opt.step()
    for p, g, m in zip(ref_p, grads, ref_m):
        orc.muon_param_step(p, g.clone(), m, lr, wd, beta)


def test_gpt2_small_hidden_weights_with_aux_adam(mb, tmp_path):
    """12 layers x {q,k,v,o 768x768; fc 3072x768; proj 768x3072} fp32, grads ~N(0, 1e-2), 1-D gains
    through Adam, MuonWithAuxAdam on a one-rank process group. Two layers are compared."""
    import torch.distributed as dist
    dist.init_process_group("nccl", init_method=f"file://{tmp_path}/pg", rank=0, world_size=1)
    try:
        g = torch.Generator().manual_seed(2000)
        layer = [(768, 768)] * 4 + [(3072, 768), (768, 3072)]
        shapes = layer * 2
        p0 = [torch.randn(s, generator=g) * 0.02 for s in shapes]
        gains0 = [torch.ones(768) for _ in range(5)]
        hidden = [torch.nn.Parameter(p.clone().to(DEV)) for p in p0]
        gains = [torch.nn.Parameter(p.clone().to(DEV)) for p in gains0]
        opt = mb.MuonWithAuxAdam([dict(params=hidden, use_muon=True, lr=0.02, weight_decay=0.01),
                                  dict(params=gains, use_muon=False, lr=3e-4, betas=(0.9, 0.95), eps=1e-10,
                                       weight_decay=0)])
        sorted_hidden = opt.param_groups[0]["params"]
        ref = {id(p): q.clone() for p, q in zip(hidden, p0)}
        mom = {id(p): torch.zeros_like(q) for p, q in zip(hidden, p0)}
        ref_g = [p.clone() for p in gains0]
        ma, va = [torch.zeros(768) for _ in gains0], [torch.zeros(768) for _ in gains0]
        for step in (1, 2):
            grads = {id(p): torch.randn(p.shape, generator=g) * 1e-2 for p in hidden}
            gg = [torch.randn(768, generator=g) * 1e-2 for _ in gains0]
            for p in hidden:
                p.grad = grads[id(p)].clone().to(DEV)
            for p, gr in zip(gains, gg):
                p.grad = gr.clone().to(DEV)
            opt.step()
            for p in hidden:
                orc.muon_param_step(ref[id(p)], grads[id(p)].clone(), mom[id(p)], 0.02, 0.01, 0.95)
            for q, gr, m, v in zip(ref_g, gg, ma, va):
                orc.adam_param_step(q, gr.clone(), m, v, step, 3e-4, 0, (0.9, 0.95), 1e-10)
        assert [tuple(p.shape) for p in sorted_hidden] == sorted([tuple(s) for s in shapes], reverse=True)
        for p, start in zip(hidden, p0):
            assert orc.rel_fro(p.detach().cpu(), ref[id(p)]) <= 1e-3, tuple(p.shape)
            # the accumulated update alone
            assert orc.rel_fro(p.detach().cpu() - start, ref[id(p)] - start) <= 2e-2, tuple(p.shape)
        for p, q in zip(gains, ref_g):
            assert torch.allclose(p.detach().cpu(), q, rtol=1e-5, atol=1e-7)
    finally:
        dist.destroy_process_group()


def test_batched_conv_filters(mb):
    """256x256x3x3 (-> 256x2304) and 128x128x3x3 (-> 128x1152) fp32 filters, grads ~N(0,1),
    SingleDeviceMuon; every same-shape set goes through one grouped launch sequence."""
    g = torch.Generator().manual_seed(3000)
    shapes = [(256, 256, 3, 3)] * 8 + [(128, 128, 3, 3)] * 8
    p0 = [torch.randn(s, generator=g) * 0.02 for s in shapes]
    params = [torch.nn.Parameter(p.clone().to(DEV)) for p in p0]
    opt = mb.SingleDeviceMuon(params, lr=0.02, weight_decay=0.01)
    ref_p = [p.clone() for p in p0]
    ref_m = [torch.zeros_like(p) for p in p0]
    before = dict(mb._lib.launch_counts())
    for _ in range(2):
        grads = [torch.randn(s, generator=g) for s in shapes]
        _step_both(mb, opt, params, ref_p, ref_m, grads, 0.02, 0.01)
    after = mb._lib.launch_counts()
    assert after["prologue"] - before["prologue"] == 4  # 2 steps x 2 shape classes
    assert after["ns_line3"] - before["ns_line3"] == 16  # 2 steps x 2 classes x 4 iterations
    for p, r, start in zip(params, ref_p, p0):
        assert p.shape == r.shape and orc.rel_fro(p.detach().cpu(), r) <= 1e-3
        assert orc.rel_fro(p.detach().cpu() - start, r - start) <= 2e-2  # the accumulated update alone


def _spectral_norm_sym(S, iters=40):
    """Largest |eigenvalue| of a symmetric matrix by power iteration (a lower bound that converges
    from below; an SVD of an 8192 x 8192 matrix would take most of a minute)."""
    v = torch.ones(S.shape[0], 1, device=S.device) / S.shape[0] ** 0.5
    v = v + 1e-3 * torch.randn(v.shape, device=S.device, generator=torch.Generator(device=S.device).manual_seed(1))
    for _ in range(iters):
        w = S @ (S @ v)
        v = w / w.norm()
    return (S @ v).norm().item()


@pytest.mark.parametrize("shape", [(4096, 14336), (14336, 4096), (4096, 4096), (1024, 4096),
                                   (8192, 28672), (28672, 8192), (8192, 8192), (1024, 8192)])
def test_llama3_shapes_properties(mb, shape):
    """Full-size bf16 matrices of the Llama-3-8B and -70B layers, grads ~N(0, 1e-3): the update must
    be orthogonal up to the band the live algorithm guarantees, scale-invariant in the gradient,
    and deterministic."""
    g = torch.Generator(device=DEV).manual_seed(4000)
    G = torch.empty(shape, device=DEV, dtype=torch.bfloat16).normal_(0, 1e-3, generator=g)
    U = mb.zeropower_via_newtonschulz5(G)
    assert U.shape == G.shape and U.dtype == torch.bfloat16
    Uf = U.float()
    gram = Uf @ Uf.T if shape[0] <= shape[1] else Uf.T @ Uf
    eye = torch.eye(gram.shape[0], device=DEV)
    if shape[0] != shape[1]:
        # singular values within [0.98, 1.02] -> eigenvalues of the Gram matrix within ~[0.96, 1.04]
        dev = _spectral_norm_sym(gram - eye)
        assert dev < 0.05, dev
    else:
        assert _spectral_norm_sym(gram) < 1.2
    # alignment with the input: <U, G> equals the nuclear norm of G for the exact polar factor
    assert (Uf * G.float()).sum().item() > 0
    # NS normalises its input, so a power-of-two rescaling of G (exact in bf16) changes nothing
    assert torch.equal(mb.zeropower_via_newtonschulz5(G * 4), U)
    assert torch.equal(mb.zeropower_via_newtonschulz5(G), U)
    # transposition symmetry: NS(G^T) == NS(G)^T bit for bit (tall inputs run as their transpose;
    # a square input is iterated as it is, so the identity only holds up to rounding there)
    if shape[0] != shape[1]:
        assert torch.equal(mb.zeropower_via_newtonschulz5(G.T.contiguous()), U.T)


def _sv_band_gpu(U):
    """(min, max) singular value of a wide or tall matrix from the eigenvalues of its fp32 Gram
    matrix, on the GPU (an SVD of 4096 x 14336 on the host takes most of a minute)."""
    Uf = U.to(DEV).float()
    gram = Uf @ Uf.mT if Uf.shape[-2] <= Uf.shape[-1] else Uf.mT @ Uf
    ev = torch.linalg.eigvalsh(gram).clamp_min(0).sqrt()
    return float(ev.min()), float(ev.max())


LLAMA_ORACLE_SHAPES = [(1024, 4096), (4096, 4096), (4096, 14336), (14336, 4096), (1024, 8192), (8192, 8192),
                       (3, 1024, 4096), (3, 4096, 4096)]


@pytest.mark.parametrize("shape", LLAMA_ORACLE_SHAPES)
def test_llama3_shapes_against_the_oracle(mb, shape):
    """The matrices of a Llama-3-8B layer and the two 70B shapes whose oracle run stays within
    seconds, bf16 gradients ~N(0, 1e-3), single and as one grouped launch of three: Newton-Schulz
    output within 2e-2 (rel-Fro) of the CPU oracle, singular values in the same band."""
    g = torch.Generator().manual_seed(4100 + len(shape) * 7 + shape[-1] // 64 + shape[-2])
    G = (torch.randn(shape, generator=g) * 1e-3).bfloat16()
    before = dict(mb._lib.launch_counts())
    U = mb.zeropower_via_newtonschulz5(G.to(DEV))
    after = mb._lib.launch_counts()
    assert after["ns_line3"] - before["ns_line3"] == 4  # one launch per iteration, batch included
    ref = orc.zeropower_via_newtonschulz5(G)
    assert U.shape == G.shape and U.dtype == torch.bfloat16
    for k in range(shape[0] if len(shape) == 3 else 1):
        u, r = (U[k], ref[k]) if len(shape) == 3 else (U, ref)
        err = orc.rel_fro(u.cpu(), r)
        assert err <= 2e-2, (shape, k, err)
        if shape[-1] != shape[-2]:
            (lo, hi), (rlo, rhi) = _sv_band_gpu(u), _sv_band_gpu(r)
            assert abs(hi - rhi) <= 0.02 and abs(lo - rlo) <= 0.05, ((lo, hi), (rlo, rhi))
            assert 0.95 < lo and hi < 1.05


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_llama3_8b_layer_through_the_optimizer(mb, dtype):
    """q, o 4096 x 4096; k, v 1024 x 4096; gate, up 14336 x 4096; down 4096 x 14336 through
    SingleDeviceMuon (grouped by shape, tall ones transposed on the fly), against the oracle's
    per-parameter step. fp32 parameters: two steps, parameters <= 1e-3 and the accumulated update
    alone <= 2e-2. bf16 parameters (the benchmark's dtype): one step, parameters <= 4e-3 and the
    momentum buffer to one bf16 ulp."""
    shapes = [(4096, 4096), (4096, 4096), (1024, 4096), (1024, 4096), (14336, 4096), (14336, 4096), (4096, 14336)]
    steps = 2 if dtype == torch.float32 else 1
    g = torch.Generator().manual_seed(4200)
    p0 = [(torch.randn(s, generator=g) * 0.02).to(dtype) for s in shapes]
    params = [torch.nn.Parameter(p.clone().to(DEV)) for p in p0]
    opt = mb.SingleDeviceMuon(params, lr=0.02, weight_decay=0.01, momentum=0.95)
    ref_p = [p.clone() for p in p0]
    ref_m = [torch.zeros_like(p) for p in p0]
    for _ in range(steps):
        grads = [(torch.randn(s, generator=g) * 1e-3).to(dtype) for s in shapes]
        _step_both(mb, opt, params, ref_p, ref_m, grads, 0.02, 0.01)
    for p, r, start, m in zip(params, ref_p, p0, ref_m):
        got = p.detach().cpu()
        if dtype == torch.float32:
            assert orc.rel_fro(got, r) <= 1e-3, tuple(p.shape)
            assert orc.rel_fro(got - start, r - start) <= 2e-2, tuple(p.shape)
            assert torch.allclose(opt.state[p]["momentum_buffer"].cpu(), m, rtol=2e-6, atol=1e-9)
        else:
            assert orc.rel_fro(got, r) <= 4e-3, tuple(p.shape)
            mom = opt.state[p]["momentum_buffer"].cpu().float()
            assert ((mom - m.float()).abs() <= m.float().abs() * 2 ** -7 + 1e-12).all()


def test_llama3_70b_shapes_through_the_optimizer(mb):
    """The Llama-3-70B shapes whose oracle run stays within seconds (q 8192 x 8192; k, v
    1024 x 8192), bf16, one step of SingleDeviceMuon against the oracle's per-parameter step:
    parameters <= 4e-3 (bf16 parameters carry 2^-9 rounding themselves), momentum to one bf16
    ulp. The gate/up/down shapes (28672 x 8192 and its transpose) are covered by the property test
    above: their oracle run takes minutes."""
    shapes = [(8192, 8192), (1024, 8192), (1024, 8192)]
    g = torch.Generator().manual_seed(4300)
    p0 = [(torch.randn(s, generator=g) * 0.02).bfloat16() for s in shapes]
    params = [torch.nn.Parameter(p.clone().to(DEV)) for p in p0]
    opt = mb.SingleDeviceMuon(params, lr=0.02, weight_decay=0.01, momentum=0.95)
    ref_p = [p.clone() for p in p0]
    ref_m = [torch.zeros_like(p) for p in p0]
    grads = [(torch.randn(s, generator=g) * 1e-3).bfloat16() for s in shapes]
    _step_both(mb, opt, params, ref_p, ref_m, grads, 0.02, 0.01)
    for p, r, m in zip(params, ref_p, ref_m):
        assert orc.rel_fro(p.detach().cpu(), r) <= 4e-3, tuple(p.shape)
        mom = opt.state[p]["momentum_buffer"].cpu().float()
        assert ((mom - m.float()).abs() <= m.float().abs() * 2 ** -7 + 1e-12).all()


def test_gradients_arriving_on_a_copy_stream(mb):
    """Gradients copied in from pinned host memory on a side stream and marked with
    mark_grad_ready: step() called at once from the main stream gives bitwise the result of a step
    whose gradients were resident before it started, for Muon and for Adam parameters."""
    g = torch.Generator().manual_seed(77)
    shapes = [(512, 1024)] * 24 + [(1024, 256)] * 8
    p0 = [torch.randn(s, generator=g) * 0.02 for s in shapes]
    grads = [[torch.randn(s, generator=g).pin_memory() for s in shapes] for _ in range(2)]
    gain0 = torch.ones(4096)
    gain_grads = [torch.randn(4096, generator=g).pin_memory() for _ in range(2)]

    def make():
        ps = [torch.nn.Parameter(p.clone().to(DEV)) for p in p0]
        gain = torch.nn.Parameter(gain0.clone().to(DEV))
        opt = mb.SingleDeviceMuonWithAuxAdam([dict(params=ps, use_muon=True, lr=0.02, weight_decay=0.01),
                                              dict(params=[gain], use_muon=False, lr=1e-3)])
        return ps + [gain], opt

    ref_params, ref_opt = make()
    params, opt = make()
    copy_stream = torch.cuda.Stream()
    for step in range(2):
        host = grads[step] + [gain_grads[step]]
        for p, h in zip(ref_params, host):
            p.grad = h.to(DEV)
        torch.cuda.synchronize()
        ref_opt.step()
        for p in params:
            if p.grad is None:
                p.grad = torch.empty_like(p)
        copy_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(copy_stream):
            for p, h in zip(params, host):
                p.grad.copy_(h, non_blocking=True)
                mb.mark_grad_ready(p)
        opt.step()  # no synchronisation with copy_stream other than the marks
        torch.cuda.synchronize()
        for p, r in zip(params, ref_params):
            assert torch.equal(p, r)
    from muon_b200 import engine
    assert not engine._grad_ready  # every mark was consumed
