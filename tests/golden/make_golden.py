"""Generates tests/golden/*.pt from the REAL reference (thib-s/Muon's muon.py) on CPU.

Run in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/reference [fixture names ...]

What the real reference can execute without a GPU, and what each fixture therefore pins:

* ``adam.pt``        real ``SingleDeviceMuonWithAuxAdam`` Adam groups, 3 steps (muon.py:104-109, :244-258).
* ``ns_lines_fp32.pt`` the real Triton kernels ``ns_line_1/2/3`` under Triton's CPU interpreter, fp32
                     inputs, tile configs pinned to 64x64x64 (the interpreter cannot execute bf16).
* ``ns_reference_bf16.pt`` the real ``zeropower_via_newtonschulz5`` driver run uncompiled on CPU, calling
                     the real Triton kernels under the interpreter with bf16 operands passed as fp32 and
                     each result rounded to bf16 once (see ``gen_ns_reference_bf16``); one case keeps the
                     output of each of its 12 kernel calls.
* ``muon_glue.pt``   real ``SingleDeviceMuon`` / ``muon_update`` (momentum lerps, Nesterov write-back,
                     4-D view, aspect scale, weight decay, apply; muon.py:8-15, :81-101) with
                     ``zeropower_via_newtonschulz5`` replaced by the oracle's restatement, because the
                     real one needs a GPU. Inputs: fp32 wide, fp32 tall, bf16, 4-D filter with kH > kW.
* ``config1_reference.pt`` real ``SingleDeviceMuon`` for 3 steps on one fp32 768 x 3072 parameter with the real
                     Newton-Schulz driver and kernels executed as for ``ns_reference_bf16.pt``; rows kept.
* ``distributed.pt`` real distributed ``Muon`` on two gloo CPU ranks (ownership, padding, all_gather,
                     state on the owner only, a parameter without gradient), NS substituted as above.
* ``api.pt``         constructor behaviour: sort order, group keys and defaults, assertion cases.
* ``ns_oracle_bf16.pt`` the oracle's own bf16 Newton-Schulz output on seeded inputs (a drift guard for the
                     restatement itself; NOT produced by the reference).

Everything is seeded; files are a few hundred KB in total.
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
os.environ["TORCH_COMPILE_DISABLE"] = "1"

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
ref_dir = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MUON_REFERENCE_DIR", "")
if not os.path.isfile(os.path.join(ref_dir, "muon.py")):
    raise SystemExit("usage: make_golden.py <directory holding the reference's muon.py>")
sys.path.insert(0, ref_dir)

import muon as ref  # noqa: E402  the real reference module
from oracle import muon_oracle as orc  # noqa: E402

assert os.path.realpath(ref.__file__).startswith(os.path.realpath(ref_dir)), ref.__file__
REAL_NS = ref.zeropower_via_newtonschulz5  # gen_muon_glue replaces the module attribute later


def _pin_tiles():
    """One 64 x 64 x 64 configuration per kernel: the autotuner needs a GPU to choose among several."""
    for k in (ref.ns_line_1_kernel, ref.ns_line_2_kernel, ref.ns_line_3_kernel):
        k.configs = [c for c in k.configs
                     if c.kwargs["BLOCK_SIZE_M"] == 64 and c.kwargs["BLOCK_SIZE_N"] == 64
                     and c.kwargs["BLOCK_SIZE_K"] == 64][:1]


def gen_adam():
    torch.manual_seed(11)
    shapes = [(768,), (1000,), (7,), (33, 5), (4, 3, 2)]
    out = {"shapes": shapes, "cases": []}
    for dtype in (torch.float32, torch.bfloat16):
        params = [torch.nn.Parameter(torch.randn(s).to(dtype)) for s in shapes]
        p0 = [p.detach().clone() for p in params]
        grads = [[(torch.randn(s) * 0.01).to(dtype) for s in shapes] for _ in range(3)]
        opt = ref.SingleDeviceMuonWithAuxAdam(
            [dict(params=params, use_muon=False, lr=3e-3, betas=(0.9, 0.95), eps=1e-10, weight_decay=0.01)])
        for step_grads in grads:
            for p, g in zip(params, step_grads):
                p.grad = g.clone()
            opt.step()
        out["cases"].append(dict(
            dtype=dtype, p0=p0, grads=grads, p=[p.detach().clone() for p in params],
            exp_avg=[opt.state[p]["exp_avg"].clone() for p in params],
            exp_avg_sq=[opt.state[p]["exp_avg_sq"].clone() for p in params],
            step=[opt.state[p]["step"] for p in params],
            hyper=dict(lr=3e-3, betas=(0.9, 0.95), eps=1e-10, weight_decay=0.01)))
    # functional form, one call
    g = torch.randn(50); b1 = torch.randn(50) * 0.1; b2 = torch.rand(50) * 0.1
    b1o, b2o = b1.clone(), b2.clone()
    u = ref.adam_update(g, b1o, b2o, 3, (0.9, 0.95), 1e-10)
    out["functional"] = dict(grad=g, buf1=b1, buf2=b2, step=3, betas=(0.9, 0.95), eps=1e-10,
                             buf1_out=b1o, buf2_out=b2o, update=u)
    return out


def gen_ns_lines_fp32():
    _pin_tiles()
    torch.manual_seed(5)
    cases = []
    for (m, n, batch) in [(96, 160, None), (64, 64, None), (130, 200, None), (72, 136, 2)]:
        shape = (m, n) if batch is None else (batch, m, n)
        X = torch.randn(shape)
        A = ref.ns_line_1(X)
        As = A / A.abs().sum(-1, keepdim=True)  # asymmetric on purpose, like muon.py:785
        B = ref.ns_line_2(As, alpha=2.4635, beta=-7.0585)
        C = ref.ns_line_3(B, X, 4.0098)
        cases.append(dict(X=X, A=A, As=As, alpha=2.4635, beta=-7.0585, B=B, a=4.0098, C=C, tile=64))
    return {"cases": cases}


class kernels_through_fp32:
    """While active, the reference's ``ns_line_1/2/3`` launchers receive their bf16 operands
    converted to fp32 (exact) and their fp32 result is rounded to bf16 once — the kernels' own
    semantics (fp32 accumulation, one rounding at the store, muon.py:404-405, :531-532, :696-697),
    executable by the Triton interpreter, which cannot compute in bf16. Every call is recorded."""

    NAMES = ("ns_line_1", "ns_line_2", "ns_line_3")

    def __init__(self, keep_inputs=False):
        self.trace, self.keep_inputs = [], keep_inputs

    def _wrap(self, name, fn):
        def wrapped(*args, out=None, **kw):
            conv = [a.float().contiguous() if torch.is_tensor(a) else a for a in args]
            res = fn(*conv, **kw).to(torch.bfloat16)
            scalars = dict(kw)
            if name == "ns_line_3":
                scalars["a"] = args[2]
            rec = dict(name=name, scalars=scalars, out=res.clone())
            if self.keep_inputs:
                rec["inputs"] = [a.clone() for a in args if torch.is_tensor(a)]
            self.trace.append(rec)
            if out is not None:
                out.copy_(res)
                return out
            return res
        return wrapped

    def __enter__(self):
        _pin_tiles()
        self.real = {n: getattr(ref, n) for n in self.NAMES}
        self.real_ns = ref.zeropower_via_newtonschulz5
        for n, f in self.real.items():
            setattr(ref, n, self._wrap(n, f))
        ref.zeropower_via_newtonschulz5 = REAL_NS
        return self

    def __exit__(self, *exc):
        for n, f in self.real.items():
            setattr(ref, n, f)
        ref.zeropower_via_newtonschulz5 = self.real_ns


def gen_ns_reference_bf16():
    """The real ``zeropower_via_newtonschulz5`` (muon.py:748-799) executed on CPU: its own driver
    code (uncompiled, so every torch op rounds to bf16) calling its own Triton kernels under the
    interpreter (see ``kernels_through_fp32``). For one case every kernel call's output is kept, so
    that the restatement can be checked call by call on the reference's own intermediate values."""
    with kernels_through_fp32(keep_inputs=True) as k:
        torch.manual_seed(41)
        cases = []
        for shape, keep_trace in [((64, 160), False), ((160, 64), False), ((96, 96), False),
                                  ((2, 72, 136), True), ((130, 200), False)]:
            k.trace.clear()
            G = torch.randn(shape).bfloat16()
            U = REAL_NS(G)
            case = dict(G=G, U=U.clone(), tile=64)
            if keep_trace:
                # Inputs of a call are outputs of earlier calls, except the rescaled X and A that the
                # driver's own elementwise code produces (muon.py:779-785): keep those two.
                case["outputs"] = [dict(name=t["name"], scalars=t["scalars"], out=t["out"]) for t in k.trace]
                case["A_rescaled"] = k.trace[1]["inputs"][0]   # operand of the first ns_line_2
                case["X_rescaled"] = k.trace[2]["inputs"][1]   # second operand of the first ns_line_3
            cases.append(case)
    return {"cases": cases}


CONFIG1 = dict(shape=(768, 3072), seed=0, steps=3, lr=0.02, weight_decay=0.01, momentum=0.95, row_stride=96)


def config1_problem():
    """One fp32 parameter 768 x 3072 (randn * 0.02), gradients ~N(0, 1), seed 0: the first
    configuration the benchmark definition lists. Regenerated from the seed by the tests."""
    g = torch.Generator().manual_seed(CONFIG1["seed"])
    p0 = torch.randn(CONFIG1["shape"], generator=g) * 0.02
    grads = [torch.randn(CONFIG1["shape"], generator=g) for _ in range(CONFIG1["steps"])]
    return p0, grads


def gen_config1_reference():
    """Real ``SingleDeviceMuon`` (muon.py:73-101) for three steps on that parameter with the real
    Newton-Schulz driver and kernels (interpreter, see ``kernels_through_fp32``): momentum, Nesterov
    blend, NS, aspect scale, weight decay and apply, all the reference's own code. Takes about a
    quarter of an hour. Kept: every 96th row of the parameter, the momentum and the mutated
    gradient after each step (the full tensors are 9 MB each), and norms of the full tensors."""
    p0, grads = config1_problem()
    s = CONFIG1["row_stride"]
    p = torch.nn.Parameter(p0.clone())
    steps = []
    with kernels_through_fp32():
        opt = ref.SingleDeviceMuon([p], lr=CONFIG1["lr"], weight_decay=CONFIG1["weight_decay"],
                                   momentum=CONFIG1["momentum"])
        for g in grads:
            p.grad = g.clone()
            opt.step()
            mom = opt.state[p]["momentum_buffer"]
            steps.append(dict(p_rows=p.detach()[::s].clone(), momentum_rows=mom[::s].clone(),
                              grad_after_rows=p.grad[::s].clone(),
                              p_norm=p.detach().double().norm().item(), momentum_norm=mom.double().norm().item()))
            print("config1 step done", flush=True)
    return dict(config=CONFIG1, p0_rows=p0[::s].clone(), grad_rows=[g[::s].clone() for g in grads], steps=steps)


def gen_muon_glue():
    ref.zeropower_via_newtonschulz5 = orc.zeropower_via_newtonschulz5  # the one substitution
    torch.manual_seed(23)
    specs = [((64, 160), torch.float32), ((160, 64), torch.float32), ((48, 96), torch.bfloat16),
             ((32, 16, 4, 2), torch.float32), ((96, 48), torch.bfloat16)]
    hyper = dict(lr=0.02, weight_decay=0.01, momentum=0.95)
    cases = []
    for shape, dtype in specs:
        p = torch.nn.Parameter((torch.randn(shape) * 0.02).to(dtype))
        p0 = p.detach().clone()
        grads = [torch.randn(shape).to(dtype) for _ in range(3)]
        opt = ref.SingleDeviceMuon([p], **hyper)
        trace = []
        for g in grads:
            p.grad = g.clone()
            opt.step()
            trace.append(dict(p=p.detach().clone(), grad_after=p.grad.clone(),
                              momentum=opt.state[p]["momentum_buffer"].clone()))
        cases.append(dict(shape=shape, dtype=dtype, p0=p0, grads=grads, trace=trace, hyper=hyper))
    # functional muon_update, nesterov on/off
    fn = []
    for nesterov in (True, False):
        g = torch.randn(40, 72); m = torch.randn(40, 72) * 0.1
        g_in, m_in = g.clone(), m.clone()
        u = ref.muon_update(g, m, beta=0.9, nesterov=nesterov)
        fn.append(dict(grad=g_in, momentum=m_in, beta=0.9, nesterov=nesterov, grad_out=g, momentum_out=m,
                       update=u.clone()))
    return {"cases": cases, "functional": fn}


def gen_api():
    out = {}
    ps = [torch.nn.Parameter(torch.zeros(s)) for s in [(32, 64), (64, 32), (64, 64), (16, 64), (64, 32)]]
    # Muon needs a process group only in step(); construction works without one.
    m = ref.Muon(list(ps))
    out["muon_sorted_shapes"] = [tuple(p.shape) for p in m.param_groups[0]["params"]]
    out["muon_group_keys"] = sorted(k for k in m.param_groups[0].keys())
    out["muon_defaults"] = {k: m.param_groups[0][k] for k in ("lr", "momentum", "weight_decay")}
    try:
        ref.Muon([dict(params=ps)])
        out["muon_rejects_group_dicts"] = False
    except AssertionError:
        out["muon_rejects_group_dicts"] = True
    s = ref.SingleDeviceMuon([dict(params=ps)])
    out["single_accepts_group_dicts"] = True
    out["single_order_kept"] = [tuple(p.shape) for p in s.param_groups[0]["params"]]
    aux = ref.MuonWithAuxAdam([dict(params=list(ps), use_muon=True),
                               dict(params=[torch.nn.Parameter(torch.zeros(5))], use_muon=False)])
    out["aux_muon_group"] = {k: v for k, v in aux.param_groups[0].items() if k != "params"}
    out["aux_adam_group"] = {k: v for k, v in aux.param_groups[1].items() if k != "params"}
    out["aux_sorted_shapes"] = [tuple(p.shape) for p in aux.param_groups[0]["params"]]
    saux = ref.SingleDeviceMuonWithAuxAdam([dict(params=list(ps), use_muon=True)])
    out["single_aux_order_kept"] = [tuple(p.shape) for p in saux.param_groups[0]["params"]]
    for bad_key in ("nesterov", "ns_steps"):
        try:
            ref.MuonWithAuxAdam([dict(params=list(ps), use_muon=True, **{bad_key: 1})])
            out[f"aux_rejects_{bad_key}"] = False
        except AssertionError:
            out[f"aux_rejects_{bad_key}"] = True
    try:
        ref.MuonWithAuxAdam([dict(params=list(ps))])
        out["aux_requires_use_muon"] = False
    except AssertionError:
        out["aux_requires_use_muon"] = True
    return out


def gen_ns_oracle():
    torch.manual_seed(31)
    cases = []
    for shape in [(64, 160), (160, 64), (96, 96), (3, 40, 72)]:
        G = torch.randn(shape)
        U = orc.zeropower_via_newtonschulz5(G)
        Uc = orc.zeropower_classic5(G)
        Uf = orc.zeropower_classic5(G, folded=True)  # the arithmetic of the CUDA path
        cases.append(dict(G=G, aol4=U.clone(), classic5=Uc.clone(), classic5_folded=Uf.clone()))
    return {"cases": cases}


DIST_SHAPES = [(24, 48)] * 4 + [(48, 24)] * 2 + [(16, 16)]
DIST_WORLD = 2


def _dist_rank(rank, world, tmpdir):
    """One gloo rank of the real distributed ``Muon`` (muon.py:18-70)."""
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    dist.init_process_group("gloo", init_method=f"file://{tmpdir}/pg", rank=rank, world_size=world)
    try:
        ref.zeropower_via_newtonschulz5 = orc.zeropower_via_newtonschulz5  # as in gen_muon_glue
        problem = torch.load(f"{tmpdir}/problem.pt")
        params = [torch.nn.Parameter(p.clone()) for p in problem["p0"]]
        opt = ref.Muon(list(params), lr=0.02, weight_decay=0.01, momentum=0.95)
        for step_grads in problem["grads"]:
            for i, (p, g) in enumerate(zip(params, step_grads)):
                p.grad = None if i == problem["no_grad_index"] else g.clone()
            opt.step()
        sorted_params = opt.param_groups[0]["params"]
        out = dict(params=[p.detach().clone() for p in params],
                   sorted_shapes=[tuple(p.shape) for p in sorted_params],
                   has_state=[i for i, p in enumerate(sorted_params) if len(opt.state[p]) > 0])
        # the same problem through MuonWithAuxAdam (muon.py:112-199), with 1-D gains in an Adam group
        params = [torch.nn.Parameter(p.clone()) for p in problem["p0"]]
        gains = [torch.nn.Parameter(g.clone()) for g in problem["gains0"]]
        aux = ref.MuonWithAuxAdam([dict(params=list(params), use_muon=True, lr=0.02, weight_decay=0.01),
                                   dict(params=gains, use_muon=False, lr=3e-3, weight_decay=0.01)])
        for step_grads, gain_grads in zip(problem["grads"], problem["gain_grads"]):
            for i, (p, g) in enumerate(zip(params, step_grads)):
                p.grad = None if i == problem["no_grad_index"] else g.clone()
            for q, g in zip(gains, gain_grads):
                q.grad = g.clone()
            aux.step()
        sorted_params = aux.param_groups[0]["params"]
        out["aux"] = dict(params=[p.detach().clone() for p in params], gains=[q.detach().clone() for q in gains],
                          has_state=[i for i, p in enumerate(sorted_params) if len(aux.state[p]) > 0],
                          adam_steps=[aux.state[q]["step"] for q in gains])
        torch.save(out, f"{tmpdir}/out{rank}.pt")
    finally:
        dist.destroy_process_group()


def gen_distributed():
    """Real ``Muon`` and real ``MuonWithAuxAdam`` on two gloo CPU ranks, shape-homogeneous windows
    (the reference's all_gather rejects mixed ones), one parameter that never receives a gradient,
    a padded tail window, two 1-D Adam parameters."""
    import tempfile
    import torch.multiprocessing as mp
    torch.manual_seed(61)
    problem = dict(p0=[torch.randn(s) * 0.02 for s in DIST_SHAPES],
                   grads=[[torch.randn(s) for s in DIST_SHAPES] for _ in range(2)], no_grad_index=1)
    problem["gains0"] = [torch.ones(48), torch.randn(24)]
    problem["gain_grads"] = [[torch.randn(48) * 0.1, torch.randn(24) * 0.1] for _ in range(2)]
    with tempfile.TemporaryDirectory() as tmp:
        torch.save(problem, f"{tmp}/problem.pt")
        mp.spawn(_dist_rank, args=(DIST_WORLD, tmp), nprocs=DIST_WORLD, join=True)
        ranks = [torch.load(f"{tmp}/out{r}.pt") for r in range(DIST_WORLD)]
    return dict(problem, world=DIST_WORLD, ranks=ranks, hyper=dict(lr=0.02, weight_decay=0.01, momentum=0.95))


if __name__ == "__main__":
    only = sys.argv[2:]
    for name, fn in [("adam", gen_adam), ("ns_lines_fp32", gen_ns_lines_fp32), ("api", gen_api),
                     ("ns_reference_bf16", gen_ns_reference_bf16),
                     ("distributed", gen_distributed), ("config1_reference", gen_config1_reference),
                     ("ns_oracle_bf16", gen_ns_oracle), ("muon_glue", gen_muon_glue)]:
        if only and name not in only:
            continue
        data = fn()
        path = os.path.join(HERE, f"{name}.pt")
        torch.save(data, path)
        print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")
