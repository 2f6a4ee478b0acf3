"""Runs the REAL reference (thib-s/Muon's muon.py: torch.compile'd driver, autotuned Triton kernels)
on a B200 and writes what the GPU tests compare against: ``reference_b200.pt``.

    python tests/golden/make_reference_b200.py <dir with the reference's muon.py> <output dir>

The first argument is the directory of the unmodified reference install (``baseline/_ref`` after
``python -m pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <reference>``).
The second receives

* ``reference_b200.pt``        the fixture: for every shape the seed, a fixed subset of rows of the
                               reference's Newton-Schulz output, its singular-value band, the
                               run-to-run spread of the reference itself, and the three-step
                               ``SingleDeviceMuon`` run of the first benchmark configuration;
* ``reference_b200_report.json`` distances of this library's output to the reference at generation
                               time, reference and library timings per shape and per workload step,
                               and the store pattern the reference's line-2 kernel leaves for a
                               non-symmetric input (which of the two values each block ends up with).

Inputs are drawn on the CPU from seeded generators (``case_input``), so the tests rebuild them
bit for bit without this script. Nothing here modifies the reference; the only settings touched are
dynamo's recompile limits (one compilation per shape is intended, muon.py:748).
"""
import importlib.util
import json
import os
import sys
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

# (shape, input dtype, gradient std, seed). Shapes and distributions of the five benchmark
# configurations; the last three are single matrices of the Llama-3-8B / 70B layers.
CASES = [
    ((768, 768), torch.float32, 1e-2, 101),
    ((768, 3072), torch.float32, 1.0, 102),
    ((3072, 768), torch.float32, 1e-2, 103),
    ((256, 2304), torch.float32, 1.0, 104),
    ((128, 1152), torch.float32, 1.0, 105),
    ((1024, 4096), torch.bfloat16, 1e-3, 106),
    ((4096, 4096), torch.bfloat16, 1e-3, 107),
    ((4096, 14336), torch.bfloat16, 1e-3, 108),
    ((14336, 4096), torch.bfloat16, 1e-3, 109),
    ((1024, 8192), torch.bfloat16, 1e-3, 110),
]
ROWS_KEPT = 32


def case_input(shape, dtype, std, seed):
    """The seeded CPU input of a case (also used by the tests)."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype)


def kept_rows(shape):
    return torch.linspace(0, shape[0] - 1, ROWS_KEPT).round().long()


def rel_fro(x, ref):
    x, ref = x.double(), ref.double()
    return float((x - ref).norm() / ref.norm().clamp_min(1e-30))


def sv_band(U):
    """Smallest and largest singular value from the eigenvalues of the fp64 Gram matrix."""
    Uf = U.double()
    gram = Uf @ Uf.mT if U.shape[-2] <= U.shape[-1] else Uf.mT @ Uf
    ev = torch.linalg.eigvalsh(gram).clamp_min(0).sqrt()
    return float(ev.min()), float(ev.max())


def time_ms(fn, reps=5):
    fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(reps):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        fn()
        t1.record()
        torch.cuda.synchronize()
        out.append(t0.elapsed_time(t1))
    out.sort()
    return out[len(out) // 2]


def load_reference(ref_dir):
    path = os.path.join(ref_dir, "muon.py")
    if not os.path.isfile(path):
        raise SystemExit(f"no muon.py in {ref_dir}")
    spec = importlib.util.spec_from_file_location("muon_reference", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["muon_reference"] = mod
    spec.loader.exec_module(mod)
    return mod


def line2_store_pattern(ref, m):
    """Feeds the reference's line-2 kernel a non-symmetric matrix and reports, per 32 x 32 block,
    whether the block holds the value computed at its own position ('d'), the transposed one
    ('t'), or a mix ('x'). This is what its two stores (muon.py:534-544) leave on this GPU with
    the tile shape its autotuner picked."""
    g = torch.Generator().manual_seed(900 + m)
    A = (torch.randn(m, m, generator=g) * 0.05).bfloat16().cuda()
    out = ref.ns_line_2(A, alpha=2.4635, beta=-7.0585)
    Af = A.float()
    D = ((Af @ Af.mT) * 2.4635 + Af * -7.0585).bfloat16()
    direct = (out == D)
    trans = (out == D.mT)
    nb = (m + 31) // 32
    rows = []
    for i in range(nb):
        row = ""
        for j in range(nb):
            d = direct[i * 32:(i + 1) * 32, j * 32:(j + 1) * 32].float().mean().item()
            t = trans[i * 32:(i + 1) * 32, j * 32:(j + 1) * 32].float().mean().item()
            row += "d" if d > 0.99 and t < 0.9 else "t" if t > 0.99 and d < 0.9 else "b" if d > 0.99 and t > 0.99 else "x"
        rows.append(row)
    best = getattr(ref.ns_line_2_kernel, "best_config", None)
    return {"m": m, "blocks": rows if nb <= 32 else rows[:8] + ["..."], "best_config": str(best),
            "frac_direct": float(direct.float().mean()), "frac_transposed": float(trans.float().mean())}


def main():
    ref_dir, out_dir = sys.argv[1], sys.argv[2]
    only_fast = "--fast" in sys.argv
    os.makedirs(out_dir, exist_ok=True)
    import torch._dynamo
    torch._dynamo.config.cache_size_limit = 256
    if hasattr(torch._dynamo.config, "recompile_limit"):
        torch._dynamo.config.recompile_limit = 256
    if hasattr(torch._dynamo.config, "accumulated_recompile_limit"):
        torch._dynamo.config.accumulated_recompile_limit = 1024
    ref = load_reference(ref_dir)
    import muon_b200

    dev = torch.device("cuda", 0)
    fixture = {"cases": [], "rows_kept": ROWS_KEPT, "torch": torch.__version__,
               "gpu": torch.cuda.get_device_name(0)}
    report = {"cases": [], "line2_store_pattern": [], "steps": []}
    t_start = time.time()

    def flush():
        torch.save(fixture, os.path.join(out_dir, "reference_b200.pt"))
        with open(os.path.join(out_dir, "reference_b200_report.json"), "w") as f:
            json.dump(report, f, indent=1)

    for shape, dtype, std, seed in CASES:
        t0 = time.time()
        G = case_input(shape, dtype, std, seed).to(dev)
        U1 = ref.zeropower_via_newtonschulz5(G).contiguous()
        torch.cuda.synchronize()
        compile_s = time.time() - t0
        U2 = ref.zeropower_via_newtonschulz5(G).contiguous()
        ours = muon_b200.zeropower_via_newtonschulz5(G).contiguous()
        torch.cuda.synchronize()
        rows = kept_rows(shape)
        lo, hi = sv_band(U1)
        olo, ohi = sv_band(ours)
        ref_ms = time_ms(lambda: ref.zeropower_via_newtonschulz5(G))
        our_ms = time_ms(lambda: muon_b200.zeropower_via_newtonschulz5(G))
        m, n = min(shape), max(shape)
        flops = 4 * (m * (m + 1) * n + m * m * (m + 1) + 2 * m * m * n)
        fixture["cases"].append(dict(shape=shape, dtype=dtype, std=std, seed=seed, rows=rows,
                                     U_rows=U1[rows.to(dev)].cpu(), sv_band=(lo, hi),
                                     fro=float(U1.double().norm()), self_spread=rel_fro(U2, U1)))
        report["cases"].append(dict(shape=list(shape), dtype=str(dtype), first_call_s=compile_s,
                                    ours_vs_reference=rel_fro(ours, U1),
                                    ours_vs_reference_kept_rows=rel_fro(ours[rows.to(dev)], U1[rows.to(dev)]),
                                    reference_self_spread=rel_fro(U2, U1),
                                    reference_sv_band=[lo, hi], ours_sv_band=[olo, ohi],
                                    reference_ms=ref_ms, ours_ms=our_ms,
                                    reference_tflops_sym=flops / ref_ms / 1e9,
                                    ours_tflops_sym=flops / our_ms / 1e9,
                                    configs={k: str(getattr(getattr(ref, k), "best_config", None))
                                             for k in ("ns_line_1_kernel", "ns_line_2_kernel", "ns_line_3_kernel")}))
        print(f"[{time.time() - t_start:7.1f}s] {shape} first call {compile_s:.1f}s  ours-vs-ref "
              f"{report['cases'][-1]['ours_vs_reference']:.3e}  self {rel_fro(U2, U1):.3e}  "
              f"ref {ref_ms:.3f} ms  ours {our_ms:.3f} ms", flush=True)
        if shape[0] * shape[1] <= 2_400_000:  # small enough to keep whole for offline analysis
            torch.save(dict(G=G.cpu(), U=U1.cpu(), ours=ours.cpu()),
                       os.path.join(out_dir, f"reference_b200_full_{shape[0]}x{shape[1]}.pt"))
        del G, U1, U2, ours
        flush()

    for m in (128, 256, 768, 1024, 4096):
        report["line2_store_pattern"].append(line2_store_pattern(ref, m))
        print("line-2 store pattern", json.dumps(report["line2_store_pattern"][-1])[:600], flush=True)
    flush()

    # ---- the first benchmark configuration, three steps of the real SingleDeviceMuon ----
    g = torch.Generator().manual_seed(0)
    p0 = torch.randn(768, 3072, generator=g) * 0.02
    grads = [torch.randn(768, 3072, generator=g) for _ in range(3)]
    p_ref = torch.nn.Parameter(p0.clone().to(dev))
    p_our = torch.nn.Parameter(p0.clone().to(dev))
    o_ref = ref.SingleDeviceMuon([p_ref], lr=0.02, weight_decay=0.01, momentum=0.95)
    o_our = muon_b200.SingleDeviceMuon([p_our], lr=0.02, weight_decay=0.01, momentum=0.95)
    steps = []
    for k in range(3):
        p_ref.grad = grads[k].clone().to(dev)
        p_our.grad = grads[k].clone().to(dev)
        o_ref.step()
        o_our.step()
        torch.cuda.synchronize()
        steps.append(dict(p_rows=p_ref.detach()[::96].cpu().clone(),
                          momentum_rows=o_ref.state[p_ref]["momentum_buffer"][::96].cpu().clone(),
                          p_norm=float(p_ref.detach().double().norm())))
        report["steps"].append(dict(config="one 768x3072 fp32 parameter, step %d" % (k + 1),
                                    params_ours_vs_reference=rel_fro(p_our.detach(), p_ref.detach()),
                                    update_ours_vs_reference=rel_fro(p_our.detach() - p0.to(dev), p_ref.detach() - p0.to(dev))))
    fixture["config1"] = dict(seed=0, lr=0.02, weight_decay=0.01, momentum=0.95, row_stride=96,
                              p0_rows=p0[::96].clone(), steps=steps)
    print("config 1:", json.dumps(report["steps"]), flush=True)
    flush()
    if only_fast:
        return

    # ---- step times of the reference's own SingleDeviceMuon beside this library's ----
    workloads = {
        "one-768x3072": ([(768, 3072)], torch.float32, 1.0),
        "gpt2-small-hidden": (([(768, 768)] * 4 + [(3072, 768), (768, 3072)]) * 12, torch.float32, 1e-2),
        "conv-filters": ([(256, 256, 3, 3)] * 64 + [(128, 128, 3, 3)] * 64, torch.float32, 1.0),
        "llama3-8b-1layer": ([(4096, 4096), (4096, 4096), (1024, 4096), (1024, 4096), (14336, 4096),
                              (14336, 4096), (4096, 14336)], torch.bfloat16, 1e-3),
    }
    report["step_times"] = {}
    for name, (shapes, dtype, std) in workloads.items():
        def make(cls):
            gen = torch.Generator(device=dev).manual_seed(5)
            ps = [torch.nn.Parameter(torch.empty(s, device=dev, dtype=dtype).normal_(0, 0.02, generator=gen))
                  for s in shapes]
            for p in ps:
                p.grad = torch.empty(p.shape, device=dev, dtype=dtype).normal_(0, std, generator=gen)
            return cls(ps, lr=0.02, weight_decay=0.01, momentum=0.95)
        o_r, o_o = make(ref.SingleDeviceMuon), make(muon_b200.SingleDeviceMuon)
        t0 = time.time()
        r_ms = time_ms(o_r.step, reps=5)
        o_ms = time_ms(o_o.step, reps=5)
        report["step_times"][name] = dict(reference_ms=r_ms, ours_ms=o_ms, matrices=len(shapes),
                                          wall_s=time.time() - t0)
        print(f"[{time.time() - t_start:7.1f}s] step {name}: reference {r_ms:.3f} ms, ours {o_ms:.3f} ms", flush=True)
        del o_r, o_o
        torch.cuda.empty_cache()
        flush()


if __name__ == "__main__":
    main()
