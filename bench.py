#!/usr/bin/env python
"""Benchmark of the Muon optimizer step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workload (default ``llama3-8b-hidden``): the 224 hidden weight matrices of a Llama-3-8B-shaped
model (32 layers x {q,o 4096x4096; k,v 1024x4096; gate,up 14336x4096; down 4096x14336}), bf16
parameters, gradients and momentum, synthetic Gaussian data (params ~N(0, 0.02^2), grads
~N(0, 1e-3^2)), optimised by the distributed ``Muon`` class at N ranks (one per GPU, NCCL).
A "step" is one ``optimizer.step()`` over all 224 matrices. The job's total work is fixed, so
scaling is "strong". ``value`` is milliseconds per step (lower is better), timed with CUDA events
on the device with everything resident in HBM; ``e2e`` is the same step with the step's gradients
copied from pinned host memory and a result scalar read back inside the timed region.

Every timed step has its own pair of CUDA events; between steps, outside the timed intervals,
the gradients are restored from a device-resident pool (the Nesterov blend overwrites them in
place, muon.py:10) and, for the small workloads, a buffer larger than L2 is written.

At N = 1 the line also carries ``other_configs`` (the three small benchmark configurations: one
768x3072 matrix, GPT-2-small hidden weights with aux Adam, batched conv filters, a few ms each;
with the default workload also two layers of Llama-3-70B shapes and the default workload under the
classic Frobenius-normalised iteration, three timed steps each) and
``reference_gpu``: step times of the unmodified reference (its torch.compile'd driver over its
autotuned Triton kernels) on a B200, either measured in this run (``--reference-gpu live``, needs
the reference installed under baseline/_ref and takes minutes to compile and autotune) or as
recorded by tests/golden/make_reference_b200.py (default).

Prints ONE JSON line on rank 0. ``--impl reference`` times the CPU restatement of the reference's
algorithm (the reference's own Newton-Schulz kernels need a GPU and Triton) on the host cores,
on a bounded sample of the same workload, and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LLAMA3_8B_LAYER = [(4096, 4096), (4096, 4096), (1024, 4096), (1024, 4096),
                   (14336, 4096), (14336, 4096), (4096, 14336)]  # q, o, k, v, gate, up, down
LLAMA3_70B_LAYER = [(8192, 8192), (8192, 8192), (1024, 8192), (1024, 8192),
                    (28672, 8192), (28672, 8192), (8192, 28672)]
GPT2_SMALL_LAYER = [(768, 768)] * 4 + [(3072, 768), (768, 3072)]

WORKLOADS = {
    # name: (shapes, dtype, grad std, description)
    "llama3-8b-hidden": (LLAMA3_8B_LAYER * 32, torch.bfloat16, 1e-3,
                         "Llama-3-8B hidden weights, 224 matrices, bf16"),
    "llama3-8b-4layers": (LLAMA3_8B_LAYER * 4, torch.bfloat16, 1e-3,
                          "Llama-3-8B hidden weights, 4 of 32 layers, bf16 (small case for profiling)"),
    "llama3-70b-2layers": (LLAMA3_70B_LAYER * 2, torch.bfloat16, 1e-3,
                           "Llama-3-70B hidden weights, 2 of 80 layers, bf16 (the full set needs 8 GPUs)"),
    "llama3-70b-40layers": (LLAMA3_70B_LAYER * 40, torch.bfloat16, 1e-3,
                            "Llama-3-70B hidden weights, 40 of 80 layers, bf16 (replicated parameters of all 80 "
                            "layers are 137 GB per GPU; meant for 8 GPUs)"),
    "one-768x3072": ([(768, 3072)], torch.float32, 1.0, "one fp32 768x3072 parameter, grads ~N(0,1)"),
    "gpt2-small-hidden": (GPT2_SMALL_LAYER * 12, torch.float32, 1e-2,
                          "GPT-2 small hidden weights, 72 matrices, fp32"),
    "conv-filters": ([(256, 256, 3, 3)] * 64 + [(128, 128, 3, 3)] * 64, torch.float32, 1.0,
                     "conv filters, 64 x 256x256x3x3 + 64 x 128x128x3x3, fp32"),
}
# the reference's live algorithm / its commented block / the live algorithm with e4m3 Gram products
NS_ITERS = {"aol4": 4, "classic5": 5, "aol4_fp8": 4}
# The three small benchmark configurations, reported under `other_configs` at N = 1:
# name -> (workload, optimizer class, number of 768-element gain vectors given to Adam,
#          lower bound in ms at the measured peaks: NS FLOPs at the burst GEMM rate + elementwise
#          bytes at the copy bandwidth)
SMALL_CONFIGS = {
    "one-768x3072": ("one-768x3072", "SingleDeviceMuon", 0, 0.03),
    "gpt2-small-hidden": ("gpt2-small-hidden", "MuonWithAuxAdam", 25, 0.91),
    "conv-filters": ("conv-filters", "SingleDeviceMuon", 0, 0.28),
}
# Two more entries of `other_configs` when the default workload runs on one GPU, three timed steps
# each: the Llama-3-70B shapes as far as one GPU holds them beside the main workload's leftovers
# (2 of 80 layers), and the main workload with the classic Frobenius-normalised iteration
# (name -> (workload, optimizer class, gain vectors, lower bound or None, NS mode or None = current)).
LARGE_CONFIGS = {
    "llama3-70b-2layers": ("llama3-70b-2layers", "SingleDeviceMuon", 0, None, None),
    "llama3-8b-hidden/classic5": ("llama3-8b-hidden", "SingleDeviceMuon", 0, None, "classic5"),
}
# DRAM bytes (read + write) per matrix element that one launch of the line-3 kernel moved in an ncu
# capture of that kernel on 8 matrices of 4096 x 14336: 2.120 GB read + 0.925 GB written (a later
# capture on 4 matrices gives the same bytes per element). Traffic of that kernel grows with the
# elements a launch covers.
LINE3_DRAM_BYTES_PER_ELEMENT = 3.045e9 / (8 * 4096 * 14336)


def as_matrices(shapes):
    """(rows, cols) each parameter presents to the iteration: 4-D filters collapse to [O, I*kH*kW]."""
    out = []
    for s in shapes:
        cols = 1
        for d in s[1:]:
            cols *= d
        out.append((s[0], cols))
    return out


def ns_flops(shapes, iters=4):
    """(symmetry-reduced, dense-equivalent) Newton-Schulz FLOPs of one step."""
    red = dense = 0.0
    for r, c in shapes:
        m, n = min(r, c), max(r, c)
        red += iters * (m * (m + 1) * n + m * m * (m + 1) + 2 * m * m * n)
        dense += iters * (4 * m * m * n + 2 * m ** 3)
    return red, dense


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm_gbs=d["hbm_gbs"], tflops_burst=d["bf16_tflops"],
                    tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self._stop, self._thread = index, [], threading.Event(), None

    def _run(self):
        try:
            proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        try:
            while not self._stop.is_set():
                line = proc.stdout.readline()
                if not line:
                    break
                parts = [x.strip() for x in line.split(",")]
                if len(parts) == 6 and parts[0].isdigit():
                    self.samples.append(parts)
        finally:
            proc.terminate()

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": statistics.median(int(s[0]) for s in self.samples),
                "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons, "samples": len(self.samples)}


# --------------------------------------------------------------------------------- ours
def cpus_near_gpu(index):
    """CPUs of the NUMA node the GPU hangs off (from sysfs), or None when that cannot be told.
    Pinned host buffers allocated by a thread running there are local to the GPU's PCIe root, so
    host-to-device copies do not cross the socket interconnect."""
    try:
        props = torch.cuda.get_device_properties(index)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        return (node, cpus) if cpus else None
    except Exception:
        return None


def make_problem(shapes, dtype, device):
    """Parameters for every matrix (replicated on every rank). Seeds depend on the matrix index
    only, so the data does not depend on the world size."""
    params = []
    for i, s in enumerate(shapes):
        g = torch.Generator(device=device).manual_seed(4000 + i)
        p = torch.empty(s, dtype=dtype, device=device).normal_(0, 0.02, generator=g)
        params.append(torch.nn.Parameter(p))
    return params


def fill_grads(opt_params, dtype, grad_std, rank, world, device):
    """Gradients only for the parameters this rank owns (the distributed step never reads the
    others, muon.py:57-65). Returns the owned parameters and a pool holding a copy of every
    gradient, from which the gradients are restored between timed steps."""
    owned, pool = [], []
    for idx, p in enumerate(opt_params):
        if idx % world == rank:
            g = torch.Generator(device=device).manual_seed(9000 + idx)
            p.grad = torch.empty(p.shape, dtype=dtype, device=device).normal_(0, grad_std, generator=g)
            owned.append(p)
            pool.append(p.grad.clone())
    return owned, pool


def timed_steps(step, n_steps, device, barrier, outside=None, world=1):
    """Mean device time (ms) of `n_steps` calls of `step`, each bracketed by its own CUDA events on
    the current stream; `outside` runs before every step, outside the timed interval. A barrier and
    a device synchronisation bracket the loop; the per-rank sum is reduced with MAX over ranks."""
    barrier()
    events = []
    for _ in range(n_steps):
        if outside is not None:
            outside()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        step()
        t1.record()
        events.append((t0, t1))
    barrier()
    total = torch.tensor([sum(a.elapsed_time(b) for a, b in events)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(total, op=dist.ReduceOp.MAX)
    return float(total.item()) / n_steps


def run_small_config(name, device, ns_mode, steps=20, warmup=3):
    """One of the other benchmark configurations on one GPU: ms per step (device time, L2
    flushed and gradients restored before every step), kernel launches per step, NS TFLOP/s over
    the step, and the host time it takes to issue a step."""
    import muon_b200
    from muon_b200 import _lib
    if name in SMALL_CONFIGS:
        workload, cls_name, n_gains, lower_ms = SMALL_CONFIGS[name]
        own_mode = None
    else:
        workload, cls_name, n_gains, lower_ms, own_mode = LARGE_CONFIGS[name]
    if own_mode is not None:
        previous_mode = muon_b200.get_ns_mode()
        muon_b200.set_ns_mode(own_mode)
        ns_mode = own_mode
    shapes, dtype, grad_std, desc = WORKLOADS[workload]
    params = make_problem(shapes, dtype, device)
    gains = [torch.nn.Parameter(torch.ones(768, device=device)) for _ in range(n_gains)]
    if cls_name == "MuonWithAuxAdam":
        opt = muon_b200.MuonWithAuxAdam([
            dict(params=list(params), use_muon=True, lr=0.02, weight_decay=0.01, momentum=0.95),
            dict(params=gains, use_muon=False, lr=3e-4, betas=(0.9, 0.95), eps=1e-10, weight_decay=0)])
    else:
        opt = muon_b200.SingleDeviceMuon(list(params), lr=0.02, weight_decay=0.01, momentum=0.95)
    owned, pool = fill_grads(params, dtype, grad_std, 0, 1, device)
    for gvec in gains:
        gvec.grad = torch.full_like(gvec, 1e-2)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def outside():
        for p, g in zip(owned, pool):
            p.grad.copy_(g)
        flush.zero_()

    def sync():
        torch.cuda.synchronize()

    for _ in range(warmup):
        outside()
        opt.step()
    counts0 = _lib.launch_counts()
    ms = timed_steps(opt.step, steps, device, sync, outside)
    counts1 = _lib.launch_counts()
    # host time to issue one step with the device idle at the start and nothing waited for
    sync()
    t0 = time.perf_counter()
    for _ in range(steps):
        opt.step()
    host_ms = (time.perf_counter() - t0) * 1e3 / steps
    sync()
    red, dense = ns_flops(as_matrices(shapes), NS_ITERS[ns_mode])
    out = {"description": desc + (f" + {n_gains} gain vectors through Adam" if n_gains else ""),
           "optimizer": cls_name, "ms_per_step": ms, "steps": steps,
           "gpu_launches_per_step": (sum(counts1.values()) - sum(counts0.values())) / steps,
           "ns_tflops_step": red / (ms * 1e-3) / 1e12, "host_issue_ms_per_step": host_ms,
           "lower_bound_ms": lower_ms, "l2_policy": "256 MB written between timed steps"}
    if own_mode is not None:
        out["ns_mode"] = own_mode
        muon_b200.set_ns_mode(*previous_mode)
    del opt, params, gains, owned, pool, flush
    muon_b200.get_backend().release_workspaces()
    torch.cuda.empty_cache()
    return out


def recorded_reference_gpu():
    """Step times of the unmodified reference on a B200 as recorded by
    tests/golden/make_reference_b200.py (committed beside the fixtures it writes)."""
    path = os.path.join(ROOT, "tests", "golden", "reference_b200_report.json")
    if not os.path.exists(path):
        return {"unavailable": "no recorded run (tests/golden/reference_b200_report.json is missing)"}
    rep = json.load(open(path))
    out = {"source": "recorded by tests/golden/make_reference_b200.py on a B200 (not measured in this run)",
           "step_ms": {k: v["reference_ms"] for k, v in rep.get("step_times", {}).items()},
           "this_library_step_ms_in_that_run": {k: v["ours_ms"] for k, v in rep.get("step_times", {}).items()},
           "ns_per_matrix": [{"shape": c["shape"], "reference_ms": c["reference_ms"],
                              "reference_ns_tflops": c["reference_tflops_sym"]} for c in rep.get("cases", [])]}
    layer = rep.get("step_times", {}).get("llama3-8b-1layer")
    if layer:
        out["llama3-8b-hidden_step_ms_extrapolated"] = layer["reference_ms"] * 32
        out["extrapolation"] = "one Llama-3-8B layer (7 matrices) x 32"
    return out


def live_reference_gpu(workload, device):
    """The unmodified reference (baseline/_ref/muon.py: torch.compile'd driver, autotuned Triton
    kernels) timed in this run with CUDA events on one GPU. Llama workloads are sampled: one layer,
    scaled by the number of layers."""
    import importlib.util
    path = os.path.join(ROOT, "baseline", "_ref", "muon.py")
    if not os.path.exists(path):
        return {"unavailable": "baseline/_ref/muon.py is not installed"}
    import torch._dynamo
    torch._dynamo.config.cache_size_limit = 256
    if hasattr(torch._dynamo.config, "recompile_limit"):
        torch._dynamo.config.recompile_limit = 256
    spec = importlib.util.spec_from_file_location("muon_reference", path)
    ref = importlib.util.module_from_spec(spec)
    sys.modules["muon_reference"] = ref
    spec.loader.exec_module(ref)
    shapes, dtype, grad_std, _ = WORKLOADS[workload]
    scale, text = 1.0, "the whole workload"
    if workload.startswith("llama3-8b"):
        scale, shapes, text = len(shapes) / 7, list(LLAMA3_8B_LAYER), "one Llama-3-8B layer, scaled by the layer count"
    elif workload.startswith("llama3-70b"):
        scale, shapes, text = len(shapes) / 7, list(LLAMA3_70B_LAYER), "one Llama-3-70B layer, scaled by the layer count"
    params = make_problem(shapes, dtype, device)
    opt = ref.SingleDeviceMuon(params, lr=0.02, weight_decay=0.01, momentum=0.95)
    fill_grads(params, dtype, grad_std, 0, 1, device)
    t0 = time.perf_counter()
    for _ in range(2):  # compile + autotune, then one warm step
        opt.step()
    torch.cuda.synchronize()
    warm_s = time.perf_counter() - t0
    ms = timed_steps(opt.step, 5, device, torch.cuda.synchronize)
    red, _ = ns_flops(as_matrices(shapes))
    return {"source": "measured in this run", "step_ms": ms * scale, "sample": text,
            "ns_tflops_step": red / (ms * 1e-3) / 1e12, "compile_and_autotune_s": warm_s}


def run_ours(args):
    import muon_b200
    from muon_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        import datetime
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device,
                                timeout=datetime.timedelta(seconds=120))

    comm_sms = int(os.environ.get("MUON_B200_COMM_SMS", "0"))
    if world > 1 and comm_sms > 0:
        _lib.check(_lib.lib.muon_b200_set_reserved_sms(comm_sms))
    muon_b200.set_ns_mode(args.ns_mode)
    iters = NS_ITERS[args.ns_mode]

    shapes, dtype, grad_std, desc = WORKLOADS[args.workload]
    mats = as_matrices(shapes)
    elements = sum(r * c for r, c in mats)
    params = make_problem(shapes, dtype, device)
    opt = muon_b200.Muon(list(params), lr=0.02, weight_decay=0.01, momentum=0.95)
    sorted_params = opt.param_groups[0]["params"]
    owned, pool = fill_grads(sorted_params, dtype, grad_std, rank, world, device)
    small = elements * params[0].element_size() * 3 < (1 << 30)  # parameters + gradients + momentum
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device) if small else None

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def restore():
        for p, g in zip(owned, pool):
            p.grad.copy_(g)
        if flush is not None:
            flush.zero_()

    for _ in range(args.warmup):
        restore()
        opt.step()
    barrier()

    # ---- device-resident steps (headline `value`) ----
    counts0 = _lib.launch_counts()
    with ClockSampler(local_rank) as clocks:
        ms_per_step = timed_steps(opt.step, args.steps, device, barrier, restore, world)
    counts1 = _lib.launch_counts()
    launches = sum(counts1.values()) - sum(counts0.values())

    # ---- the same steps again with every kernel bracketed by events (roofline) ----
    # In this pass the elementwise stages are not overlapped with the GEMMs of another launch
    # group, so that every kernel's duration is its own (co-running kernels stretch each other).
    backend = muon_b200.get_backend()
    overlap = backend.overlap_elementwise
    backend.overlap_elementwise = False
    _lib.timing_enable(True)
    timed_steps(opt.step, args.steps, device, barrier, restore, world)
    _lib.timing_enable(False)
    backend.overlap_elementwise = overlap
    per_kind = _lib.timing_collect()

    # ---- end to end: gradients arrive from pinned host memory, a scalar goes back ----
    # one pinned buffer per gradient, allocated from a CPU of the GPU's NUMA node where that is known
    allowed = os.sched_getaffinity(0)
    near = cpus_near_gpu(local_rank)
    numa_note = "NUMA node of the GPU unknown: buffers allocated wherever the process ran"
    if near is not None and near[1] & allowed:
        os.sched_setaffinity(0, near[1] & allowed)
        numa_note = f"buffers allocated on NUMA node {near[0]}, the GPU's"
    try:
        pinned = [g.to("cpu").pin_memory() for g in pool]
    finally:
        os.sched_setaffinity(0, allowed)
    h2d_bytes = sum(g.numel() * g.element_size() for g in pool)
    result_host = torch.zeros(1, dtype=torch.float32).pin_memory()
    probe = sorted_params[0]
    copy_stream = torch.cuda.Stream(device=device)

    def e2e_step():
        # The gradients come in on a copy stream, in the order the optimizer consumes them, each
        # marked with its own event: step() starts on the first ones while the rest are in flight.
        copy_stream.wait_stream(torch.cuda.current_stream())  # the previous step has read them
        with torch.cuda.stream(copy_stream):
            for p, h in zip(owned, pinned):
                p.grad.copy_(h, non_blocking=True)
                muon_b200.mark_grad_ready(p)
        opt.step()
        result_host.copy_(probe.detach().view(-1)[:1].float(), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_step()  # page the pinned buffers in
    e2e_ms = timed_steps(e2e_step, args.steps, device, barrier,
                         (lambda: flush.zero_()) if flush is not None else None, world)

    status = muon_b200.device_status()
    h2d = torch.tensor([float(h2d_bytes)], device=device)
    dist.all_reduce(h2d)
    del pinned

    other_configs, reference_gpu = None, None
    if world == 1 and rank == 0 and not args.no_other_configs:
        del opt, params, sorted_params, owned, pool, probe
        backend.release_workspaces()
        torch.cuda.empty_cache()
        other_configs = {name: run_small_config(name, device, args.ns_mode) for name in SMALL_CONFIGS
                         if SMALL_CONFIGS[name][0] != args.workload}
        if args.workload == "llama3-8b-hidden":
            for name, cfg in LARGE_CONFIGS.items():
                if cfg[4] is None or cfg[4] != args.ns_mode:
                    other_configs[name] = run_small_config(name, device, args.ns_mode, steps=3, warmup=3)
        reference_gpu = live_reference_gpu(args.workload, device) if args.reference_gpu == "live" \
            else recorded_reference_gpu()

    if rank == 0:
        peaks = load_peaks()
        red, dense = ns_flops(mats, iters)
        ms3, work3, n3 = per_kind["ns_line3"]
        ns_ms = sum(per_kind[k][0] for k in ("ns_line1", "ns_line2", "ns_line3"))
        ns_work = sum(per_kind[k][1] for k in ("ns_line1", "ns_line2", "ns_line3"))
        achieved = work3 / (ms3 * 1e-3) / 1e12 if ms3 > 0 else None
        peak = peaks["tflops_sustained"]
        kernels = {k: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[2] / args.steps,
                       "rate": (v[1] / (v[0] * 1e-3) / (1e12 if k.startswith("ns_") else 1e9)) if v[0] > 0 else None,
                       "unit": "TFLOP/s" if k.startswith("ns_") else "GB/s"}
                   for k, v in per_kind.items() if v[2] > 0}
        clock = clocks.summary()
        line = {
            "metric": "muon_step_ms", "value": ms_per_step, "unit": "ms", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": args.workload, "description": desc, "matrices": len(shapes),
                       "elements": elements, "param_dtype": str(dtype).split(".")[-1],
                       "ns_mode": args.ns_mode, "ns_iters": iters, "parallelism": f"muon-round-robin-dp{world}",
                       "l2_policy": ("256 MB written between timed steps" if small else
                                     "inputs (>= 14 GB per step at full size) are larger than the 126 MB L2"),
                       "gradients": "restored from a device-resident pool before every step, outside the "
                                    "timed intervals (each step has its own pair of CUDA events)"},
            "steps_per_s": 1e3 / ms_per_step,
            # the same step normalised by the SM clock it ran at (the device is power-capped and the
            # clock differs from GPU to GPU): compare this across runs rather than ms
            "ms_x_sm_mhz": ms_per_step * clock["sm_mhz"] if clock.get("sm_mhz") else None,
            "ns_tflops_step": red / (ms_per_step * 1e-3) / 1e12,
            "ns_tflops_step_dense_equiv": dense / (ms_per_step * 1e-3) / 1e12,
            "ns_tflops_kernels": ns_work / (ns_ms * 1e-3) / 1e12 if ns_ms > 0 else None,
            "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": int(h2d.item()),
                    "d2h_bytes_per_step": 4,
                    "note": "one pinned host buffer per gradient (" + numa_note + "); copies on a copy stream, "
                            "each gradient marked ready"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "kernel": "ns_gemm_kernel<MODE_BX> (line 3: a*X + B*X)",
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": (achieved / peak) if achieved else None,
                         "peak_kind": f"{peaks['source']} bf16 GEMM, sustained (kernel timed inside a long step); "
                                      f"burst figure is {peaks['tflops_burst']}",
                         "launches": int(n3), "avg_launch_ms": ms3 / n3 if n3 else None,
                         # average DRAM bytes per launch, scaled from the ncu capture by elements covered
                         "traffic": (LINE3_DRAM_BYTES_PER_ELEMENT * elements * iters
                                     / world / (n3 / args.steps)) if n3 and args.workload.startswith("llama3-8b") else None,
                         "traffic_algorithmic": ((2 * elements + sum(min(r, c) ** 2 for r, c in mats))
                                                 * 2 * iters / world / (n3 / args.steps)) if n3 else None,
                         "rank": 0},
            "kernels": kernels,
            "kernels_note": "per-kernel CUDA-event times from a second pass over the same steps with the "
                            "elementwise stages serialised behind the GEMMs (the timed `value` overlaps them)",
            "overlap_elementwise": bool(overlap),
            "clocks": clock,
            "device_status": status,
        }
        if other_configs is not None:
            line["other_configs"] = other_configs
        if reference_gpu is not None:
            line["reference_gpu"] = reference_gpu
        print(json.dumps(line), flush=True)
    barrier()
    dist.destroy_process_group()


# --------------------------------------------------------------------------- reference
def cpu_sample_step(shapes_sample, dtype, grad_std, threads, ns_mode="aol4"):
    """One oracle Muon step over the sample matrices on the host cores; returns seconds."""
    import functools
    from oracle import muon_oracle as orc
    torch.set_num_threads(threads)
    ns = {"aol4": orc.zeropower_via_newtonschulz5, "aol4_fp8": orc.zeropower_aol4_fp8,
          "classic5": functools.partial(orc.zeropower_classic5, fused=True)}[ns_mode]
    items = []
    for i, s in enumerate(shapes_sample):
        g = torch.Generator().manual_seed(4000 + i)
        p = (torch.randn(s, generator=g) * 0.02).to(dtype)
        gr = (torch.randn(s, generator=g) * grad_std).to(dtype)
        items.append((p, gr, torch.zeros_like(p)))
    t0 = time.perf_counter()
    for p, gr, m in items:
        orc.muon_param_step(p, gr, m, 0.02, 0.01, 0.95, ns=ns)
    return time.perf_counter() - t0


def reference_sample(workload):
    shapes, dtype, grad_std, _ = WORKLOADS[workload]
    if workload.startswith("llama3"):
        sample = list(LLAMA3_8B_LAYER)
        text = "one Llama-3-8B layer (7 matrices; 1 of the 32); scaled to the full step by NS FLOPs"
    elif workload == "one-768x3072":
        sample, text = [(768, 3072)], "the whole workload (one matrix)"
    else:
        sample = [(768, 768)] * 4 + [(3072, 768), (768, 3072)]
        text = "one GPT-2 small layer (6 matrices); scaled to the full step by NS FLOPs"
    scale = ns_flops(as_matrices(shapes))[1] / ns_flops(sample)[1]
    return sample, dtype, grad_std, scale, text


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    shapes, dtype, _, desc = WORKLOADS[args.workload]
    sample, dtype, grad_std, scale, text = reference_sample(args.workload)
    threads = os.cpu_count() or 1
    warm = max(0, min(args.warmup, 1))
    for _ in range(warm):
        cpu_sample_step(sample, dtype, grad_std, threads, args.ns_mode)
    # As many sampled steps as asked for, within about two minutes of host time.
    times, t_begin = [], time.perf_counter()
    while len(times) < max(1, args.steps) and (not times or time.perf_counter() - t_begin < 120):
        times.append(cpu_sample_step(sample, dtype, grad_std, threads, args.ns_mode))
    ms = statistics.median(times) * 1e3 * scale
    line = {
        "impl": "reference", "metric": "muon_step_ms", "value": ms, "unit": "ms", "n_gpus": args.gpus,
        "steps": len(times), "warmup": warm, "ms_per_step": ms, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "description": desc, "matrices": len(shapes),
                   "elements": sum(r * c for r, c in as_matrices(shapes)),
                   "param_dtype": str(dtype).split(".")[-1], "ns_mode": args.ns_mode,
                   "ns_iters": NS_ITERS[args.ns_mode], "parallelism": "host cores"},
        "cpu_baseline": {"value": ms, "unit": "ms", "cores": threads, "kind": "port",
                         "sample": text + f" (x{scale:.1f}); oracle restatement of muon.py on torch CPU; "
                                          f"{len(times)} sampled steps (of {args.steps} asked for) in "
                                          f"{time.perf_counter() - t_begin:.0f} s"},
        "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's own NS kernels are Triton GPU kernels and cannot run on host cores; "
                "this is the CPU restatement (oracle) of the same algorithm",
    }
    print(json.dumps(line), flush=True)


def attach_cpu_baseline(args, line):
    sample, dtype, grad_std, scale, text = reference_sample(args.workload)
    threads = os.cpu_count() or 1
    t = cpu_sample_step(sample, dtype, grad_std, threads, args.ns_mode)
    line["cpu_baseline"] = {"value": t * 1e3 * scale, "unit": "ms", "cores": threads, "kind": "port",
                            "sample": text + f" (x{scale:.1f}); one timed pass of {t:.1f} s"}
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="llama3-8b-hidden")
    ap.add_argument("--ns-mode", choices=sorted(NS_ITERS), default="aol4",
                    help="aol4: the algorithm the reference executes; classic5: the Frobenius-normalised "
                         "quintic iteration of its commented block (1.25x the NS FLOPs); aol4_fp8: aol4 with "
                         "the symmetric products of iterations 2..4 on e4m3 operands")
    ap.add_argument("--reference-gpu", choices=["recorded", "live"], default="recorded",
                    help="live: time the unmodified reference from baseline/_ref on this GPU (minutes)")
    ap.add_argument("--no-other-configs", action="store_true",
                    help="skip the three small configurations and the reference_gpu key")
    ap.add_argument("--no-cpu-baseline", action="store_true",
                    help="skip the host-core baseline leg (it takes tens of seconds)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.gpus == 1 and not args.no_cpu_baseline:
        # Capture our JSON line, add the CPU baseline measured in the same run, print once.
        import contextlib
        import io
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            run_ours(args)
        out = buf.getvalue().strip().splitlines()
        line = json.loads(out[-1])
        print(json.dumps(attach_cpu_baseline(args, line)), flush=True)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
