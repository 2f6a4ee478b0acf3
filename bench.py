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
    "gpt2-small-hidden": (GPT2_SMALL_LAYER * 12, torch.float32, 1e-2,
                          "GPT-2 small hidden weights, 72 matrices, fp32"),
    "conv-filters": ([(256, 256, 3, 3)] * 64 + [(128, 128, 3, 3)] * 64, torch.float32, 1.0,
                     "conv filters, 64 x 256x256x3x3 + 64 x 128x128x3x3, fp32"),
}
NS_ITERS = 4  # the reference's live algorithm
# DRAM bytes (read + write) per matrix element that one launch of the line-3 kernel moved in the
# ncu capture summarised in profiles/ns_gemm_line3_llama3-8b-4layers.md: 2.120 GB read + 0.925 GB
# written for 8 matrices of 4096 x 14336. Traffic of that kernel grows with the elements a launch
# covers.
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


def ns_flops(shapes, iters=NS_ITERS):
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
def make_problem(shapes, dtype, grad_std, device, rank, world):
    """Parameters for every matrix (replicated), gradients only for the ones this rank owns
    (the distributed step never reads the others, muon.py:57-65). Seeds depend on the matrix
    index only, so the data does not depend on the world size."""
    params = []
    for i, s in enumerate(shapes):
        g = torch.Generator(device=device).manual_seed(4000 + i)
        p = torch.empty(s, dtype=dtype, device=device).normal_(0, 0.02, generator=g)
        params.append(torch.nn.Parameter(p))
    return params


def fill_grads(opt_params, dtype, grad_std, rank, world, device):
    owned = []
    for idx, p in enumerate(opt_params):
        if idx % world == rank:
            g = torch.Generator(device=device).manual_seed(9000 + idx)
            p.grad = torch.empty(p.shape, dtype=dtype, device=device).normal_(0, grad_std, generator=g)
            owned.append(p)
    return owned


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

    shapes, dtype, grad_std, desc = WORKLOADS[args.workload]
    mats = as_matrices(shapes)
    params = make_problem(shapes, dtype, grad_std, device, rank, world)
    opt = muon_b200.Muon(list(params), lr=0.02, weight_decay=0.01, momentum=0.95)
    sorted_params = opt.param_groups[0]["params"]
    owned = fill_grads(sorted_params, dtype, grad_std, rank, world, device)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(n_steps, before_step=None, after_step=None):
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n_steps):
            if before_step:
                before_step()
            opt.step()
            if after_step:
                after_step()
        t1.record()
        barrier()
        ms = torch.tensor([t0.elapsed_time(t1)], device=device)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / n_steps

    for _ in range(args.warmup):
        opt.step()
    barrier()

    # ---- device-resident steps (headline `value`) ----
    counts0 = _lib.launch_counts()
    with ClockSampler(local_rank) as clocks:
        ms_per_step = timed(args.steps)
    counts1 = _lib.launch_counts()
    launches = sum(counts1.values()) - sum(counts0.values())

    # ---- the same steps again with every kernel bracketed by events (roofline) ----
    # In this pass the elementwise stages are not overlapped with the GEMMs of another launch
    # group, so that every kernel's duration is its own (co-running kernels stretch each other).
    backend = muon_b200.get_backend()
    overlap = backend.overlap_elementwise
    backend.overlap_elementwise = False
    _lib.timing_enable(True)
    timed(args.steps)
    _lib.timing_enable(False)
    backend.overlap_elementwise = overlap
    per_kind = _lib.timing_collect()

    # ---- end to end: gradients arrive from pinned host memory, a scalar goes back ----
    pinned = {}
    for p in owned:
        key = tuple(p.shape)
        if key not in pinned:
            pinned[key] = p.grad.detach().to("cpu").pin_memory()
    h2d_bytes = sum(p.grad.numel() * p.grad.element_size() for p in owned)
    result_host = torch.zeros(1, dtype=torch.float32).pin_memory()
    probe = sorted_params[0]

    copy_stream = torch.cuda.Stream(device=device)

    def copy_in():
        # The gradients come in on a copy stream, in the order the optimizer consumes them, each
        # marked with its own event: step() starts on the first ones while the rest are in flight.
        copy_stream.wait_stream(torch.cuda.current_stream())  # the previous step has read them
        with torch.cuda.stream(copy_stream):
            for p in owned:
                p.grad.copy_(pinned[tuple(p.shape)], non_blocking=True)
                muon_b200.mark_grad_ready(p)

    def read_back():
        result_host.copy_(probe.detach().view(-1)[:1].float(), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_ms = timed(args.steps, before_step=copy_in, after_step=read_back)

    status = muon_b200.device_status()
    h2d = torch.tensor([float(h2d_bytes)], device=device)
    dist.all_reduce(h2d)

    if rank == 0:
        peaks = load_peaks()
        red, dense = ns_flops(mats)
        ms3, work3, n3 = per_kind["ns_line3"]
        ns_ms = sum(per_kind[k][0] for k in ("ns_line1", "ns_line2", "ns_line3"))
        ns_work = sum(per_kind[k][1] for k in ("ns_line1", "ns_line2", "ns_line3"))
        achieved = work3 / (ms3 * 1e-3) / 1e12 if ms3 > 0 else None
        peak = peaks["tflops_sustained"]
        kernels = {k: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[2] / args.steps,
                       "rate": (v[1] / (v[0] * 1e-3) / (1e12 if k.startswith("ns_") else 1e9)) if v[0] > 0 else None,
                       "unit": "TFLOP/s" if k.startswith("ns_") else "GB/s"}
                   for k, v in per_kind.items() if v[2] > 0}
        line = {
            "metric": "muon_step_ms", "value": ms_per_step, "unit": "ms", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": args.workload, "description": desc, "matrices": len(shapes),
                       "elements": sum(r * c for r, c in mats), "param_dtype": str(dtype).split(".")[-1],
                       "ns_mode": "aol4", "ns_iters": NS_ITERS, "parallelism": f"muon-round-robin-dp{world}",
                       "l2_policy": "inputs (>= 14 GB per step at full size) are larger than the 126 MB L2"},
            "steps_per_s": 1e3 / ms_per_step,
            "ns_tflops_step": red / (ms_per_step * 1e-3) / 1e12,
            "ns_tflops_step_dense_equiv": dense / (ms_per_step * 1e-3) / 1e12,
            "ns_tflops_kernels": ns_work / (ns_ms * 1e-3) / 1e12 if ns_ms > 0 else None,
            "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": int(h2d.item()),
                    "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "kernel": "ns_gemm_kernel<MODE_BX> (line 3: a*X + B*X)",
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": (achieved / peak) if achieved else None,
                         "peak_kind": f"{peaks['source']} bf16 GEMM, sustained (kernel timed inside a long step); "
                                      f"burst figure is {peaks['tflops_burst']}",
                         "launches": int(n3), "avg_launch_ms": ms3 / n3 if n3 else None,
                         # average DRAM bytes per launch, scaled from the ncu capture by elements covered
                         "traffic": (LINE3_DRAM_BYTES_PER_ELEMENT * sum(r * c for r, c in mats) * NS_ITERS
                                     / world / (n3 / args.steps)) if n3 and args.workload.startswith("llama3-8b") else None,
                         "traffic_algorithmic": ((2 * sum(r * c for r, c in mats) + sum(min(r, c) ** 2 for r, c in mats))
                                                 * 2 * NS_ITERS / world / (n3 / args.steps)) if n3 else None,
                         "rank": 0},
            "kernels": kernels,
            "kernels_note": "per-kernel CUDA-event times from a second pass over the same steps with the "
                            "elementwise stages serialised behind the GEMMs (the timed `value` overlaps them)",
            "overlap_elementwise": bool(overlap),
            "clocks": clocks.summary(),
            "device_status": status,
        }
        print(json.dumps(line), flush=True)
    barrier()
    dist.destroy_process_group()


# --------------------------------------------------------------------------- reference
def cpu_sample_step(shapes_sample, dtype, grad_std, threads):
    """One oracle Muon step over the sample matrices on the host cores; returns seconds."""
    from oracle import muon_oracle as orc
    torch.set_num_threads(threads)
    items = []
    for i, s in enumerate(shapes_sample):
        g = torch.Generator().manual_seed(4000 + i)
        p = (torch.randn(s, generator=g) * 0.02).to(dtype)
        gr = (torch.randn(s, generator=g) * grad_std).to(dtype)
        items.append((p, gr, torch.zeros_like(p)))
    t0 = time.perf_counter()
    for p, gr, m in items:
        orc.muon_param_step(p, gr, m, 0.02, 0.01, 0.95)
    return time.perf_counter() - t0


def reference_sample(workload):
    shapes, dtype, grad_std, _ = WORKLOADS[workload]
    if workload.startswith("llama3"):
        sample = list(LLAMA3_8B_LAYER)
        text = "one Llama-3-8B layer (7 matrices; 1 of the 32); scaled to the full step by NS FLOPs"
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
    for _ in range(min(args.warmup, 1)):
        cpu_sample_step(sample, dtype, grad_std, threads)
    times = [cpu_sample_step(sample, dtype, grad_std, threads) for _ in range(max(1, min(args.steps, 3)))]
    ms = statistics.median(times) * 1e3 * scale
    line = {
        "impl": "reference", "metric": "muon_step_ms", "value": ms, "unit": "ms", "n_gpus": args.gpus,
        "steps": len(times), "warmup": min(args.warmup, 1), "ms_per_step": ms, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "description": desc, "matrices": len(shapes),
                   "elements": sum(r * c for r, c in as_matrices(shapes)),
                   "param_dtype": str(dtype).split(".")[-1], "ns_mode": "aol4", "ns_iters": NS_ITERS,
                   "parallelism": "host cores"},
        "cpu_baseline": {"value": ms, "unit": "ms", "cores": threads, "kind": "port",
                         "sample": text + f" (x{scale:.1f}); oracle restatement of muon.py on torch CPU"},
        "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's own NS kernels are Triton GPU kernels and cannot run on host cores; "
                "this is the CPU restatement (oracle) of the same algorithm",
    }
    print(json.dumps(line), flush=True)


def attach_cpu_baseline(args, line):
    sample, dtype, grad_std, scale, text = reference_sample(args.workload)
    threads = os.cpu_count() or 1
    t = cpu_sample_step(sample, dtype, grad_std, threads)
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
