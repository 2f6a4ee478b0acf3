"""Host-side engine: turns lists of torch tensors into grouped calls of the C ABI.

``CudaBackend`` is the product path. It hands raw device pointers of the callers'
tensors to ``libmuon_b200.so`` on the current CUDA stream; PyTorch is used only to own
memory (the Newton-Schulz workspace is a cached ``torch.uint8`` buffer) and for streams.

Tensors that are not on an sm_100 CUDA device are rejected: there is no CPU path.
The optimizer classes talk to whatever ``get_backend()`` returns, so that their
ownership / windowing logic can be unit-tested on CPU ranks with a stand-in backend
installed by the tests; the package itself never installs anything but ``CudaBackend``.
"""
from __future__ import annotations

import ctypes
import math
from typing import Sequence

import torch
from torch import Tensor

from . import _lib
from ._lib import BF16, F16, F32, F64, NS_AOL4, NS_AOL4_FP8, NS_CLASSIC5, NS_HAVE_SUMSQ, check, i64_array, lib, ptr_array

_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
# element types the cast at the entry of Newton-Schulz accepts (muon.py:760 takes any float dtype)
_NS_INPUT_CODE = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16, torch.float64: F64}
_NS_MODES = {"aol4": NS_AOL4, "classic5": NS_CLASSIC5, "aol4_fp8": NS_AOL4_FP8}

# Module-level Newton-Schulz setting. It cannot be a param-group key: the reference's
# group key sets are asserted exactly (muon.py:148, :155).
_ns_mode = "aol4"
_ns_steps = 0  # 0 = the mode's default (4 for aol4, 5 for classic5)


def set_ns_mode(mode: str = "aol4", steps: int = 0) -> None:
    """Select the Newton-Schulz variant used by every optimizer and by ``muon_update``.

    ``"aol4"`` (default) is the algorithm the reference executes (muon.py:748-799);
    ``"classic5"`` is the Frobenius-normalised quintic iteration of its commented block
    (muon.py:265-291); ``"aol4_fp8"`` is ``"aol4"`` with the two symmetric products of iterations
    2..4 taken in 8-bit floating point (e4m3): faster, about 1e-2 away from ``"aol4"`` in relative
    Frobenius norm on wide and tall matrices, up to 4e-2 on square ones; no counterpart in the
    reference.
    """
    global _ns_mode, _ns_steps
    if mode not in _NS_MODES:
        raise ValueError(f"unknown NS mode {mode!r}; expected one of {sorted(_NS_MODES)}")
    if steps < 0:
        raise ValueError("steps must be >= 0")
    _ns_mode, _ns_steps = mode, int(steps)


def get_ns_mode() -> tuple[str, int]:
    return _ns_mode, _ns_steps


# Gradients that are produced on another stream than the one step() runs on (copied in from
# host memory, reduced by a communication stream, written by a backward stream): the event that
# completes when the gradient holds its value, keyed by the gradient's address.
_grad_ready: dict[int, "torch.cuda.Event"] = {}


def mark_grad_ready(tensor: Tensor, event: "torch.cuda.Event | None" = None) -> None:
    """Tell the engine that `tensor` (a gradient, or a parameter, meaning its ``.grad``) gets its
    value from work enqueued on the CURRENT stream up to this call (or by `event`, if given).

    ``step()`` may then be called from another stream without waiting for that stream: the engine
    makes the first kernel that reads the gradient wait for the event, launch group by launch
    group, so Newton-Schulz of the gradients that arrived first runs while later ones are still
    in flight. Gradients without a mark are assumed ready in the order of step()'s own stream,
    which is the reference's behaviour. A mark is consumed by the step that uses it."""
    if isinstance(tensor, torch.nn.Parameter):
        if tensor.grad is None:
            raise ValueError("mark_grad_ready: the parameter has no gradient yet; allocate p.grad (or pass "
                             "the gradient tensor itself) before marking it")
        g = tensor.grad
    else:
        g = tensor
    _require_cuda(g, "gradient")
    if event is None:
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(g.device))
    _grad_ready[g.data_ptr()] = event


def _wait_grads(stream, grads: Sequence[Tensor]) -> None:
    """Make `stream` wait for the readiness events of `grads` (those that have one)."""
    if not _grad_ready:
        return
    for g in grads:
        ev = _grad_ready.pop(g.data_ptr(), None)
        if ev is not None:
            stream.wait_event(ev)


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"muon_b200: {what} must live on a CUDA (sm_100) device, got device={t.device}; "
            "there is no CPU implementation")


def dtype_code(t: Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise ValueError(f"muon_b200 supports float32, bfloat16 and float16 tensors, got {t.dtype}") from None


def view_2d(shape: Sequence[int]) -> tuple[int, int]:
    """Rows/cols of the matrix the iteration sees: 4-D filters collapse their last three
    dimensions (muon.py:11-12); 2-D tensors are taken as they are."""
    if len(shape) == 2:
        return int(shape[0]), int(shape[1])
    if len(shape) == 4:
        return int(shape[0]), int(shape[1] * shape[2] * shape[3])
    raise ValueError(f"Muon parameters must be 2-D or 4-D, got shape {tuple(shape)}")


def aspect_scale(shape: Sequence[int]) -> float:
    """max(1, size(-2)/size(-1))**0.5 on the gradient's ORIGINAL shape (muon.py:14); for a
    4-D filter that is kH/kW, not rows/cols of the collapsed matrix."""
    return max(1, shape[-2] / shape[-1]) ** 0.5


def tri_tiles(m: int) -> int:
    """Work units of the triangular schedule for an m x m product: 256 x 256 tiles computed
    by CTA pairs when m > 128, one 128 x 256 tile otherwise (mirrors csrc/ns_gemm.cu)."""
    if m <= 128:
        return 1
    t = (m + 255) // 256
    return t * (t + 1) // 2


# A launch ends with one partly filled wave of the 74 CTA pairs of a B200; with this many
# work units per launch that tail costs at most about a twelfth of the launch.
_TARGET_UNITS_PER_LAUNCH = 888


def batch_size_for(m: int, n: int, count: int, workspace_cap_bytes: int) -> int:
    """How many same-shape matrices share one grouped launch: enough work units on the
    triangular products (lines 1 and 2) to amortise the last partial wave, within the
    workspace cap."""
    want = max(1, math.ceil(_TARGET_UNITS_PER_LAUNCH / max(1, tri_tiles(m))))
    per_matrix = 2 * (2 * m * ((n + 7) // 8 * 8) + 2 * m * ((m + 7) // 8 * 8)) + 2048
    fit = max(1, workspace_cap_bytes // per_matrix)
    return max(1, min(count, want, fit))


def plan_launches(m: int, n: int, count: int, workspace_cap_bytes: int, sm_pairs: int = 74) -> list[int]:
    """Split `count` same-shape matrices into grouped launches.

    Every launch of the triangular products ends with a partly filled wave of the `sm_pairs`
    CTA pairs, so the cost of a split is the sum over launches of ceil(units / sm_pairs) waves
    (+ a small per-launch charge). Among balanced splits that fit the workspace cap and do not
    exceed twice the default batch size (launches stay fine-grained enough to overlap the
    exchange in the distributed step), the cheapest one is returned."""
    if count <= 0:
        return []
    units = max(1, tri_tiles(m))
    want = batch_size_for(m, n, count, workspace_cap_bytes)
    per_matrix = 2 * (2 * m * ((n + 7) // 8 * 8) + 2 * m * ((m + 7) // 8 * 8)) + 2048
    max_b = max(1, min(count, 2 * want, workspace_cap_bytes // per_matrix))
    best, best_cost = None, None
    for launches in range(-(-count // max_b), count + 1):
        bounds = [round(i * count / launches) for i in range(launches + 1)]
        sizes = [e - s for s, e in zip(bounds[:-1], bounds[1:])]
        if max(sizes) > max_b:
            continue
        cost = sum(-(-(units * b) // sm_pairs) for b in sizes) + 0.25 * launches
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = sizes, cost
        if launches >= -(-count // max(1, want // 2)):
            break
    return best


def ramped_sizes(sizes: list[int], growth: float = 0.25) -> list[int]:
    """Split the first launch groups of `sizes` into small groups that grow slowly: a group may
    hold one member more than `growth` times everything before it (1, 1, 1, 1, 2, 2, 3, 3, 4, 5,
    6, 8, ...), never more than the planned group it comes from.

    Used when the gradients of a same-shape set are still arriving one after the other (copied in
    from host memory, say): a group's kernels wait for all its gradients, so with groups that
    double, each group waits for a transfer twice as long as the work that is meant to hide it.
    With growth g the transfer of group i is hidden behind the work of the groups before it as
    long as one gradient arrives at most (1 + g) times faster than it is consumed; measured on the
    Llama-shaped step, a 117 MB gradient takes 2.1 ms over PCIe and 2.75 ms to orthogonalise."""
    count, cap = sum(sizes), max(sizes)
    out, total = [], 0
    while total < count and 1 + int(growth * total) < cap:
        take = min(count - total, 1 + int(growth * total))
        out.append(take)
        total += take
    left = count - total
    if left > 0:  # the rest in balanced groups of at most `cap`
        groups = -(-left // cap)
        cuts = [round(i * left / groups) for i in range(groups + 1)]
        out.extend(e - s for s, e in zip(cuts[:-1], cuts[1:]))
    return out


class CudaBackend:
    """Calls the sm_100a library. One instance per process; workspaces cached per device."""

    name = "cuda"

    def __init__(self, workspace_cap_bytes: int = 4 << 30):
        self.workspace_cap_bytes = workspace_cap_bytes
        self._workspaces: dict[tuple[int, int, int], Tensor] = {}
        self._side_streams: dict[int, torch.cuda.Stream] = {}
        self.launch_groups = 0  # grouped C-ABI calls issued (for accounting)
        # Run prologue/epilogue of one launch group beside the GEMMs of another (see
        # _muon_step_pipelined). MUON_B200_OVERLAP=0 switches it off.
        import os
        self.overlap_elementwise = os.environ.get("MUON_B200_OVERLAP", "1") not in ("0", "false", "no")

    # -- memory ------------------------------------------------------------------------
    def workspace(self, device: torch.device, nbytes: int, slot: int = 0) -> Tensor:
        """uint8 buffer >= nbytes, private to (device, current stream, slot)."""
        key = (device.index if device.index is not None else torch.cuda.current_device(),
               _stream_ptr(device), slot)
        buf = self._workspaces.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(nbytes + 256, dtype=torch.uint8, device=device)
            self._workspaces[key] = buf
        return buf

    @staticmethod
    def _sm_pairs(device: torch.device) -> int:
        return max(1, torch.cuda.get_device_properties(device).multi_processor_count // 2)

    @staticmethod
    def _aligned_ptr(buf: Tensor) -> int:
        return (buf.data_ptr() + 255) & ~255

    def release_workspaces(self) -> None:
        self._workspaces.clear()

    # -- Muon --------------------------------------------------------------------------
    def muon_step(self, params: Sequence[Tensor], grads: Sequence[Tensor], moms: Sequence[Tensor],
                  lr: float, weight_decay: float, beta: float, nesterov: bool = True,
                  after_group=None, max_group: int | None = None, peer_ptrs=None) -> None:
        """prologue -> Newton-Schulz -> update for same-shape, same-dtype parameters (one set of
        `muon_step_sets`)."""
        self.muon_step_sets([(params, grads, moms)], lr, weight_decay, beta, nesterov, after_group,
                            max_group=max_group, peer_ptrs=peer_ptrs)

    def muon_step_sets(self, sets, lr: float, weight_decay: float, beta: float, nesterov: bool = True,
                       after_group=None, max_group: int | None = None, halve_groups: bool = False,
                       peer_ptrs=None) -> None:
        """prologue -> Newton-Schulz -> update for several sets of parameters, each set of one
        shape and dtype: `sets` is a list of (params, grads, moms).

        Every set is cut into launch groups (see plan_launches; at most `max_group` members per
        group when given, at most half of the set with `halve_groups`), and all groups of all sets
        go through ONE pipeline: the prologue of group i+1 (and, where the update is a kernel of
        its own, the update of group i-1) run on a side stream beside the GEMMs of group i, also
        across the boundary between two sets. `after_group(params_of_group, event)` is called
        once the update of a group has been enqueued; `event` completes when those parameters hold
        their new values. `peer_ptrs(param)` (optional) returns the addresses of that parameter's
        copies in other GPUs' memory; the update kernel then stores every new value there as well."""
        mode, steps = _ns_mode, _ns_steps
        jobs = []
        for params, grads, moms in sets:
            if not params:
                continue
            p0 = params[0]
            rows, cols = view_2d(p0.shape)
            code = dtype_code(p0)
            for p, g, m in zip(params, grads, moms):
                _require_cuda(p, "parameter")
                if p.shape != p0.shape or p.dtype != p0.dtype or g.dtype != p0.dtype or m.dtype != p0.dtype:
                    raise ValueError("muon_step needs tensors of one shape and one dtype")
                if not (p.is_contiguous() and g.is_contiguous() and m.is_contiguous()):
                    raise ValueError("muon_step needs contiguous parameter, gradient and momentum")
                if p.device != sets[0][0][0].device:
                    raise ValueError("muon_step_sets needs all parameters on one device")
            m_, n_ = min(rows, cols), max(rows, cols)
            sizes = plan_launches(m_, n_, len(params), self.workspace_cap_bytes, self._sm_pairs(p0.device))
            if _grad_ready and len(params) > 1 and grads[0].data_ptr() in _grad_ready:
                # The gradients are still arriving (copied in or reduced on another stream): start
                # with small groups, so that the first kernels only wait for the first arrivals.
                sizes = ramped_sizes(sizes)
            cap = max_group
            if halve_groups:
                half = max(1, -(-len(params) // 2))
                cap = half if cap is None else min(cap, half)
            if cap is not None and max(sizes) > cap:
                launches = -(-len(params) // max(1, cap))
                cuts = [round(i * len(params) / launches) for i in range(launches + 1)]
                sizes = [e - s for s, e in zip(cuts[:-1], cuts[1:])]
            start = 0
            for b in sizes:
                sl = slice(start, start + b)
                jobs.append(dict(params=params[sl], grads=grads[sl], moms=moms[sl], rows=rows, cols=cols,
                                 code=code, m=m_, n=n_, tall=rows > cols, scale=aspect_scale(p0.shape),
                                 layout=_lib.ns_layout(b, m_, n_, _NS_MODES[mode])))
                start += b
        if not jobs:
            return
        dev = jobs[0]["params"][0].device
        hyper = dict(lr=lr, weight_decay=weight_decay, beta=beta, nesterov=nesterov, mode=_NS_MODES[mode],
                     steps=steps, eps=1e-7)
        if self.overlap_elementwise and len(jobs) >= 2:
            self._run_jobs_pipelined(dev, jobs, hyper, after_group, peer_ptrs)
        else:
            self._run_jobs_serial(dev, jobs, hyper, after_group, peer_ptrs)

    def _run_jobs_serial(self, dev, jobs, hyper, after_group, peer_ptrs) -> None:
        with torch.cuda.device(dev):
            current = torch.cuda.current_stream(dev)
            stream = current.cuda_stream
            for job in jobs:
                layout = job["layout"]
                ws = self.workspace(dev, layout.total_bytes)
                wptr = self._aligned_ptr(ws)
                _wait_grads(current, job["grads"])
                n = len(job["params"])
                if peer_ptrs is None:
                    check(lib.muon_b200_muon_step(
                        ptr_array([p.data_ptr() for p in job["params"]]),
                        ptr_array([g.data_ptr() for g in job["grads"]]),
                        ptr_array([m.data_ptr() for m in job["moms"]]),
                        n, job["rows"], job["cols"], job["code"], hyper["lr"], hyper["weight_decay"], hyper["beta"],
                        1 if hyper["nesterov"] else 0, job["scale"], hyper["mode"], hyper["steps"], None, hyper["eps"],
                        wptr, layout.total_bytes, stream))
                else:
                    run_mode = self._prologue(job, hyper, wptr, stream)
                    slot = ctypes.c_int(0)
                    check(lib.muon_b200_ns_run(wptr, n, job["m"], job["n"], run_mode, hyper["steps"], None,
                                               hyper["eps"], ctypes.byref(slot), stream))
                    u = wptr + (layout.x_offset_bytes if slot.value == 0 else layout.c_offset_bytes)
                    # the update kernel also writes the peers' copies
                    self._epilogue(job["params"], peer_ptrs, job["rows"], job["cols"], job["code"], u, layout,
                                   job["tall"], hyper["lr"], hyper["weight_decay"], job["scale"], stream)
                self.launch_groups += 1
                if after_group is not None:
                    done = torch.cuda.Event()
                    done.record(current)
                    after_group(job["params"], done)

    @staticmethod
    def _prologue(job, hyper, wptr, stream) -> int:
        """Momentum blend + bf16 X into the workspace. Returns the mode to run the iteration with: in
        the classic mode the kernel also leaves the sums of squares of X (the Frobenius norm of
        muon.py:282), and the run is told so."""
        layout = job["layout"]
        classic = hyper["mode"] == NS_CLASSIC5
        check(lib.muon_b200_prologue_sumsq(
            ptr_array([g.data_ptr() for g in job["grads"]]), ptr_array([m.data_ptr() for m in job["moms"]]),
            len(job["params"]), job["rows"], job["cols"], job["code"], hyper["beta"], 1 if hyper["nesterov"] else 0,
            wptr + layout.x_offset_bytes, layout.ldn, layout.x_bs, 1 if job["tall"] else 0,
            wptr + layout.sumsq_offset_bytes if classic else None, layout.sumsq_bs, stream))
        return hyper["mode"] | NS_HAVE_SUMSQ if classic else hyper["mode"]

    @staticmethod
    def _epilogue(plist, peer_ptrs, rows, cols, code, u, layout, tall, lr, weight_decay, scale, stream) -> None:
        """Update epilogue of one launch group, with the peer copies when `peer_ptrs` is given."""
        local = ptr_array([p.data_ptr() for p in plist])
        if peer_ptrs is None:
            check(lib.muon_b200_epilogue(local, len(plist), rows, cols, code, u, layout.ldn, layout.x_bs,
                                         1 if tall else 0, lr, weight_decay, scale, stream))
            return
        per_param = [peer_ptrs(p) for p in plist]      # [tensor][peer]
        n_peers = len(per_param[0])
        flat = [per_param[i][r] for r in range(n_peers) for i in range(len(plist))]  # [peer][tensor]
        check(lib.muon_b200_epilogue_push(local, ptr_array(flat), n_peers, len(plist), rows, cols, code, u,
                                          layout.ldn, layout.x_bs, 1 if tall else 0, lr, weight_decay, scale,
                                          stream))

    def _run_jobs_pipelined(self, dev, jobs, hyper, after_group=None, peer_ptrs=None) -> None:
        """The HBM-bound stages of one launch group run on a side stream while the tensor-bound
        Newton-Schulz kernels of another group run on the caller's stream. The persistent GEMM CTAs
        leave registers, threads and ~30 KiB of shared memory free on every SM, so the elementwise
        CTAs are co-resident.

        Side stream:  P(0) | for i: P(i+1), [wait NS(i), E(i)]       (two workspaces, i % 2)
        Main stream:        for i: wait P(i), NS(i)                    then waits for the side stream
        E(i), the update as a kernel of its own, only exists with `peer_ptrs` (it also writes the
        peers' copies); otherwise the last GEMM of NS(i) applies the update itself.
        """
        with torch.cuda.device(dev):
            main = torch.cuda.current_stream(dev)
            side = self._side_stream(dev)
            biggest = max(job["layout"].total_bytes for job in jobs)
            ws_ptr = [self._aligned_ptr(self.workspace(dev, biggest, slot)) for slot in (0, 1)]
            side.wait_stream(main)  # gradients and parameters are ready in main-stream order

            def prologue(i):
                _wait_grads(side, jobs[i]["grads"])
                run_modes[i] = self._prologue(jobs[i], hyper, ws_ptr[i % 2], side.cuda_stream)
                ev = torch.cuda.Event()
                ev.record(side)
                return ev

            run_modes = [hyper["mode"]] * len(jobs)

            p_done = prologue(0)
            for i, job in enumerate(jobs):
                l, n = job["layout"], len(job["params"])
                next_p = prologue(i + 1) if i + 1 < len(jobs) else None
                main.wait_event(p_done)
                if peer_ptrs is None:
                    # the last GEMM of the iteration applies the update itself (where it can)
                    check(lib.muon_b200_ns_run_update(
                        ws_ptr[i % 2], run_modes[i], hyper["steps"], None, hyper["eps"],
                        ptr_array([p.data_ptr() for p in job["params"]]), n, job["rows"], job["cols"], job["code"],
                        hyper["lr"], hyper["weight_decay"], job["scale"], main.cuda_stream))
                    ns_done = torch.cuda.Event()
                    ns_done.record(main)
                    side.wait_event(ns_done)  # the next prologue but one reuses this workspace
                    if after_group is not None:
                        after_group(job["params"], ns_done)
                else:
                    slot = ctypes.c_int(0)
                    check(lib.muon_b200_ns_run(ws_ptr[i % 2], n, job["m"], job["n"], run_modes[i], hyper["steps"],
                                               None, hyper["eps"], ctypes.byref(slot), main.cuda_stream))
                    ns_done = torch.cuda.Event()
                    ns_done.record(main)
                    side.wait_event(ns_done)
                    u = ws_ptr[i % 2] + (l.x_offset_bytes if slot.value == 0 else l.c_offset_bytes)
                    # the update kernel also writes the peers' copies
                    self._epilogue(job["params"], peer_ptrs, job["rows"], job["cols"], job["code"], u, l, job["tall"],
                                   hyper["lr"], hyper["weight_decay"], job["scale"], side.cuda_stream)
                    if after_group is not None:
                        done = torch.cuda.Event()
                        done.record(side)
                        after_group(job["params"], done)
                p_done = next_p
                self.launch_groups += 1
            main.wait_stream(side)

    # -- pieces for row-sharded parameters (sharded.py) -----------------------------------
    def muon_orthogonalize(self, grads: Sequence[Tensor], moms: Sequence[Tensor], shape: Sequence[int],
                           beta: float, nesterov: bool, out: Tensor) -> None:
        """Momentum blend (in place on moms and grads) + Newton-Schulz + aspect scale for full
        matrices of one shape (muon.py:9-14), the result left in memory instead of applied:
        out[k, :rows, :cols] = bf16(U_k * scale) in the parameter's own orientation. `out` is
        bf16 [count, R >= rows, ld >= cols], contiguous, ld a multiple of 8."""
        mode, steps = _ns_mode, _ns_steps
        rows, cols = view_2d(shape)
        if not grads:
            return
        if out.dtype != torch.bfloat16 or not out.is_contiguous() or out.ndim != 3 or out.shape[0] != len(grads) \
                or out.shape[1] < rows or out.shape[2] < cols or out.shape[2] % 8:
            raise ValueError("muon_orthogonalize: out must be contiguous bf16 [count, >= rows, ld >= cols], ld % 8 == 0")
        code = dtype_code(grads[0])
        for g, m in zip(grads, moms):
            _require_cuda(g, "gradient")
            if g.dtype != grads[0].dtype or m.dtype != g.dtype or g.numel() != rows * cols or m.numel() != rows * cols:
                raise ValueError("muon_orthogonalize needs full gradients and momenta of one shape and dtype")
            if not (g.is_contiguous() and m.is_contiguous()):
                raise ValueError("muon_orthogonalize needs contiguous gradient and momentum")
        dev = grads[0].device
        m_, n_ = min(rows, cols), max(rows, cols)
        tall = rows > cols
        hyper = dict(beta=beta, nesterov=nesterov, mode=_NS_MODES[mode], steps=steps, eps=1e-7)
        sizes = plan_launches(m_, n_, len(grads), self.workspace_cap_bytes, self._sm_pairs(dev))
        with torch.cuda.device(dev):
            current = torch.cuda.current_stream(dev)
            stream = current.cuda_stream
            start = 0
            for b in sizes:
                layout = _lib.ns_layout(b, m_, n_, _NS_MODES[mode])
                job = dict(params=grads[start:start + b], grads=grads[start:start + b], moms=moms[start:start + b],
                           rows=rows, cols=cols, code=code, tall=tall, layout=layout)
                wptr = self._aligned_ptr(self.workspace(dev, layout.total_bytes))
                _wait_grads(current, job["grads"])
                run_mode = self._prologue(job, hyper, wptr, stream)
                slot = ctypes.c_int(0)
                check(lib.muon_b200_ns_run(wptr, b, m_, n_, run_mode, steps, None, hyper["eps"], ctypes.byref(slot),
                                           stream))
                u = wptr + (layout.x_offset_bytes if slot.value == 0 else layout.c_offset_bytes)
                # bf16(U * scale), transposed back for tall parameters (muon.py:14, :797-798)
                check(lib.muon_b200_cast_bf16(u, BF16, m_, n_, layout.ldn, layout.x_bs,
                                              out.data_ptr() + start * out.stride(0) * 2, out.stride(1), out.stride(0),
                                              b, 1 if tall else 0, aspect_scale(shape), stream))
                self.launch_groups += 1
                start += b

    def apply_update(self, shards: Sequence[Tensor], u: Tensor, rows: int, cols: int, lr: float,
                     weight_decay: float) -> None:
        """p = p*(1 - lr*wd) - lr*u (muon.py:66-67) on `rows` x `cols` pieces of parameters: shards[k]
        is contiguous with rows*cols elements, its update is u[k, :rows, :cols], u bf16
        [count, R >= rows, ld >= cols] contiguous with ld a multiple of 8, already scaled."""
        if not shards or rows == 0:
            return
        if u.dtype != torch.bfloat16 or not u.is_contiguous() or u.ndim != 3 or u.shape[0] != len(shards) \
                or u.shape[1] < rows or u.shape[2] < cols or u.shape[2] % 8:
            raise ValueError("apply_update: u must be contiguous bf16 [count, >= rows, ld >= cols], ld % 8 == 0")
        code = dtype_code(shards[0])
        for p in shards:
            _require_cuda(p, "parameter")
            if p.dtype != shards[0].dtype or p.numel() != rows * cols or not p.is_contiguous():
                raise ValueError("apply_update needs contiguous pieces of one size and dtype")
        dev = shards[0].device
        with torch.cuda.device(dev):
            check(lib.muon_b200_epilogue(ptr_array([p.data_ptr() for p in shards]), len(shards), rows, cols, code,
                                         u.data_ptr(), u.stride(1), u.stride(0), 0, lr, weight_decay, 1.0,
                                         _stream_ptr(dev)))

    def _side_stream(self, device: torch.device):
        key = device.index if device.index is not None else torch.cuda.current_device()
        s = self._side_streams.get(key)
        if s is None:
            s = self._side_streams[key] = torch.cuda.Stream(device=device)
        return s

    # -- Adam --------------------------------------------------------------------------
    def adam_step(self, params: Sequence[Tensor], grads: Sequence[Tensor], exp_avgs: Sequence[Tensor],
                  exp_avg_sqs: Sequence[Tensor], steps: Sequence[int], lr: float, weight_decay: float,
                  betas: tuple[float, float], eps: float) -> None:
        """Fused Adam on tensors of any sizes; one dtype per call."""
        if not params:
            return
        code = dtype_code(params[0])
        for p, g, m, v in zip(params, grads, exp_avgs, exp_avg_sqs):
            _require_cuda(p, "parameter")
            if not (p.dtype == g.dtype == m.dtype == v.dtype == params[0].dtype):
                raise ValueError("adam_step needs one dtype across parameter, gradient and state")
            if not (p.is_contiguous() and g.is_contiguous() and m.is_contiguous() and v.is_contiguous()):
                raise ValueError("adam_step needs contiguous tensors")
        dev = params[0].device
        with torch.cuda.device(dev):
            _wait_grads(torch.cuda.current_stream(dev), grads)
            check(lib.muon_b200_adam(
                ptr_array([p.data_ptr() for p in params]), ptr_array([g.data_ptr() for g in grads]),
                ptr_array([m.data_ptr() for m in exp_avgs]), ptr_array([v.data_ptr() for v in exp_avg_sqs]),
                i64_array([p.numel() for p in params]), i64_array(list(steps)), len(params), code,
                lr, weight_decay, betas[0], betas[1], eps, _stream_ptr(dev)))
            self.launch_groups += 1

    # -- functional pieces -------------------------------------------------------------
    def newton_schulz(self, G: Tensor, epsilon: float = 1e-7, mode: str | None = None,
                      steps: int | None = None) -> Tensor:
        """Orthogonalise G ([r, c] or [b, r, c], float32 / bfloat16 / float16 / float64). Returns
        bf16 of G's logical shape: a transposed view of a contiguous buffer when r > c, like the
        reference (muon.py:797-798). One library call does the cast, the transposition and the
        iteration; the result is a fresh tensor, the scratch is cached per device and stream."""
        _require_cuda(G, "G")
        if G.ndim not in (2, 3):
            raise ValueError(f"Input tensor must be 2D or 3D, but got {G.ndim}D tensor.")
        if G.dtype not in _NS_INPUT_CODE:
            raise ValueError(f"Newton-Schulz takes floating-point input, got {G.dtype}")
        mode = _ns_mode if mode is None else mode
        steps = _ns_steps if steps is None else steps
        batch = G.shape[0] if G.ndim == 3 else 1
        r, c = int(G.shape[-2]), int(G.shape[-1])
        if batch == 0 or r == 0 or c == 0:
            raise _lib.MuonB200Error(-1, "Newton-Schulz needs batch, rows, cols >= 1")
        src = G.reshape(batch, r, c)
        if src.stride(-1) != 1 or src.stride(-2) < c or (batch > 1 and src.stride(0) < (r - 1) * src.stride(-2) + c):
            src = src.contiguous()  # rows must be contiguous, non-overlapping and in order
        tall = r > c
        m_, n_ = (c, r) if tall else (r, c)
        ldn = (n_ + 7) // 8 * 8
        dev = G.device
        with torch.cuda.device(dev):
            need = lib.muon_b200_zeropower_scratch_bytes(batch, r, c, _NS_MODES[mode])
            scratch = self.workspace(dev, need, slot=2)
            out = torch.empty(batch, m_, ldn, dtype=torch.bfloat16, device=dev)
            check(lib.muon_b200_zeropower(src.data_ptr(), _NS_INPUT_CODE[G.dtype], r, c, src.stride(-2),
                                          src.stride(0) if batch > 1 else r * src.stride(-2), batch,
                                          out.data_ptr(), ldn, m_ * ldn, self._aligned_ptr(scratch), need,
                                          _NS_MODES[mode], steps, None, epsilon, _stream_ptr(dev)))
            self.launch_groups += 1
        out = out[:, :, :n_]
        if tall:
            out = out.mT
        return out if G.ndim == 3 else out[0]


def _install_stats_dump() -> None:
    """MUON_B200_STATS=1: time every kernel launch with CUDA events and print, at interpreter
    exit, device time, launches and achieved rate per kernel kind."""
    import atexit
    import os
    import sys
    if os.environ.get("MUON_B200_STATS", "0") not in ("1", "true", "yes"):
        return
    _lib.timing_enable(True)

    def dump():
        try:
            stats = _lib.timing_collect()
        except Exception as e:  # the CUDA context may already be gone
            print(f"[muon_b200] stats unavailable: {e}", file=sys.stderr)
            return
        for kind, (ms, work, launches) in stats.items():
            if launches:
                unit, scale = ("TFLOP/s", 1e12) if kind.startswith("ns_") else ("GB/s", 1e9)
                print(f"[muon_b200] {kind:14s} launches={launches:7d} device_ms={ms:10.3f} "
                      f"rate={work / (ms * 1e-3) / scale:8.1f} {unit}", file=sys.stderr)

    atexit.register(dump)


_install_stats_dump()

_backend = None


def get_backend():
    """The active backend; created on first use."""
    global _backend
    if _backend is None:
        _backend = CudaBackend()
    return _backend


def _set_backend_for_testing(backend):
    """Test seam: swap the backend object (pass None to restore the CUDA one). Returns the
    previous backend. Product code never calls this."""
    global _backend
    prev, _backend = _backend, backend
    return prev
