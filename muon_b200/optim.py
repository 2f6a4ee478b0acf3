"""The four optimizer classes of the reference (muon.py:18-260), same constructors, same
param-group keys, same state keys, same ownership rule — with the per-parameter torch ops
replaced by grouped calls into the sm_100a library.

What differs on purpose, and only in scheduling:

* same-shape parameters are orthogonalised together in one grouped launch sequence
  instead of one at a time;
* in the distributed classes each window's ``all_gather`` is issued asynchronously and
  overlaps the next windows' Newton-Schulz work; all of them are waited for before
  ``step`` returns, so callers observe the reference's post-condition (every rank holds
  every updated parameter).
"""
from __future__ import annotations

from collections import OrderedDict

import torch
import torch.distributed as dist

from .engine import get_backend, plan_launches, view_2d
from .exchange import get_peer_push
from .ownership import get_ownership, owners


def _ensure_grad_and_state(optimizer, p) -> None:
    """muon.py:59-64: a missing gradient becomes zeros, so that every rank reaches every
    collective; the momentum buffer is created on first use."""
    if p.grad is None:
        p.grad = torch.zeros_like(p)
    elif not p.grad.is_contiguous():
        p.grad = p.grad.contiguous()
    state = optimizer.state[p]
    if len(state) == 0:
        state["momentum_buffer"] = torch.zeros_like(p)


def _bucket_by_shape(params):
    """Stable buckets of same-shape, same-dtype, same-device parameters."""
    buckets: "OrderedDict[tuple, list]" = OrderedDict()
    for p in params:
        buckets.setdefault((tuple(p.shape), p.dtype, p.device), []).append(p)
    return buckets


def _muon_update_params(optimizer, params, group, **step_options) -> None:
    """Body of the reference's per-parameter loop (muon.py:91-99) for a list of parameters: same-shape
    parameters form a set, and all sets go to the engine in one call, which runs one pipeline of
    grouped launches over them."""
    backend = get_backend()
    for p in params:
        _ensure_grad_and_state(optimizer, p)
    sets = [(plist, [p.grad for p in plist], [optimizer.state[p]["momentum_buffer"] for p in plist])
            for plist in _bucket_by_shape(params).values()]
    if hasattr(backend, "muon_step_sets"):
        backend.muon_step_sets(sets, group["lr"], group["weight_decay"], group["momentum"], **step_options)
        return
    step_options.pop("halve_groups", None)
    for plist, grads, moms in sets:
        backend.muon_step(plist, grads, moms, group["lr"], group["weight_decay"], group["momentum"],
                          **step_options)


def _adam_update_params(optimizer, group) -> None:
    """Adam branch (muon.py:184-197): replicated on every rank, no collective."""
    backend = get_backend()
    params = group["params"]
    for p in params:
        if p.grad is None:
            p.grad = torch.zeros_like(p)
        elif not p.grad.is_contiguous():
            p.grad = p.grad.contiguous()
        state = optimizer.state[p]
        if len(state) == 0:
            state["exp_avg"] = torch.zeros_like(p)
            state["exp_avg_sq"] = torch.zeros_like(p)
            state["step"] = 0
        state["step"] += 1
    by_kind: "OrderedDict[tuple, list]" = OrderedDict()
    for p in params:
        by_kind.setdefault((p.dtype, p.device), []).append(p)
    for plist in by_kind.values():
        backend.adam_step(plist, [p.grad for p in plist],
                          [optimizer.state[p]["exp_avg"] for p in plist],
                          [optimizer.state[p]["exp_avg_sq"] for p in plist],
                          [optimizer.state[p]["step"] for p in plist],
                          group["lr"], group["weight_decay"], group["betas"], group["eps"])


def _next_chunk(params, owned, done_upto, backend):
    """The next parameters this rank updates in one grouped launch sequence: the same-shape run
    starting at owned[done_upto], cut to the first launch the planner proposes."""
    p0 = params[owned[done_upto]]
    rows, cols = view_2d(p0.shape)
    run = 0
    for idx in owned[done_upto:]:
        if params[idx].shape != p0.shape or params[idx].dtype != p0.dtype:
            break
        run += 1
    limit = plan_launches(min(rows, cols), max(rows, cols), run,
                          getattr(backend, "workspace_cap_bytes", 4 << 30))[0]
    return [params[idx] for idx in owned[done_upto:done_upto + limit]]


# Gathers issued but not yet known to be complete, per step. An earlier version kept every
# window's gather of a step in flight (over a hundred at a time); the number is now bounded.
_MAX_GATHERS_IN_FLIGHT = 16


def _throttle_gathers(pending, settled: int, device) -> int:
    """Wait (on the host) for the oldest gathers until at most _MAX_GATHERS_IN_FLIGHT are
    outstanding. Returns the new count of settled entries of `pending`."""
    while len(pending) - settled > _MAX_GATHERS_IN_FLIGHT:
        work = pending[settled]
        if work is not None:
            work.wait()
            if device.type == "cuda":  # Work.wait() only orders the stream: wait for the stream too
                torch.cuda.current_stream(device).synchronize()
        settled += 1
    return settled


def _distributed_muon_group_step(optimizer, group) -> None:
    """Windowed round-robin of muon.py:54-68. Window k holds params[kW:(k+1)W]; rank r
    updates params[kW + r] and every rank then receives the whole window. (With the `balanced`
    ownership policy the assignment is by cost instead, see ownership.py; the result is the same.)"""
    backend = get_backend()
    world, rank = dist.get_world_size(), dist.get_rank()
    params = group["params"]
    # muon.py:55 — the pad entries alias one scratch tensor and only ever receive.
    params_pad = params + [torch.empty_like(params[-1])] * (world - len(params) % world)
    policy = get_ownership()
    who = owners([tuple(p.shape) for p in params], world, policy)
    owned = [i for i, r in enumerate(who) if r == rank]
    done_upto = 0  # owned[:done_upto] have been updated
    pending, settled = [], 0
    if world == 1:
        # Nothing to exchange: the whole group goes to the engine, which plans its own launches.
        _muon_update_params(optimizer, params, group)
        return
    push = get_peer_push(optimizer, group)
    if push is not None:
        # Copy-engine exchange: same ownership and update order, pushes instead of gathers. Every
        # launch group is pushed as soon as its epilogue is enqueued. The exchange of a group can
        # only start when the group is done, and at 8 GPUs the copies take about as long as the
        # compute: groups are capped to half of a same-shape run so the copy engines start early.
        # (Quarters were tried at 4 GPUs: the smaller launches lost in GEMM efficiency what they
        # gained in overlap.)
        mine = [params[i] for i in owned]
        push.begin_step()
        if push.mode == "st":
            # The update kernel stores into the peer copies itself: nothing to enqueue afterwards.
            _muon_update_params(optimizer, mine, group, peer_ptrs=push.peer_ptrs)
        else:
            _muon_update_params(optimizer, mine, group, after_group=push.push, halve_groups=world >= 4)
        push.end_step()
        return
    if policy != "round_robin":
        # Not the window pattern all_gather needs: this rank updates what it owns, then every
        # parameter is broadcast by its owner, in list order on every rank.
        _muon_update_params(optimizer, [params[i] for i in owned], group)
        for i, p in enumerate(params):
            pending.append(dist.broadcast(p, src=who[i], async_op=True))
            settled = _throttle_gathers(pending, settled, params[0].device)
        for work in pending[settled:]:
            if work is not None:
                work.wait()
        return
    for base_i in range(0, len(params), world):
        mine = base_i + rank
        if mine < len(params) and done_upto < len(owned) and owned[done_upto] == mine:
            # Update this window's parameter together with the same-shape ones this rank
            # owns in the following windows (one grouped launch sequence).
            chunk = _next_chunk(params, owned, done_upto, backend)
            _muon_update_params(optimizer, chunk, group)
            done_upto += len(chunk)
        window = params_pad[base_i:base_i + world]
        if all(w.shape == window[0].shape and w.dtype == window[0].dtype for w in window):
            pending.append(dist.all_gather(window, params_pad[mine], async_op=True))
        else:
            # A window that mixes shapes (the sort puts 3072x768 before 768x3072, and a class
            # whose count the world size does not divide spills into the next one): all_gather
            # needs equal sizes (the reference fails here, muon.py:68), so every real parameter
            # of the window is broadcast from its owner instead. Pad entries carry no data.
            for r, w in enumerate(window):
                if base_i + r < len(params):
                    pending.append(dist.broadcast(w, src=r, async_op=True))
        settled = _throttle_gathers(pending, settled, params[0].device)
    for work in pending[settled:]:
        if work is not None:
            work.wait()


class Muon(torch.optim.Optimizer):
    """Distributed Muon (muon.py:18-70): momentum SGD whose 2-D updates are orthogonalised
    by a Newton-Schulz iteration. Requires an initialised default process group.

    Arguments:
        lr: learning rate, in units of spectral norm per update.
        weight_decay: AdamW-style decoupled weight decay.
        momentum: momentum coefficient.
    """

    def __init__(self, params, lr=0.02, weight_decay=0, momentum=0.95):
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=momentum)
        assert isinstance(params, list) and len(params) >= 1 and isinstance(params[0], torch.nn.Parameter)
        params = sorted(params, key=lambda x: x.size(), reverse=True)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            _distributed_muon_group_step(self, group)
        return loss


class SingleDeviceMuon(torch.optim.Optimizer):
    """Muon for non-distributed settings (muon.py:73-101)."""

    def __init__(self, params, lr=0.02, weight_decay=0, momentum=0.95):
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=momentum)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            _muon_update_params(self, group["params"], group)
        return loss


def _apply_group_defaults(param_groups, sort_muon_params: bool) -> None:
    """muon.py:140-155 / :207-221: per-group defaults and exact key-set checks."""
    for group in param_groups:
        assert "use_muon" in group
        if group["use_muon"]:
            if sort_muon_params:
                group["params"] = sorted(group["params"], key=lambda x: x.size(), reverse=True)
            group["lr"] = group.get("lr", 0.02)
            group["momentum"] = group.get("momentum", 0.95)
            group["weight_decay"] = group.get("weight_decay", 0)
            assert set(group.keys()) == set(["params", "lr", "momentum", "weight_decay", "use_muon"])
        else:
            group["lr"] = group.get("lr", 3e-4)
            group["betas"] = group.get("betas", (0.9, 0.95))
            group["eps"] = group.get("eps", 1e-10)
            group["weight_decay"] = group.get("weight_decay", 0)
            assert set(group.keys()) == set(["params", "lr", "betas", "eps", "weight_decay", "use_muon"])


class MuonWithAuxAdam(torch.optim.Optimizer):
    """Distributed Muon with an internal Adam for the parameters Muon does not suit
    (muon.py:112-199). Every group carries ``use_muon``; Muon groups accept ``lr``,
    ``momentum``, ``weight_decay``; Adam groups accept ``lr``, ``betas``, ``eps``,
    ``weight_decay``."""

    def __init__(self, param_groups):
        _apply_group_defaults(param_groups, sort_muon_params=True)
        super().__init__(param_groups, dict())

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            if group["use_muon"]:
                _distributed_muon_group_step(self, group)
            else:
                _adam_update_params(self, group)
        return loss


class SingleDeviceMuonWithAuxAdam(torch.optim.Optimizer):
    """Non-distributed variant of MuonWithAuxAdam (muon.py:202-260)."""

    def __init__(self, param_groups):
        _apply_group_defaults(param_groups, sort_muon_params=False)
        super().__init__(param_groups, dict())

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            if group["use_muon"]:
                _muon_update_params(self, group["params"], group)
            else:
                _adam_update_params(self, group)
        return loss
