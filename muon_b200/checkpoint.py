"""World-size-independent optimizer checkpoints for the distributed classes.

In ``Muon`` / ``MuonWithAuxAdam`` a momentum buffer exists only on the rank that owns the
parameter (muon.py:57-64), so ``optimizer.state_dict()`` differs from rank to rank and can only
be loaded back with the same world size and parameter order. The two functions here gather
that sharded state into one dictionary keyed by the parameter's position in its (sorted) group,
and scatter such a dictionary back according to the ownership rule of the *current* world size.
The reference has no counterpart; its ``state_dict`` / ``load_state_dict`` keep working unchanged.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .ownership import owned_indices

FORMAT = "muon_b200.consolidated.v1"


def _world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


def consolidated_state_dict(optimizer, dst: int = 0):
    """Collective. Returns on rank ``dst`` (None elsewhere) a dict with, per param group, the
    momentum buffer of every Muon parameter (gathered from its owner, on CPU) or the Adam state
    (replicated, taken from ``dst``), plus the group's hyper-parameters and the parameter shapes."""
    world, rank = _world()
    groups = []
    for group in optimizer.param_groups:
        params = group["params"]
        hyper = {k: v for k, v in group.items() if k != "params"}
        entry = {"hyper": hyper, "shapes": [tuple(p.shape) for p in params]}
        if group.get("use_muon", True):
            mine = {i: optimizer.state[p]["momentum_buffer"].detach().cpu()
                    for i, p in enumerate(params) if "momentum_buffer" in optimizer.state.get(p, {})}
            if world > 1:
                parts = [None] * world if rank == dst else None
                dist.gather_object(mine, parts, dst=dst)
            else:
                parts = [mine]
            if rank == dst:
                merged = {}
                for part in parts:
                    merged.update(part)
                entry["momentum"] = merged
        elif rank == dst:
            entry["adam"] = {i: {k: (v.detach().cpu() if torch.is_tensor(v) else v)
                                 for k, v in optimizer.state[p].items()}
                             for i, p in enumerate(params) if len(optimizer.state.get(p, {}))}
        groups.append(entry)
    if rank != dst:
        return None
    return {"format": FORMAT, "saved_world_size": world, "groups": groups}


def load_consolidated_state_dict(optimizer, state) -> None:
    """Every rank passes the same dictionary (from ``consolidated_state_dict``). Each rank keeps
    the momentum of the parameters it owns under the current world size and ownership policy
    (ownership.py; by default index % world == rank) and drops the rest; Adam state is restored on every rank. Hyper-parameters are restored too."""
    if not isinstance(state, dict) or state.get("format") != FORMAT:
        raise ValueError("not a consolidated muon_b200 optimizer state")
    world, rank = _world()
    distributed_cls = type(optimizer).__name__ in ("Muon", "MuonWithAuxAdam")
    if len(state["groups"]) != len(optimizer.param_groups):
        raise ValueError("checkpoint and optimizer have different numbers of param groups")
    for group, entry in zip(optimizer.param_groups, state["groups"]):
        params = group["params"]
        if [tuple(p.shape) for p in params] != [tuple(s) for s in entry["shapes"]]:
            raise ValueError("checkpoint and optimizer disagree on the parameter shapes of a group")
        for k, v in entry["hyper"].items():
            group[k] = v
        if group.get("use_muon", True):
            momentum = entry.get("momentum", {})
            mine = set(owned_indices(params, world, rank)) if distributed_cls else set(range(len(params)))
            for i, p in enumerate(params):
                owned = i in mine
                optimizer.state.pop(p, None)
                if owned and i in momentum:
                    optimizer.state[p]["momentum_buffer"] = momentum[i].to(device=p.device, dtype=p.dtype).clone()
        else:
            for i, p in enumerate(params):
                optimizer.state.pop(p, None)
                if i in entry.get("adam", {}):
                    optimizer.state[p].update({k: (v.to(device=p.device, dtype=p.dtype).clone() if torch.is_tensor(v) else v)
                                               for k, v in entry["adam"][i].items()})
