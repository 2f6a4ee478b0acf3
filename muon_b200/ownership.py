"""Which rank updates which parameter of a distributed Muon group.

``round_robin`` (default) is the reference's rule (muon.py:54-58): with the group's parameters
sorted by size, rank r owns the parameters r, r + W, r + 2W, ... The result of a step does not
depend on who owns what (every parameter's update is a function of its own gradient and momentum
only), so other assignments are equally valid; what changes is how evenly the Newton-Schulz work
is spread.

``balanced`` spreads by cost instead of by count: parameters are taken in order of decreasing
Newton-Schulz FLOPs (ties in list order) and each goes to the rank with the least work so far
(ties to the lowest rank). Round-robin leaves up to one matrix of the most expensive shape of
difference between ranks whenever a shape's count is not a multiple of the world size (GPT-2
small's 12 + 12 matrices with a 3072 side on 8 ranks; any model whose layer count the world size
does not divide); ``balanced`` bounds the difference by one matrix of the cheapest shape.

Every rank computes the same assignment from the same list. Momentum buffers live on the owner
only (muon.py:59-64), so a policy must stay the same from step to step;
``consolidated_state_dict`` / ``load_consolidated_state_dict`` move a checkpoint between
policies and world sizes.
"""
from __future__ import annotations

import os
from typing import Sequence

POLICIES = ("round_robin", "balanced")
_policy: str | None = None


def set_ownership(policy: str) -> None:
    """Process-wide ownership policy of the distributed classes; set it on every rank, before the
    first step."""
    global _policy
    if policy not in POLICIES:
        raise ValueError(f"ownership policy must be one of {POLICIES}, got {policy!r}")
    _policy = policy


def get_ownership() -> str:
    if _policy is not None:
        return _policy
    p = os.environ.get("MUON_B200_OWNERSHIP", "round_robin").lower()
    if p not in POLICIES:
        raise ValueError(f"MUON_B200_OWNERSHIP must be one of {POLICIES}, got {p!r}")
    return p


def ns_cost(shape: Sequence[int]) -> int:
    """Newton-Schulz FLOPs per iteration of a parameter of this shape, symmetric products counted
    once: m(m+1)n + m^2(m+1) + 2 m^2 n for the m x n (m <= n) 2-D view."""
    rows = int(shape[0])
    cols = 1
    for s in shape[1:]:
        cols *= int(s)
    m, n = min(rows, cols), max(rows, cols)
    return m * (m + 1) * n + m * m * (m + 1) + 2 * m * m * n


def owners(shapes: Sequence[Sequence[int]], world: int, policy: str | None = None) -> list[int]:
    """owner[i] = rank that updates parameter i of a group whose parameters have `shapes`."""
    policy = policy or get_ownership()
    if policy == "round_robin" or world <= 1:
        return [i % world for i in range(len(shapes))] if world > 0 else []
    if policy != "balanced":
        raise ValueError(f"unknown ownership policy {policy!r}")
    cost = [ns_cost(s) for s in shapes]
    order = sorted(range(len(shapes)), key=lambda i: (-cost[i], i))
    load = [0] * world
    out = [0] * len(shapes)
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        out[i] = r
        load[r] += cost[i]
    return out


def owned_indices(params, world: int, rank: int, policy: str | None = None) -> list[int]:
    """Indices (increasing) of the parameters of `params` that `rank` updates."""
    who = owners([tuple(p.shape) for p in params], world, policy)
    return [i for i, r in enumerate(who) if r == rank]
