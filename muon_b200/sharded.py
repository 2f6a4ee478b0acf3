"""Muon for parameters that are sharded by rows across the ranks (FSDP2-style).

The reference's distributed classes need every rank to hold every full parameter (muon.py:41
asserts plain ``torch.nn.Parameter``s and muon.py:68 gathers full parameters). With fully sharded
data parallelism a rank only holds rows ``[r*c, (r+1)*c)`` of every parameter and of its gradient,
``c = ceil(rows / W)`` — the layout of ``DTensor`` with ``Shard(0)`` on a one-dimensional mesh,
which is what ``torch.distributed.fsdp.fully_shard`` leaves. ``ShardedMuon`` takes such
parameters (``DTensor``s, or plain local shards plus their full shapes) and runs, per set of
same-shape parameters:

1. one ``all_to_all``: every rank sends its rows of the gradient of parameter j to the rank that
   owns j (j mod W within the set), so an owner ends up with the full gradients of its parameters;
2. on the owner: momentum blend, Newton-Schulz and the aspect scale, exactly the kernels of the
   other classes (momentum buffers are full matrices and live on the owner only, as in
   muon.py:59-64);
3. one ``all_to_all`` back, of the *updates* in bf16 (half the bytes of fp32 parameters): every rank
   receives its rows of every update;
4. every rank applies ``p = p*(1 - lr*wd) - lr*u`` to its own rows with the update kernel.

Every element goes through the same arithmetic as in ``SingleDeviceMuon`` on the full parameter,
so the shards are bit-identical to the corresponding rows of a single-device run.
"""
from __future__ import annotations

from collections import OrderedDict

import torch
import torch.distributed as dist

from .engine import get_backend, view_2d

try:  # DTensor moved between releases; the class is only needed for isinstance checks
    from torch.distributed.tensor import DTensor
except Exception:  # pragma: no cover
    DTensor = None


def _local(t):
    return t.to_local() if DTensor is not None and isinstance(t, DTensor) else t


def shard_rows(rows: int, world: int, rank: int) -> tuple[int, int]:
    """(chunk, rows held by `rank`) for a dimension of `rows` split like torch.chunk / Shard(0):
    chunks of ceil(rows / world), the last ranks possibly short or empty."""
    chunk = -(-rows // world)
    return chunk, max(0, min(rows, (rank + 1) * chunk) - rank * chunk)


class ShardedMuon(torch.optim.Optimizer):
    """Muon over row-sharded parameters.

    Arguments:
        params: list of parameters, the same list in the same order on every rank. Each is a
            ``DTensor`` with placements ``(Shard(0),)`` on a 1-D mesh, or a plain tensor holding
            this rank's rows, in which case ``full_shapes`` gives the unsharded shape of each.
        lr, weight_decay, momentum: as for ``Muon`` (muon.py:18-38).
        full_shapes: unsharded shapes, one per parameter (only for plain tensors).
        process_group: the group the rows are sharded over (default: the mesh's group for
            ``DTensor``s, else the default group).
    """

    def __init__(self, params, lr=0.02, weight_decay=0, momentum=0.95, full_shapes=None, process_group=None):
        params = list(params)
        assert len(params) >= 1
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=momentum)
        if full_shapes is not None and len(full_shapes) != len(params):
            raise ValueError("full_shapes needs one shape per parameter")
        self._full_shape = {}
        group = process_group
        for i, p in enumerate(params):
            if DTensor is not None and isinstance(p, DTensor):
                mesh = p.device_mesh
                if mesh.ndim != 1 or len(p.placements) != 1 or not p.placements[0].is_shard(0):
                    raise ValueError("ShardedMuon takes DTensors sharded on dimension 0 of a one-dimensional mesh")
                if group is None:
                    group = mesh.get_group()
                self._full_shape[id(p)] = tuple(p.shape)
            else:
                if full_shapes is None:
                    raise ValueError("plain tensors need full_shapes (their unsharded shapes)")
                self._full_shape[id(p)] = tuple(int(s) for s in full_shapes[i])
            if len(self._full_shape[id(p)]) < 2:
                raise ValueError("Muon is for parameters with at least two dimensions")
        self._group = group
        # the largest first, like the reference's sort (muon.py:42), on the unsharded shapes
        order = sorted(range(len(params)), key=lambda i: self._full_shape[id(params[i])], reverse=True)
        super().__init__([params[i] for i in order], defaults)

    # ------------------------------------------------------------------------------------
    def _world(self):
        return dist.get_world_size(self._group), dist.get_rank(self._group)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        world, rank = self._world()
        for group in self.param_groups:
            sets: "OrderedDict[tuple, list]" = OrderedDict()
            for p in group["params"]:
                sets.setdefault((self._full_shape[id(p)], p.dtype), []).append(p)
            for (shape, _), plist in sets.items():
                self._step_set(plist, shape, group, world, rank)
        return loss

    def _step_set(self, plist, shape, group, world, rank) -> None:
        backend = get_backend()
        rows, cols = view_2d(shape)
        chunk, mine_rows = shard_rows(rows, world, rank)
        ld = (cols + 7) // 8 * 8  # pitch of the update blocks: rows of 16-byte multiples
        n = len(plist)
        locals_ = []
        for p in plist:
            lp = _local(p)
            if lp.numel() != mine_rows * cols:
                raise ValueError(f"rank {rank} should hold {mine_rows} rows of a {tuple(shape)} parameter, "
                                 f"got a shard of shape {tuple(lp.shape)}")
            locals_.append(lp)
        dev, dtype = locals_[0].device, locals_[0].dtype
        # parameter j of the set is owned by rank j mod W; blocks are ordered by owner
        by_owner = [list(range(d, n, world)) for d in range(world)]
        counts = [len(ix) for ix in by_owner]
        order = [j for ix in by_owner for j in ix]
        n_mine = counts[rank]

        # 1. gradients to their owners (a missing gradient counts as zeros, muon.py:59-61)
        send = torch.zeros(n, chunk, cols, dtype=dtype, device=dev)
        for slot, j in enumerate(order):
            g = plist[j].grad
            if g is not None and mine_rows:
                send[slot, :mine_rows].copy_(_local(g).reshape(mine_rows, cols))
        recv = torch.empty(world, n_mine, chunk, cols, dtype=dtype, device=dev)
        dist.all_to_all_single(recv.view(world * n_mine, chunk * cols), send.view(n, chunk * cols),
                               output_split_sizes=[n_mine] * world, input_split_sizes=counts, group=self._group)

        # 2. the owner's share: full gradients -> scaled orthogonal updates
        upd = torch.zeros(n_mine, world * chunk, ld, dtype=torch.bfloat16, device=dev)
        if n_mine:
            full = recv.transpose(0, 1).contiguous().view(n_mine, world * chunk, cols)
            grads = [full[k, :rows] for k in range(n_mine)]
            moms = []
            for j in by_owner[rank]:
                state = self.state[plist[j]]
                if len(state) == 0:
                    state["momentum_buffer"] = torch.zeros(rows, cols, dtype=dtype, device=dev)
                moms.append(state["momentum_buffer"])
            backend.muon_orthogonalize(grads, moms, shape, group["momentum"], True, upd)

        # 3. updates back to the rows' holders, bf16
        back_send = upd.view(n_mine, world, chunk, ld).transpose(0, 1).contiguous()
        back = torch.empty(n, chunk, ld, dtype=torch.bfloat16, device=dev)
        dist.all_to_all_single(back.view(n, chunk * ld), back_send.view(world * n_mine, chunk * ld),
                               output_split_sizes=counts, input_split_sizes=[n_mine] * world, group=self._group)

        # 4. every rank updates its own rows (block `slot` of `back` belongs to parameter order[slot])
        if mine_rows:
            backend.apply_update([locals_[j] for j in order], back, mine_rows, cols, group["lr"], group["weight_decay"])
