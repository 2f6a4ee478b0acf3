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

Sets are cut into units of at most 32 parameters and the units are pipelined: the gradients of
unit k+1 and the updates of unit k-1 are exchanged (asynchronous collectives) while unit k is
orthogonalised.

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
    """This rank's rows of `t`: the local shard of a DTensor (redistributed to Shard(0) first when
    it arrives in another placement, e.g. a gradient that is still Partial), or `t` itself."""
    if DTensor is None or not isinstance(t, DTensor):
        return t
    if len(t.placements) != 1 or not t.placements[0].is_shard(0):
        from torch.distributed.tensor import Shard
        t = t.redistribute(placements=[Shard(0)])
    return t.to_local()


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
        self.max_per_unit = 32  # parameters per exchange/orthogonalise unit (rounded to the world size)
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
        # Work units: same-shape parameters, at most `max_per_unit` at a time, so that the exchanges
        # of one unit run while another unit is being orthogonalised.
        units = []
        for group in self.param_groups:
            sets: "OrderedDict[tuple, list]" = OrderedDict()
            for p in group["params"]:
                sets.setdefault((self._full_shape[id(p)], p.dtype), []).append(p)
            for (shape, _), plist in sets.items():
                per = max(world, self.max_per_unit // world * world)
                for start in range(0, len(plist), per):
                    units.append(_Unit(plist[start:start + per], shape, group, world, rank))
        # Pipeline: gradients of unit k+1 travel while unit k is orthogonalised; the updates of unit k
        # travel back while unit k+1 is orthogonalised and are applied after that.
        if units:
            units[0].send_gradients(self._group)
        previous = None
        for k, unit in enumerate(units):
            if k + 1 < len(units):
                units[k + 1].send_gradients(self._group)
            unit.orthogonalize(self)
            unit.send_updates(self._group)
            if previous is not None:
                previous.apply()
            previous = unit
        if previous is not None:
            previous.apply()
        return loss


class _Unit:
    """One exchange -> orthogonalise -> exchange -> apply unit of ShardedMuon.step (same-shape
    parameters; parameter j of the unit is owned by rank j mod W)."""

    def __init__(self, plist, shape, group, world, rank):
        self.plist, self.shape, self.group, self.world, self.rank = plist, shape, group, world, rank
        self.rows, self.cols = view_2d(shape)
        self.chunk, self.mine_rows = shard_rows(self.rows, world, rank)
        self.ld = (self.cols + 7) // 8 * 8  # pitch of the update blocks: rows of 16-byte multiples
        n = len(plist)
        self.locals = []
        for p in plist:
            lp = _local(p)
            if lp.numel() != self.mine_rows * self.cols:
                raise ValueError(f"rank {rank} should hold {self.mine_rows} rows of a {tuple(shape)} parameter, "
                                 f"got a shard of shape {tuple(lp.shape)}")
            if not lp.is_contiguous():
                raise ValueError("ShardedMuon needs contiguous local shards")
            self.locals.append(lp)
        # blocks are ordered by owner
        self.by_owner = [list(range(d, n, world)) for d in range(world)]
        self.counts = [len(ix) for ix in self.by_owner]
        self.order = [j for ix in self.by_owner for j in ix]
        self.n_mine = self.counts[rank]
        self.grad_work = self.upd_work = None

    def send_gradients(self, pg) -> None:
        """1. gradient rows to their owners (a missing gradient counts as zeros, muon.py:59-61)."""
        n, chunk, cols, world = len(self.plist), self.chunk, self.cols, self.world
        dev, dtype = self.locals[0].device, self.locals[0].dtype
        send = torch.zeros(n, chunk, cols, dtype=dtype, device=dev)
        for slot, j in enumerate(self.order):
            g = self.plist[j].grad
            if g is not None and self.mine_rows:
                send[slot, :self.mine_rows].copy_(_local(g).reshape(self.mine_rows, cols))
        self.recv = torch.empty(world, self.n_mine, chunk, cols, dtype=dtype, device=dev)
        self.grad_work = dist.all_to_all_single(
            self.recv.view(world * self.n_mine, chunk * cols), send.view(n, chunk * cols),
            output_split_sizes=[self.n_mine] * world, input_split_sizes=self.counts, group=pg, async_op=True)
        self._send = send  # stays alive until the exchange has completed

    def orthogonalize(self, optimizer) -> None:
        """2. the owner's share: full gradients -> scaled orthogonal updates."""
        world, chunk, cols = self.world, self.chunk, self.cols
        dev, dtype = self.locals[0].device, self.locals[0].dtype
        self.grad_work.wait()
        self._send = None
        self.upd = torch.zeros(self.n_mine, world * chunk, self.ld, dtype=torch.bfloat16, device=dev)
        if self.n_mine:
            full = self.recv.transpose(0, 1).contiguous().view(self.n_mine, world * chunk, cols)
            grads = [full[k, :self.rows] for k in range(self.n_mine)]
            moms = []
            for j in self.by_owner[self.rank]:
                state = optimizer.state[self.plist[j]]
                if len(state) == 0:
                    state["momentum_buffer"] = torch.zeros(self.rows, cols, dtype=dtype, device=dev)
                moms.append(state["momentum_buffer"])
            get_backend().muon_orthogonalize(grads, moms, self.shape, self.group["momentum"], True, self.upd)
        self.recv = None

    def send_updates(self, pg) -> None:
        """3. update rows back to their holders, bf16."""
        n, world, chunk, ld = len(self.plist), self.world, self.chunk, self.ld
        back_send = self.upd.view(self.n_mine, world, chunk, ld).transpose(0, 1).contiguous()
        self.back = torch.empty(n, chunk, ld, dtype=torch.bfloat16, device=self.upd.device)
        self.upd_work = dist.all_to_all_single(
            self.back.view(n, chunk * ld), back_send.view(world * self.n_mine, chunk * ld),
            output_split_sizes=self.counts, input_split_sizes=[self.n_mine] * world, group=pg, async_op=True)
        self._send = back_send
        self.upd = None

    def apply(self) -> None:
        """4. every rank updates its own rows (block `slot` of `back` belongs to parameter order[slot])."""
        self.upd_work.wait()
        self._send = None
        if self.mine_rows:
            get_backend().apply_update([self.locals[j] for j in self.order], self.back, self.mine_rows, self.cols,
                                       self.group["lr"], self.group["weight_decay"])
        self.back = None
