"""Cross-rank exchange of updated parameters for the distributed optimizers.

The reference ends every window with ``dist.all_gather`` of the freshly updated parameters
(muon.py:68). Two transports implement that exchange here:

``nccl``  the same ``dist.all_gather`` call, issued asynchronously. NCCL moves the data with
          copy kernels that need SMs; the Newton-Schulz GEMMs are persistent grids that fill
          the device, so the two compete and little of the transfer is hidden.

``ce``    every rank maps the other ranks' parameter tensors into its address space (CUDA IPC,
          through ``torch.multiprocessing.reductions``) and, as soon as one of its own
          parameters is updated, pushes it to the seven peers with device-to-device copies on
          a side stream. Those copies run on the GPU's copy engines over NVLink and take no SM,
          so they overlap the remaining Newton-Schulz work. Two tiny NCCL all-reduces bracket
          the step: the first makes sure every rank has reached ``step()`` (and, in stream
          order, finished whatever read the parameters before) before any push lands in its
          memory; the second returns only after every rank's pushes have completed, which gives
          ``step()`` the reference's post-condition that all ranks hold all updated parameters.

``MUON_B200_EXCHANGE`` selects ``nccl`` (default), ``ce``, or ``auto`` (``ce`` when every rank
can map its peers, else ``nccl``). CPU tensors (the gloo test ranks) always use ``all_gather``.

Status of ``ce``: functionally verified (tests/test_gpu_distributed.py) but not the default.
Tensors imported through ``torch.multiprocessing.reductions`` are mapped in a context of the
*peer's* device; a copy into them from this rank's device is not a direct NVLink transfer
(measured 35 GB/s on B200 against 730 GB/s for a copy between two devices of one process), so
this transport is currently slower than NCCL. Mapping the peers with the IPC handle opened on
this rank's own device is what makes it a copy-engine NVLink push.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def _mode() -> str:
    m = os.environ.get("MUON_B200_EXCHANGE", "nccl").lower()
    if m not in ("auto", "ce", "nccl"):
        raise ValueError(f"MUON_B200_EXCHANGE must be auto, ce or nccl, got {m!r}")
    return m


class PeerPush:
    """Peer-mapped views of one param group's tensors on every other rank + a copy stream."""

    def __init__(self, params):
        from torch.multiprocessing.reductions import reduce_tensor

        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.device = params[0].device
        exported, error = None, None
        try:
            exported = [reduce_tensor(p.detach()) for p in params]
        except Exception as e:  # e.g. allocator backends whose blocks cannot be shared
            error = repr(e)
        gathered = [None] * self.world
        dist.all_gather_object(gathered, (exported, error))
        errors = [g[1] for g in gathered if g[1] is not None]
        self.views = None
        if not errors:
            try:
                self.views = []
                for r, (items, _) in enumerate(gathered):
                    if r == self.rank:
                        self.views.append(None)
                        continue
                    self.views.append([fn(*args) for fn, args in items])
            except Exception as e:
                errors.append(repr(e))
                self.views = None
        ok = [None] * self.world
        dist.all_gather_object(ok, self.views is not None)
        self.ok = all(ok)
        self.error = "; ".join(errors) if errors else (None if self.ok else "a peer could not map this rank")
        if not self.ok:
            self.views = None
            return
        self.stream = torch.cuda.Stream(device=self.device)
        self._token = torch.zeros(1, device=self.device)
        self.index = {id(p): i for i, p in enumerate(params)}

    def begin_step(self) -> None:
        """All ranks are inside step() (stream-ordered after their earlier work) from here on."""
        dist.all_reduce(self._token)

    def push(self, updated) -> None:
        """Copy each freshly updated local parameter into every peer's copy of it."""
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        self.stream.wait_event(ready)
        with torch.cuda.stream(self.stream):
            for p in updated:
                i = self.index[id(p)]
                src = p.detach()
                for r in range(self.world):
                    if r != self.rank:
                        self.views[r][i].copy_(src, non_blocking=True)

    def end_step(self) -> None:
        """Returns (in stream order) once every rank's pushes have landed."""
        torch.cuda.current_stream(self.device).wait_stream(self.stream)
        dist.all_reduce(self._token)


def get_peer_push(optimizer, group):
    """PeerPush of `group`, built collectively on first use; None when the NCCL/gloo gather is to
    be used. Every rank takes the same decision."""
    cache = optimizer.__dict__.setdefault("_muon_b200_exchange", {})
    key = id(group)
    if key in cache:
        return cache[key]
    params = group["params"]
    mode = _mode()
    usable = mode != "nccl" and dist.get_world_size() > 1 and all(p.is_cuda for p in params) \
        and "nccl" in str(dist.get_backend())
    push = None
    if usable:
        push = PeerPush(params)
        if not push.ok:
            if mode == "ce":
                raise RuntimeError(f"MUON_B200_EXCHANGE=ce but peers cannot be mapped: {push.error}")
            push = None
    cache[key] = push
    return push
