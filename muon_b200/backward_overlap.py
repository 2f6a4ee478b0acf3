"""Start the Muon update of a parameter set while the backward pass is still running.

The reference updates everything in ``optimizer.step()``, after the whole backward pass
(muon.py:81-101). The update of one parameter depends on nothing but that parameter, its gradient
and its momentum, so it can start as soon as the gradient exists. ``StepInBackward`` registers a
hook on every Muon parameter (``Tensor.register_post_accumulate_grad_hook``); when the gradients of
all same-shape parameters of a group have been accumulated, their grouped update (prologue,
Newton-Schulz, epilogue: the same calls ``step()`` makes) is enqueued on a side stream that waits
for the backward stream up to that point. ``StepInBackward.step()`` then updates what is left
(parameters that received no gradient, Adam groups) and joins the side stream. The arithmetic and
its grouping are those of ``optimizer.step()``, so the parameters come out bit for bit the same.

Single-device classes (``SingleDeviceMuon``, ``SingleDeviceMuonWithAuxAdam``): nothing else to say.

Distributed classes (``Muon``, ``MuonWithAuxAdam``; muon.py:45-70): each rank updates the
parameters it owns and writes them into the other ranks' copies (the ``st`` / ``ce`` exchange of
``muon_b200.exchange``; the all_gather transport is not supported here). A write into a peer's
parameter may only happen once that peer's backward pass no longer reads it. Every rank therefore
enters a one-element all-reduce on the side stream when a set's last gradient has arrived: it
completes when all ranks are past that point of their backward passes, and the set's update and
pushes are ordered after it. The hooks fire in the same order on every rank (same autograd graph),
so the all-reduces pair up. The gradients must be final when autograd accumulates them (a
data-parallel wrapper that all-reduces gradients after the backward pass is not compatible).

Use one backward pass per step (no gradient accumulation over several backward passes), and call
``step()`` of this object instead of the optimizer's.

    opt = SingleDeviceMuonWithAuxAdam(groups)      # or Muon(...) / MuonWithAuxAdam(...)
    overlap = StepInBackward(opt)
    loss.backward()        # updates start inside
    overlap.step()         # finishes the step
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import optim as _optim
from .exchange import get_peer_push
from .ownership import owned_indices


class StepInBackward:
    def __init__(self, optimizer):
        single = isinstance(optimizer, (_optim.SingleDeviceMuon, _optim.SingleDeviceMuonWithAuxAdam))
        distributed = isinstance(optimizer, (_optim.Muon, _optim.MuonWithAuxAdam))
        if not (single or distributed):
            raise TypeError("StepInBackward supports the four optimizer classes of muon_b200")
        self.optimizer = optimizer
        self._distributed = distributed and dist.get_world_size() > 1
        self._sets = []        # dicts: group, params (one shape bucket), waiting (ids), done, push, mine
        self._set_of = {}      # id(param) -> its set
        self._handles = []
        self._stream = None
        self._pushes = []      # PeerPush objects of the Muon groups (distributed only)
        self._begun = False
        self._token = None
        for group in optimizer.param_groups:
            if not group.get("use_muon", True):
                continue
            push = None
            if self._distributed:
                push = get_peer_push(optimizer, group)  # collective: every rank constructs this object
                if push is None:
                    raise TypeError("StepInBackward on a distributed optimizer needs the push exchange "
                                    "(CUDA parameters, NCCL process group, MUON_B200_EXCHANGE=auto, st or ce)")
                self._pushes.append(push)
            world = dist.get_world_size() if self._distributed else 1
            rank = dist.get_rank() if self._distributed else 0
            # muon.py:56-58, or the cost-balanced assignment (ownership.py)
            owned = {id(group["params"][i]) for i in owned_indices(group["params"], world, rank)}
            for plist in _optim._bucket_by_shape(group["params"]).values():
                mine = [p for p in plist if id(p) in owned]
                entry = dict(group=group, params=plist, waiting={id(p) for p in plist}, done=False,
                             push=push, mine=mine)
                self._sets.append(entry)
                for p in plist:
                    self._set_of[id(p)] = entry
                    self._handles.append(p.register_post_accumulate_grad_hook(self._on_grad))

    # -- hooks -------------------------------------------------------------------------------
    def _on_grad(self, p) -> None:
        entry = self._set_of[id(p)]
        if entry["done"]:
            raise RuntimeError("StepInBackward: a parameter received a second gradient before step(); "
                               "use one backward pass per step")
        entry["waiting"].discard(id(p))
        if not entry["waiting"]:
            self._run(entry)

    @torch.no_grad()
    def _run(self, entry) -> None:
        params = entry["params"]
        if not params[0].is_cuda:
            _optim._muon_update_params(self.optimizer, params, entry["group"])
            entry["done"] = True
            return
        device = params[0].device
        current = torch.cuda.current_stream(device)
        if self._stream is None:
            self._stream = torch.cuda.Stream(device=device)
        if self._distributed and not self._begun:
            for push in self._pushes:  # every rank is inside this step from here on
                push.begin_step()
            self._begun = True
        # Everything the backward pass has enqueued so far (these gradients, and the last reads
        # of these parameters) comes first.
        self._stream.wait_stream(current)
        with torch.cuda.stream(self._stream):
            if self._distributed:
                # Completes when every rank's backward pass has delivered this set: from then on
                # nobody reads these parameters, and the owners may overwrite them everywhere.
                if self._token is None:
                    self._token = torch.zeros(1, device=device)
                dist.all_reduce(self._token)
                push = entry["push"]
                if entry["mine"]:
                    if push.mode == "st":
                        _optim._muon_update_params(self.optimizer, entry["mine"], entry["group"],
                                                   peer_ptrs=push.peer_ptrs)
                    else:
                        _optim._muon_update_params(self.optimizer, entry["mine"], entry["group"],
                                                   after_group=push.push)
            else:
                _optim._muon_update_params(self.optimizer, params, entry["group"])
        for p in params:  # the caching allocator must not reuse them under the side stream
            if p.grad is not None:
                p.grad.record_stream(self._stream)
        entry["done"] = True

    # -- the rest of the step ----------------------------------------------------------------
    @torch.no_grad()
    def step(self) -> None:
        """What is left of ``optimizer.step()`` after the backward pass (no closure: the backward
        pass has already run)."""
        for entry in self._sets:
            if not entry["done"]:
                # some parameters got no gradient in this pass: the reference treats them as zeros
                # (muon.py:59-61); every rank reaches this set in the same order
                self._run(entry)
        for group in self.optimizer.param_groups:
            if not group.get("use_muon", True):
                _optim._adam_update_params(self.optimizer, group)
        if self._stream is not None:
            torch.cuda.current_stream(self._stream.device).wait_stream(self._stream)
        if self._distributed:
            for push in self._pushes:
                push.end_step()  # returns (in stream order) once every rank's writes have landed
            self._begun = False
        for entry in self._sets:
            entry["waiting"] = {id(p) for p in entry["params"]}
            entry["done"] = False

    def remove(self) -> None:
        """Detach the hooks; the optimizer is then used through its own ``step()`` again."""
        for h in self._handles:
            h.remove()
        self._handles = []
