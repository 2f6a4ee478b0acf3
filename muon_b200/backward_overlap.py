"""Start the Muon update of a parameter set while the backward pass is still running.

The reference updates everything in ``optimizer.step()``, after the whole backward pass
(muon.py:81-101). For the single-device classes the update of one parameter depends on nothing
but that parameter, its gradient and its momentum, so it can start as soon as the gradient
exists. ``StepInBackward`` registers a hook on every Muon parameter
(``Tensor.register_post_accumulate_grad_hook``); when the gradients of all same-shape parameters
of a group have been accumulated, their grouped update (prologue, Newton-Schulz, epilogue: the
same calls ``step()`` makes) is enqueued on a side stream that waits for the backward stream up to
that point. ``StepInBackward.step()`` then updates what is left (parameters that received no
gradient, Adam groups) and joins the side stream. The arithmetic and its grouping are those of
``optimizer.step()``, so the parameters come out bit for bit the same.

Use one backward pass per step (no gradient accumulation over several backward passes), and call
``step()`` of this object instead of the optimizer's. The distributed classes are not supported:
their exchange needs every rank to enter the same collectives in the same order.

    opt = SingleDeviceMuonWithAuxAdam(groups)
    overlap = StepInBackward(opt)
    loss.backward()        # updates start inside
    overlap.step()         # finishes the step
"""
from __future__ import annotations

import torch

from . import optim as _optim


class StepInBackward:
    def __init__(self, optimizer):
        if not isinstance(optimizer, (_optim.SingleDeviceMuon, _optim.SingleDeviceMuonWithAuxAdam)):
            raise TypeError("StepInBackward supports SingleDeviceMuon and SingleDeviceMuonWithAuxAdam; "
                            "the distributed classes exchange parameters in a fixed order")
        self.optimizer = optimizer
        self._sets = []        # dicts: group, params (one shape bucket), waiting (ids), done
        self._set_of = {}      # id(param) -> its set
        self._handles = []
        self._stream = None
        for group in optimizer.param_groups:
            if not group.get("use_muon", True):
                continue
            for plist in _optim._bucket_by_shape(group["params"]).values():
                entry = dict(group=group, params=plist, waiting={id(p) for p in plist}, done=False)
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
        if params[0].is_cuda:
            device = params[0].device
            current = torch.cuda.current_stream(device)
            if self._stream is None:
                self._stream = torch.cuda.Stream(device=device)
            # Everything the backward pass has enqueued so far (these gradients, and the last reads
            # of these parameters) comes first.
            self._stream.wait_stream(current)
            with torch.cuda.stream(self._stream):
                _optim._muon_update_params(self.optimizer, params, entry["group"])
            for p in params:  # the caching allocator must not reuse them under the side stream
                p.grad.record_stream(self._stream)
        else:
            _optim._muon_update_params(self.optimizer, params, entry["group"])
        entry["done"] = True

    # -- the rest of the step ----------------------------------------------------------------
    @torch.no_grad()
    def step(self) -> None:
        """What is left of ``optimizer.step()`` after the backward pass (no closure: the backward
        pass has already run)."""
        for entry in self._sets:
            if not entry["done"]:
                # some parameters got no gradient in this pass: the reference treats them as zeros
                self._run(entry)
        for group in self.optimizer.param_groups:
            if not group.get("use_muon", True):
                _optim._adam_update_params(self.optimizer, group)
        if self._stream is not None:
            torch.cuda.current_stream(self._stream.device).wait_stream(self._stream)
        for entry in self._sets:
            entry["waiting"] = {id(p) for p in entry["params"]}
            entry["done"] = False

    def remove(self) -> None:
        """Detach the hooks; the optimizer is then used through its own ``step()`` again."""
        for h in self._handles:
            h.remove()
        self._handles = []
