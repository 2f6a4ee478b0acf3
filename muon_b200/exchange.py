"""Cross-rank exchange of updated parameters for the distributed optimizers.

The reference ends every window with ``dist.all_gather`` of the freshly updated parameters
(muon.py:68). Two transports implement that exchange here:

``nccl``  the same ``dist.all_gather`` call, issued asynchronously. NCCL moves the data with
          copy kernels that need SMs; the Newton-Schulz GEMMs are persistent grids that fill
          the device, so the two compete and only part of the transfer is hidden.

``st``    same mappings as ``ce`` below, but nothing is copied afterwards: the update epilogue
          kernel itself stores every new parameter value into the W-1 peer copies as it computes
          it (``muon_b200_epilogue_push``, plain global stores over NVLink). The exchange of a
          launch group is finished when its epilogue kernel is, that kernel runs beside the next
          group's GEMMs, and the copy engines stay free for host-to-device traffic. Up to 8 ranks.

``ce``    every rank maps the other ranks' parameter allocations on its own device (CUDA IPC
          handles opened with peer access, ``muon_b200_ipc_export`` / ``muon_b200_ipc_open``)
          and, as soon as some of its own parameters are updated, pushes them to the peers
          with device-to-device copies on a side stream (``muon_b200_push_copies``). Those
          copies run on the copy engines over NVLink and take no SM, so they overlap the
          remaining Newton-Schulz work. Two tiny NCCL all-reduces bracket the step: the first
          makes sure every rank has reached ``step()`` (and, in stream order, finished whatever
          read the parameters before) before any push lands in its memory; the second returns
          only after every rank's pushes have completed, which gives ``step()`` the reference's
          post-condition that all ranks hold all updated parameters.

``MUON_B200_EXCHANGE`` selects ``nccl``, ``ce``, or ``auto`` (default). ``auto`` means ``ce``; when
the peers cannot be mapped it raises and names the reason instead of switching transports behind
the caller's back: the ``nccl`` transport is slower (its copy kernels compete with the GEMMs for
SMs) and an early version of it stopped twice in a 2-GPU run for a reason that was never found, so
it is only used when asked for by name. CPU tensors (the gloo test ranks) always use
``all_gather``. The ``ce`` transport needs parameters that live in plain ``cudaMalloc`` blocks
(PyTorch's default allocator without expandable segments) and stay allocated while the optimizer
lives.
"""
from __future__ import annotations

import ctypes
import os
import weakref

import torch
import torch.distributed as dist

DEFAULT_MODE = "auto"

# CUDA refuses to open an IPC handle twice in one process, so mappings are shared process-wide:
# handle bytes -> [base address on this device, number of PeerPush objects using it].
_OPEN_HANDLES: dict = {}


def _mode() -> str:
    m = os.environ.get("MUON_B200_EXCHANGE", DEFAULT_MODE).lower()
    if m not in ("auto", "ce", "st", "nccl"):
        raise ValueError(f"MUON_B200_EXCHANGE must be auto, ce, st or nccl, got {m!r}")
    return m


MAX_STORE_PEERS = 7  # peer copies one launch of the epilogue kernel can address


class PeerPush:
    """Addresses of one param group's tensors in every other rank's memory + a copy stream."""

    def __init__(self, params):
        from ._lib import lib

        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.device = params[0].device
        exported, errors = [], []
        with torch.cuda.device(self.device):
            for p in params:
                handle = ctypes.create_string_buffer(64)
                off = ctypes.c_int64(0)
                rc = lib.muon_b200_ipc_export(p.data_ptr(), handle, ctypes.byref(off), None)
                if rc != 0 or not p.is_contiguous():
                    errors.append(lib.muon_b200_last_error().decode() if rc else "non-contiguous parameter")
                    break
                exported.append((handle.raw, off.value, p.numel() * p.element_size()))
        gathered = [None] * self.world
        dist.all_gather_object(gathered, (exported, errors))
        errors = [e for g in gathered for e in g[1]]
        # Every rank must hold the same parameters in the same order, or ownership (a function of the position in the list)
        # and the pushes would pair up different tensors: compare the byte sizes rank by rank.
        sizes = [[item[2] for item in g[0]] for g in gathered]
        if not errors and any(s != sizes[0] for s in sizes):
            bad = [r for r, s in enumerate(sizes) if s != sizes[0]]
            raise RuntimeError(f"muon_b200: ranks {bad} hold a different parameter list than rank 0 "
                               "(count, order or sizes differ); the distributed optimizer needs "
                               "identical, identically ordered parameters on every rank")
        self.ptrs = None  # ptrs[r][i]: address of parameter i in rank r's memory, mapped here
        self._opened = {}
        if not errors:
            try:
                with torch.cuda.device(self.device):
                    self.ptrs = [self._map(items) if r != self.rank else None
                                 for r, (items, _) in enumerate(gathered)]
            except RuntimeError as e:
                errors.append(str(e))
                self.ptrs = None
        ok = [None] * self.world
        dist.all_gather_object(ok, self.ptrs is not None)
        self.ok = all(ok)
        self.error = "; ".join(errors) if errors else (None if self.ok else "a peer could not map this rank")
        if not self.ok:
            self.close()
            return
        self.nbytes = [e[2] for e in exported]
        # The peers hold the addresses exported above: a parameter whose storage is replaced later
        # (`p.data = ...`, a `.to()` of the module) would silently stop receiving its updates.
        self._params = list(params)
        self._exported_ptrs = [p.data_ptr() for p in params]
        self._token = torch.zeros(1, device=self.device)
        self.index = {id(p): i for i, p in enumerate(params)}
        # Peers in the order r+1, r+2, ... so that ranks do not all start on the same receiver.
        self.peers = [(self.rank + k) % self.world for k in range(1, self.world)]
        # One copy stream per peer: the copies to different peers run on different copy engines
        # at the same time. A single stream of back-to-back copies reached 390 GB/s per GPU in an
        # 8-GPU all-to-all, about half of what the NVLink ports carry.
        self.streams = [torch.cuda.Stream(device=self.device) for _ in self.peers]

    def _map(self, items):
        from ._lib import lib
        out = []
        for handle, offset, _ in items:
            base = self._opened.get(handle)
            if base is None:
                shared = _OPEN_HANDLES.get(handle)
                if shared is None:
                    ptr = ctypes.c_void_p(0)
                    rc = lib.muon_b200_ipc_open(handle, ctypes.byref(ptr))
                    if rc != 0:
                        raise RuntimeError(lib.muon_b200_last_error().decode())
                    shared = _OPEN_HANDLES[handle] = [ptr.value, 0]
                shared[1] += 1
                base = self._opened[handle] = shared[0]
            out.append(base + offset)
        return out

    def close(self) -> None:
        """Drop this object's use of its mappings; a mapping is removed with its last user."""
        _release_handles(self._opened)
        self._opened = {}
        self.ptrs = None

    def begin_step(self) -> None:
        """All ranks are inside step() (stream-ordered after their earlier work) from here on."""
        for i, p in enumerate(self._params):
            if p.data_ptr() != self._exported_ptrs[i]:
                raise RuntimeError(
                    f"muon_b200: the storage of parameter {i} {tuple(p.shape)} was replaced after the "
                    "optimizer mapped it into the other ranks (copy-engine exchange); keep parameter "
                    "storages in place, or set MUON_B200_EXCHANGE=nccl")
        dist.all_reduce(self._token)

    def push(self, updated, ready=None) -> None:
        """Copy each freshly updated local parameter into every peer's copy of it, once `ready`
        (default: everything enqueued so far on the current stream) has completed."""
        from ._lib import check, lib, ptr_array
        if ready is None:
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(self.device))
        with torch.cuda.device(self.device):
            for r, stream in zip(self.peers, self.streams):
                stream.wait_event(ready)
                for p in updated:
                    i = self.index[id(p)]
                    check(lib.muon_b200_push_copies(ptr_array([self.ptrs[r][i]]), 1, p.data_ptr(),
                                                    self.nbytes[i], stream.cuda_stream))

    def peer_ptrs(self, p) -> list:
        """Addresses, on this device, of parameter `p` in every other rank's memory."""
        i = self.index[id(p)]
        return [self.ptrs[r][i] for r in self.peers]

    def end_step(self) -> None:
        """Returns (in stream order) once every rank's pushes have landed."""
        current = torch.cuda.current_stream(self.device)
        for stream in self.streams:
            current.wait_stream(stream)
        dist.all_reduce(self._token)


def _release_handles(opened: dict) -> None:
    from ._lib import lib
    for handle, base in opened.items():
        shared = _OPEN_HANDLES.get(handle)
        if shared is None:
            continue
        shared[1] -= 1
        if shared[1] <= 0:
            lib.muon_b200_ipc_close(base)
            del _OPEN_HANDLES[handle]


def _close_all(cache: dict) -> None:
    for push in cache.values():
        if push is not None:
            push.close()
    cache.clear()


def get_peer_push(optimizer, group):
    """PeerPush of `group`, built collectively on first use; None when the NCCL/gloo gather is to
    be used. Every rank takes the same decision. The cache is keyed on the parameters' storage
    addresses (``load_state_dict`` replaces the group dicts, not the parameters) and closed when
    the optimizer is collected."""
    cache = optimizer.__dict__.get("_muon_b200_exchange")
    if cache is None:
        cache = optimizer.__dict__["_muon_b200_exchange"] = {}
        weakref.finalize(optimizer, _close_all, cache)
    params = group["params"]
    key = tuple(p.data_ptr() for p in params)
    if key in cache:
        return cache[key]
    mode = _mode()
    usable = mode != "nccl" and dist.get_world_size() > 1 and all(p.is_cuda for p in params) \
        and "nccl" in str(dist.get_backend())
    push = None
    if usable:
        push = PeerPush(params)
        if not push.ok:
            raise RuntimeError(
                f"muon_b200: the copy-engine exchange cannot map the other ranks' parameters ({push.error}). "
                "Keep parameters in plain cudaMalloc blocks (no expandable segments), or ask for the "
                "all_gather transport by name with MUON_B200_EXCHANGE=nccl")
    if push is not None:
        push.mode = "st" if mode == "st" and len(push.peers) <= MAX_STORE_PEERS else "ce"
    cache[key] = push
    return push
