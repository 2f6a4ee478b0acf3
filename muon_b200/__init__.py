"""muon_b200 — the Muon optimizer step on NVIDIA B200 (sm_100a).

Drop-in for the public names of thib-s/Muon's ``muon`` module. All arithmetic runs in
``libmuon_b200.so`` (hand-written CUDA behind a C ABI, see ``include/muon_b200.h``);
importing this package fails if that library has not been built.
"""
from ._lib import MuonB200Error, device_status  # noqa: F401  (import fails loudly without the library)
from .backward_overlap import StepInBackward  # noqa: F401
from .checkpoint import consolidated_state_dict, load_consolidated_state_dict  # noqa: F401
from .engine import get_backend, get_ns_mode, mark_grad_ready, set_ns_mode  # noqa: F401
from .ownership import get_ownership, set_ownership  # noqa: F401
from .sharded import ShardedMuon  # noqa: F401
from .ops import (  # noqa: F401
    adam_update,
    muon_update,
    ns_line_1,
    ns_line_2,
    ns_line_3,
    zeropower_via_newtonschulz5,
)
from .optim import (  # noqa: F401
    Muon,
    MuonWithAuxAdam,
    SingleDeviceMuon,
    SingleDeviceMuonWithAuxAdam,
)

__all__ = [
    "Muon", "SingleDeviceMuon", "MuonWithAuxAdam", "SingleDeviceMuonWithAuxAdam",
    "muon_update", "adam_update", "zeropower_via_newtonschulz5",
    "ns_line_1", "ns_line_2", "ns_line_3",
    "set_ns_mode", "get_ns_mode", "get_backend", "device_status", "MuonB200Error",
    "mark_grad_ready", "StepInBackward", "consolidated_state_dict", "load_consolidated_state_dict",
    "set_ownership", "get_ownership", "ShardedMuon",
]
