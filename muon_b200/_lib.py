"""ctypes binding of ``libmuon_b200.so`` (declared in ``include/muon_b200.h``).

The library is the only compute path: if it cannot be loaded, importing this module
raises, and nothing in the package falls back to PyTorch or CPU arithmetic.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_int64, c_void_p

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libmuon_b200.so")

F32, BF16, F16, F64 = 0, 1, 2, 3
NS_AOL4, NS_CLASSIC5, NS_AOL4_FP8 = 0, 1, 2
NS_HAVE_SUMSQ = 0x100  # MUON_B200_NS_HAVE_SUMSQ

ERR_NAMES = {
    -1: "INVALID_ARG",
    -2: "ALIGNMENT",
    -3: "CUDA",
    -4: "UNSUPPORTED",
    -5: "DEVICE_TIMEOUT",
}


class MuonB200Error(RuntimeError):
    """A libmuon_b200 entry point returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"muon_b200 error {ERR_NAMES.get(code, code)}: {message}")
        self.code = code


class NsLayout(ctypes.Structure):
    _fields_ = [(name, c_int64) for name in (
        "total_bytes", "x_offset_bytes", "c_offset_bytes", "a_offset_bytes", "b_offset_bytes",
        "partials_offset_bytes", "ldn", "x_bs", "ldm", "a_bs", "x8_offset_bytes", "e8_offset_bytes",
        "ld8n", "ld8m", "sumsq_offset_bytes", "sumsq_bs")]


# name -> (restype, argtypes); mirrors include/muon_b200.h one to one.
PROTOTYPES = {
    "muon_b200_version": (c_int, []),
    "muon_b200_last_error": (c_char_p, []),
    "muon_b200_device_status": (c_int, [POINTER(c_int), c_int]),
    "muon_b200_set_reserved_sms": (c_int, [c_int]),
    "muon_b200_get_reserved_sms": (c_int, []),
    "muon_b200_set_graph_replay": (c_int, [c_int]),
    "muon_b200_get_graph_replay": (c_int, []),
    "muon_b200_ns_run_static": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int,
                                        c_int64, c_int64, c_int, c_int, POINTER(c_float), c_float,
                                        c_void_p]),
    "muon_b200_zeropower": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p,
                                    c_int64, c_int64, c_void_p, c_int64, c_int, c_int, POINTER(c_float),
                                    c_float, c_void_p]),
    "muon_b200_zeropower_scratch_bytes": (c_int64, [c_int, c_int64, c_int64, c_int]),
    "muon_b200_cast_bf16": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int64,
                                    c_int64, c_int, c_int, c_float, c_void_p]),
    "muon_b200_ns_static_scratch_bytes": (c_int64, []),
    "muon_b200_ns_static_required_bytes": (c_int64, [c_int, c_int64, c_int64]),
    "muon_b200_ipc_export": (c_int, [c_void_p, c_void_p, POINTER(c_int64), POINTER(c_int64)]),
    "muon_b200_ipc_open": (c_int, [c_void_p, POINTER(c_void_p)]),
    "muon_b200_ipc_close": (c_int, [c_void_p]),
    "muon_b200_push_copies": (c_int, [POINTER(c_void_p), c_int, c_void_p, c_int64, c_void_p]),
    "muon_b200_kernel_kinds": (c_int, []),
    "muon_b200_launch_counts": (c_int, [POINTER(c_int64), c_int]),
    "muon_b200_timing_enable": (c_int, [c_int]),
    "muon_b200_timing_collect": (c_int, [POINTER(c_double), POINTER(c_double), POINTER(c_int64), c_int]),
    "muon_b200_timing_collect_records": (c_int, [c_int, POINTER(c_int), POINTER(c_int64), POINTER(c_double),
                                                 POINTER(c_double), POINTER(c_int)]),
    "muon_b200_ns_line1": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int,
                                   c_int64, c_int64, c_void_p]),
    "muon_b200_ns_line1_scratch": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int,
                                           c_int64, c_int64, c_void_p, c_int64, c_void_p]),
    "muon_b200_ns_line1_scratch_bytes": (c_int64, [c_int, c_int64, c_int64]),
    "muon_b200_ns_line2": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int,
                                   c_int64, c_float, c_float, c_int, c_void_p]),
    "muon_b200_ns_line3": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p,
                                   c_int64, c_int64, c_int, c_int64, c_int64, c_float, c_void_p]),
    "muon_b200_ns_workspace_layout": (c_int, [c_int, c_int64, c_int64, POINTER(NsLayout)]),
    "muon_b200_ns_workspace_layout_mode": (c_int, [c_int, c_int64, c_int64, c_int, POINTER(NsLayout)]),
    "muon_b200_ns_run": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int, POINTER(c_float),
                                 c_float, POINTER(c_int), c_void_p]),
    "muon_b200_ns_run_update": (c_int, [c_void_p, c_int, c_int, POINTER(c_float), c_float, POINTER(c_void_p),
                                        c_int, c_int64, c_int64, c_int, c_double, c_double, c_double,
                                        c_void_p]),
    "muon_b200_prologue": (c_int, [POINTER(c_void_p), POINTER(c_void_p), c_int, c_int64, c_int64,
                                   c_int, c_double, c_int, c_void_p, c_int64, c_int64, c_int,
                                   c_void_p]),
    "muon_b200_prologue_sumsq": (c_int, [POINTER(c_void_p), POINTER(c_void_p), c_int, c_int64, c_int64,
                                         c_int, c_double, c_int, c_void_p, c_int64, c_int64, c_int,
                                         c_void_p, c_int64, c_void_p]),
    "muon_b200_epilogue": (c_int, [POINTER(c_void_p), c_int, c_int64, c_int64, c_int, c_void_p,
                                   c_int64, c_int64, c_int, c_double, c_double, c_double, c_void_p]),
    "muon_b200_epilogue_push": (c_int, [POINTER(c_void_p), POINTER(c_void_p), c_int, c_int, c_int64, c_int64,
                                        c_int, c_void_p, c_int64, c_int64, c_int, c_double, c_double,
                                        c_double, c_void_p]),
    "muon_b200_muon_step": (c_int, [POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p), c_int,
                                    c_int64, c_int64, c_int, c_double, c_double, c_double, c_int,
                                    c_double, c_int, c_int, POINTER(c_float), c_float, c_void_p,
                                    c_int64, c_void_p]),
    "muon_b200_adam": (c_int, [POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p),
                               POINTER(c_void_p), POINTER(c_int64), POINTER(c_int64), c_int, c_int,
                               c_double, c_double, c_double, c_double, c_double, c_void_p]),
}


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing. Build it with `python muon_b200/build.py` (needs nvcc); "
            "muon_b200 has no fallback path without its CUDA library.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


def check(rc: int) -> None:
    if rc != 0:
        raise MuonB200Error(rc, lib.muon_b200_last_error().decode("utf-8", "replace"))


def ptr_array(ptrs) -> ctypes.Array:
    return (c_void_p * len(ptrs))(*ptrs)


def i64_array(vals) -> ctypes.Array:
    return (c_int64 * len(vals))(*vals)


def device_status(reset: bool = True) -> int:
    """Synchronises the device and returns the kernels' status word (0 = healthy)."""
    st = c_int(0)
    lib.muon_b200_device_status(ctypes.byref(st), 1 if reset else 0)
    return st.value


KERNEL_KINDS = ("ns_line1", "ns_line2", "ns_line3", "prologue", "epilogue", "aol_rescale",
                "fro_normalize", "adam")


def launch_counts() -> dict:
    """Kernel launches issued by the library in this process, per kernel kind."""
    n = len(KERNEL_KINDS)
    buf = (c_int64 * n)()
    check(lib.muon_b200_launch_counts(buf, n))
    return dict(zip(KERNEL_KINDS, list(buf)))


def timing_enable(on: bool) -> None:
    check(lib.muon_b200_timing_enable(1 if on else 0))


def timing_collect() -> dict:
    """{kind: (device ms, work units, launches)} since the last collect (see the header)."""
    n = len(KERNEL_KINDS)
    ms, work, cnt = (c_double * n)(), (c_double * n)(), (c_int64 * n)()
    check(lib.muon_b200_timing_collect(ms, work, cnt, n))
    return {k: (ms[i], work[i], cnt[i]) for i, k in enumerate(KERNEL_KINDS)}


def timing_collect_records(max_records: int = 1 << 16) -> list:
    """[(kind, tag, device ms, work units)] per launch since the last collect (see the header)."""
    kinds, tags = (c_int * max_records)(), (c_int64 * max_records)()
    ms, work, n = (c_double * max_records)(), (c_double * max_records)(), c_int(0)
    check(lib.muon_b200_timing_collect_records(max_records, kinds, tags, ms, work, ctypes.byref(n)))
    return [(KERNEL_KINDS[kinds[i]], tags[i], ms[i], work[i]) for i in range(n.value)]


def ns_layout(batch: int, m: int, n: int, mode: int = NS_AOL4) -> NsLayout:
    out = NsLayout()
    check(lib.muon_b200_ns_workspace_layout_mode(batch, m, n, mode, ctypes.byref(out)))
    return out
