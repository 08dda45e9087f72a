"""A timeline of a step's kernels: when each started, when the kernel before it had finished, when its input
had arrived, when it was done.

The kernels hold marks that are compiled in only when the library is built with PRELUDE_TIMELINE=1 (set it
before the first import; the build then makes a second library beside the ordinary one).  A mark stores the
device-wide nanosecond clock, by thread 0 of a grid's first block and of its last.  ``enable()`` hands the
kernels a record to write to; ``read()`` returns what they wrote, in the order of the clock.

The reference wraps its layers in NVTX ranges and reads a profiler's trace (crates/prelude-core/src/profiling.rs:10-55,
benchmark/profile.sh); marks inside the kernels show what a trace cannot: how long a kernel that was launched
ahead of time sat waiting for the one before it, and how long its input took to arrive after that.
"""
from __future__ import annotations

import ctypes
from typing import List, NamedTuple, Optional

import torch

from . import library as _l

UNITS = ("norm", "gemm_stream", "rope", "attention_decode")
KERNELS = {1: "add_rmsnorm", 2: "gemm_stream", 3: "qknorm_rope_kvwrite", 4: "attention_decode"}
MARKS = {0: "entry", 1: "after_wait", 2: "input", 3: "done", 4: "exit"}
CAPACITY = 8192

_record: Optional[torch.Tensor] = None


class Mark(NamedTuple):
    kernel: str
    mark: str
    last_block: bool
    ns: int


def available() -> bool:
    """Whether the loaded library was built with the marks in."""
    return hasattr(_l.library(), "pb_timeline_set_norm")


def enable(device="cuda:0") -> None:
    global _record
    lib = _l.library()
    if not available():
        raise _l.KernelLibraryError("this library has no timeline marks: set PRELUDE_TIMELINE=1 before the first import")
    _record = torch.zeros(1 + CAPACITY, dtype=torch.int64, device=device)
    for unit in UNITS:
        fn = getattr(lib, f"pb_timeline_set_{unit}")
        fn.argtypes, fn.restype = [ctypes.c_void_p], ctypes.c_int
        if fn(_record.data_ptr()) != 0:
            raise _l.KernelLibraryError(f"cannot hand the timeline record to {unit}")


def reset() -> None:
    if _record is not None:
        _record.zero_()


def read() -> List[Mark]:
    if _record is None:
        return []
    host = _record.cpu().tolist()
    n = min(host[0] & 0xFFFFFFFF, CAPACITY)
    out = []
    for word in host[1:1 + n]:
        word &= (1 << 64) - 1
        out.append(Mark(KERNELS.get(word >> 56, str(word >> 56)), MARKS.get((word >> 52) & 0xF, "?"),
                        bool((word >> 51) & 1), word & ((1 << 51) - 1)))
    out.sort(key=lambda m: m.ns)
    return out
