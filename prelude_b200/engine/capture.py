"""What a stream capture needs from the Python side.

While a stream is being captured, destroying a CUDA graph is "not permitted"
and invalidates the capture.  Graph objects of an engine that is no longer
used sit in reference cycles (graph -> recorded closures -> batch -> graph)
until Python's cycle collector finds them, and the collector runs whenever
enough objects have been allocated - in the middle of a capture as well, which
allocates plenty.  So every capture in this package runs inside
``no_collection()``: the garbage that exists is collected before the capture
begins, and the collector stays off until it has ended.
"""
from __future__ import annotations

import contextlib
import gc


@contextlib.contextmanager
def no_collection():
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        yield
    finally:
        if was_enabled:
            gc.enable()
