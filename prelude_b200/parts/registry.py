"""Registries of parts, and the interface every part has.

A part is built in two stages so that the list of tensors a model needs is
known before anything touches a GPU:

    part = PartClass(spec, prefix)        # cheap: sizes and constants only
    part.tensors()                        # {tensor name: TensorReq}
    part.load(get, ctx)                   # get(name) -> CPU tensor; ctx: RunContext

Families and the calls the model makes on their members:

  norm          ``forward(x) -> y`` and ``add_forward(x, res) -> y`` (res += x in
                place, float32; y = norm(res) in the run's type; x may be None).
  position      what its mixers understand; the mixer owns the use of it.  The attention
                mixer reads ``cos`` and ``sin`` (float32 [positions, rotary_dim / 2], or
                None: no rotation), ``rotary_dim``, and ``interleaved`` (absent or False:
                angle j turns elements j and j + rotary_dim / 2; True: 2 j and 2 j + 1).
  mixer         ``cache_need() -> KvPagesNeed | StateNeed | None`` and
                ``forward(x, batch, cache, write_cache) -> y`` with x, y [T, hidden].
  feed_forward  ``forward(x) -> y``.
  block         ``forward(delta, res, batch, cache, write_cache) -> delta'``: ``res``
                is the float32 residual stream, updated in place; ``delta`` is what
                the previous block left to be added (None for the first).
  embedding     ``forward(batch) -> res``: the float32 residual stream [T, hidden] that
                the step's tokens start from; ``table`` is what a tied head may take.
  head          ``tensors() -> (required, optional)``, ``load(get, ctx, embedding)`` and
                ``forward(x) -> logits``: x [W, hidden] are the wanted rows after the
                final norm, logits float32 [W, vocab].

Any part may carry ``capturable = False``: it then decides on the host from data that
only the device has during a replay (a loop over requests, a branch on a value), so a
step through it cannot be recorded as a CUDA graph; the engine launches such a model's
steps kernel by kernel (``RuntimeCaps.cuda_graph``).

A part takes every size and constant from its spec and never looks at the
model around it.  A new part: write its spec dataclass with a ``kind`` string,
write the class, decorate it with ``@register_part(family, kind)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch

FAMILIES = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")
_PARTS: Dict[Tuple[str, str], type] = {}


def register_part(family: str, kind: str) -> Callable:
    if family not in FAMILIES:
        raise ValueError(f"unknown part family {family!r}; families: {FAMILIES}")

    def deco(cls):
        _PARTS[(family, kind)] = cls
        return cls
    return deco


def unregister_part(family: str, kind: str) -> None:
    _PARTS.pop((family, kind), None)


def part_class(family: str, kind: str) -> type:
    try:
        return _PARTS[(family, kind)]
    except KeyError:
        known = sorted(k for f, k in _PARTS if f == family)
        raise KeyError(f"no {family} part of kind {kind!r} is registered; known: {known}") from None


def make_part(family: str, spec, prefix: str):
    return part_class(family, spec.kind)(spec, prefix)


@dataclass(frozen=True)
class RunContext:
    """Where and in which type a model runs.  ``dtype`` is torch.float32 (the
    true 32-bit path: every matrix, activation and cache page in float32, all
    products on the float32 units) or torch.bfloat16 (the serving path)."""
    device: torch.device
    dtype: torch.dtype


@dataclass(frozen=True)
class RuntimeCaps:
    """What the engine may do with a model, put together from what its parts say
    (the reference keeps the same record per architecture,
    crates/prelude-core/src/engine/types.rs:152-160, and switches captured steps
    off where a part cannot be recorded, crates/prelude-cuda/src/executor.rs:38-42)."""
    kv_cache: bool            # some layer keeps keys and values in pages
    paged_attention: bool     # ... and reads them through block tables
    varlen: bool              # steps may mix portions of different lengths (every part here takes ragged batches)
    state_slots: bool         # some layer keeps fixed-size state per request
    cuda_graph: bool          # every part can be recorded: decode steps and prompt steps may be captured


def capturable(part) -> bool:
    """Whether a part (and the parts it is made of, which it lists in ``parts()``) can be recorded in a CUDA graph."""
    if not getattr(part, "capturable", True):
        return False
    inner = getattr(part, "parts", None)
    return all(capturable(p) for p in inner()) if callable(inner) else True


@dataclass(frozen=True)
class KvPagesNeed:
    """A mixer that keeps keys and values of ``n_kv_heads`` x ``head_dim`` per
    token in pages; ``window`` set means only the last ``window`` tokens are
    ever read again."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps one tensor of fixed ``shape`` per request."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
