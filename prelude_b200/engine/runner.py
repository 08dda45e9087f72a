"""The step function: one batch of (request, its next tokens) through the model.

``ModelRunner.step`` takes, for each request of the step, its next tokens and
the places among them whose logits are wanted.  Portions of prompts stand
beside single decoded tokens, cut anywhere.  It makes room in the cache, packs
the batch, runs only the tokens it was given against the cache that earlier
steps left, and returns float32 logits for the wanted places, in the order of
the entries and of their ``want`` lists.  A request's position is how many of
its tokens the cache already holds.

It is the reference's ``batch_mixed_paged``
(crates/prelude-core/src/engine/model_runner/paged_mixed.rs:13-335) with two
differences: logits come back for any wanted place instead of the last row of
every request, and room in the cache is made here rather than by the caller.
Trace replay, the scheduler and the tests all go through this one function.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages
from ..ops.library import KernelLibraryError, require_device
from ..parts.model import DecoderModel
from .batch import StepBatch, StepError, StepItem, build_step_batch, raise_on_status


@dataclass
class StepEntry:
    """One request's share of a step."""
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager):
        require_device()
        self.model, self.cache = model, cache
        self.device = model.ctx.device
        self.caches = cache.layer_caches(len(model.order))
        self.steps_run = 0
        self.last_batch: Optional[StepBatch] = None
        self.step_graphs = None             # engine.step_graph.StepGraphs: prompt steps captured piece by piece
        self.graph_steps_run = 0

    def enable_step_graphs(self, max_tokens: Optional[int] = None) -> bool:
        """Capture steps with prompt tokens piece by piece, up to ``max_tokens`` of them (default 1,024, or
        PRELUDE_STEP_GRAPH_MAX_TOKENS: longer steps keep the GPU busy longer than the host needs to launch them
        one kernel at a time, so capturing them gains nothing).  Needs the device-resident block tables;
        PRELUDE_STEP_GRAPHS=0 turns it off."""
        import os
        from .step_graph import StepGraphs
        if os.environ.get("PRELUDE_STEP_GRAPHS", "1") == "0" or not self.cache.device_tables:
            return False
        cap = int(os.environ.get("PRELUDE_STEP_GRAPH_MAX_TOKENS", "1024"))
        self.step_graphs = StepGraphs(self, cap if max_tokens is None else max_tokens)
        return True

    # -- room in the cache --------------------------------------------------------------
    def reserve(self, entries: Sequence[StepEntry]) -> List[int]:
        """Register new requests and grow every entry's cache to hold its tokens.
        All or nothing: raises OutOfPages before anything is taken when the
        step as a whole does not fit.  Returns each entry's start position."""
        cache = self.cache
        seen = set()
        demand: Dict[int, int] = {}
        new_requests = 0
        for e in entries:
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.request_id!r} brings no tokens")
            live = cache.has_request(e.request_id)
            new_requests += 0 if live else 1
            start = cache.tokens_of(e.request_id) if live else 0
            for gid, n in cache.pages_needed(e.request_id if live else None, start + len(e.tokens)).items():
                demand[gid] = demand.get(gid, 0) + n
        for gid, n in demand.items():
            free = cache.groups[gid].allocator.num_free
            if n > free:
                raise OutOfPages(f"the step needs {n} new pages in cache group {gid}, {free} of {cache.num_pages} are free")
        if new_requests > cache.slots.num_free:
            raise OutOfPages(f"the step starts {new_requests} requests, {cache.slots.num_free} state slots are free")
        starts = []
        for e in entries:
            if not cache.has_request(e.request_id):
                cache.add_request(e.request_id)
            start = cache.tokens_of(e.request_id)
            cache.grow(e.request_id, start + len(e.tokens))
            starts.append(start)
        return starts

    # -- the step -----------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], check_status: bool = True) -> torch.Tensor:
        starts = self.reserve(entries)
        items = [StepItem(e.request_id, e.tokens, s, e.want) for e, s in zip(entries, starts)]
        rids = [e.request_id for e in entries]
        spec = self.model.spec
        slots = [self.cache.slot_of(r) for r in rids]
        n_tokens = sum(len(e.tokens) for e in entries)
        sg = self.step_graphs
        if (sg is not None and n_tokens > len(entries)
                and sg.usable(n_tokens, len(entries), max(s + len(e.tokens) for e, s in zip(entries, starts)))):
            # a step with prompt tokens, replayed from its captured pieces: same kernels, fixed buffers
            graph = sg.get(n_tokens)
            graph.load(items, slots, spec.vocab_size, spec.max_positions)
            self.cache.flush_table_updates()
            self.cache.zero_fresh_state()
            logits = graph.run()
            batch = graph.batch
            self.graph_steps_run += 1
        else:
            batch = build_step_batch(items, self.cache.block_tables(rids), slots, self.device, spec.vocab_size,
                                     spec.max_positions)
            self.cache.zero_fresh_state()
            logits = self.model.forward(batch, self.caches)
            if self.cache.device_tables:
                # a launched step reads the tables it was given; the device-resident ones are kept up to date all
                # the same, so that what is queued for them stays short and a later captured step finds them current
                self.cache.flush_table_updates()
        for r in rids:
            self.cache.trim(r)
        self.steps_run += 1
        self.last_batch = batch
        if check_status:
            raise_on_status(int(batch.status.item()))
        return logits

    def finish(self, request_id: Hashable) -> None:
        """The request has ended: what it holds goes back to the pools."""
        self.cache.release(request_id)
