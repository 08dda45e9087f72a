"""Decode steps captured as CUDA graphs.

A step in which every request brings exactly one token has a fixed shape per
batch size, and several hundred small launches; it is captured once per batch
size and replayed, as in the reference
(crates/prelude-cuda/src/cuda_graph.rs:45-339: one graph per batch size, fixed
input buffers, eager fallback when a step does not fit).

What changes between replays lives in device buffers at fixed addresses:
tokens, positions, the state slot of every row (which is also the row of the
device-resident block table that the kernels read), and the sampling options.
One host-to-device copy fills them; block-table entries that changed since the
last step are written by a small scatter kernel before the replay.  Sampling
is part of the captured step, so one device-to-host copy of ``batch`` token
ids ends it.

With ``self_feeding`` the captured step ends with a kernel that makes the
sampled token the next input and moves positions on, so that steps can be
replayed back to back without the host (used to time the device alone).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..ops import kernels as K
from .batch import StepBatch, raise_on_status
from .capture import no_collection


class DecodeGraph:
    """One captured decode step for a fixed batch size."""

    def __init__(self, runner, batch_size: int, self_feeding: bool = False):
        self.runner, self.bs, self.self_feeding = runner, batch_size, self_feeding
        cache = runner.cache
        if not cache.device_tables:
            raise RuntimeError("captured decode needs device-resident block tables (max_request_tokens)")
        dev = runner.device
        bs = batch_size
        # One device buffer holds everything that changes from step to step, so that one host-to-device copy fills it:
        #   seeds int64 [bs] | counters int64 [bs] | temperatures float32 [bs] |
        #   tokens | positions | kv_len | slots (int32 [bs] each) | status int32 [1] | sampled int32 [bs]
        # (status and the sampled tokens side by side: one device-to-host copy reads both)
        # and behind it what never changes: 0..bs-1 (the request of every token, and the rows whose logits are
        # wanted) and 0..bs (cumulative query lengths).
        self.n_loaded = 8 * bs + 8 * bs + 4 * bs + 4 * (5 * bs + 1)
        total = self.n_loaded + 4 * (2 * bs + 1)
        self.buf = torch.zeros(total, dtype=torch.uint8, device=dev)
        self.host_buf = torch.zeros(self.n_loaded, dtype=torch.uint8, pin_memory=True)

        def views(b):
            o = 0
            seeds = b[o:o + 8 * bs].view(torch.int64); o += 8 * bs
            counters = b[o:o + 8 * bs].view(torch.int64); o += 8 * bs
            temps = b[o:o + 4 * bs].view(torch.float32); o += 4 * bs
            ints = b[o:o + 4 * (5 * bs + 1)].view(torch.int32)
            return seeds, counters, temps, ints

        self.seeds, self.counters, self.temps, self.ints = views(self.buf)
        self._h_seeds, self._h_counters, self._h_temps, self._h_ints = (t.numpy() for t in views(self.host_buf))
        fixed = self.buf[self.n_loaded:].view(torch.int32)
        fixed[:bs] = torch.arange(bs, dtype=torch.int32, device=dev)
        fixed[bs:] = torch.arange(bs + 1, dtype=torch.int32, device=dev)
        self.tokens, self.positions = self.ints[0:bs], self.ints[bs:2 * bs]
        self.kv_len, self.slots = self.ints[2 * bs:3 * bs], self.ints[3 * bs:4 * bs]
        self.status = self.ints[4 * bs:4 * bs + 1]
        self.sampled = self.ints[4 * bs + 1:5 * bs + 1]
        self.host_out = torch.zeros(bs + 1, dtype=torch.int32, pin_memory=True)     # status | sampled
        self._events: List[torch.cuda.Event] = []
        self.host_burst: Optional[torch.Tensor] = None      # [steps, bs] sampled tokens of a queued run of replays
        # The batch means what a launched decode step's batch means: a token's request is its index in the batch,
        # kv_len counts the token itself, the host copies are filled by load().  What differs is where the block
        # tables live: the device-resident ones have a row per state slot.
        self.batch = StepBatch(
            n_tokens=bs, n_seqs=bs, token_ids=self.tokens, positions=self.positions, token_seq=fixed[:bs],
            cu_q=fixed[bs:], q_start=self.positions, kv_len=self.kv_len, state_slots=self.slots,
            logit_rows=fixed[:bs], block_tables=dict(cache.device_tables), status=self.status,
            token_table_row=self.slots, q_lens=np.ones(bs, np.int32), q_start_host=np.zeros(bs, np.int32),
            kv_len_host=np.ones(bs, np.int32), state_slots_host=np.zeros(bs, np.int32), max_q_len=1, decode_only=True)
        self.batch.extras["captured"] = True
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches = 0
        self.logits: Optional[torch.Tensor] = None

    def _body(self) -> None:
        self.logits = self.runner.model.forward(self.batch, self.runner.caches)
        K.sample(self.logits, self.temps, self.seeds, self.counters, out=self.sampled)
        if self.self_feeding:
            K.decode_advance(self.tokens, self.positions, self.kv_len, self.counters, self.sampled,
                             self.runner.model.spec.max_positions)

    def capture(self) -> None:
        """Warm up once eagerly on the current buffer contents, then capture."""
        from ..ops import library
        saved = self.buf.clone()
        stream = torch.cuda.Stream(device=self.runner.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            self._body()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        self.buf.copy_(saved)           # a self-feeding warm-up has moved tokens, positions and counters
        before = library.launch_count
        graph = torch.cuda.CUDAGraph()
        with no_collection(), torch.cuda.graph(graph):
            self._body()
        self.launches = library.launch_count - before
        self.graph = graph
        self.buf.copy_(saved)

    def load(self, tokens: Sequence[int], positions: Sequence[int], slots: Sequence[int],
             temperatures: Sequence[float], seeds: Sequence[int], counters: Sequence[int]) -> None:
        """Fill the fixed buffers for the next replay (one host-to-device copy).  The status word travels with
        them as zero, so a code that a kernel raised in an earlier step does not outlive it."""
        bs = self.bs
        h = self._h_ints
        h[0:bs], h[bs:2 * bs], h[3 * bs:4 * bs] = tokens, positions, slots
        h[2 * bs:3 * bs] = h[bs:2 * bs] + 1                 # tokens in the cache after this step
        h[4 * bs] = 0
        self._h_temps[:] = temperatures
        self._h_seeds[:] = [x & (2**63 - 1) for x in seeds]
        self._h_counters[:] = counters
        self.buf[:self.n_loaded].copy_(self.host_buf, non_blocking=True)
        b = self.batch
        b.q_start_host, b.kv_len_host = h[bs:2 * bs].copy(), h[2 * bs:3 * bs].copy()
        b.state_slots_host = h[3 * bs:4 * bs].copy()

    @property
    def h2d_bytes(self) -> int:
        return self.host_buf.numel()

    @property
    def d2h_bytes(self) -> int:
        return self.host_out.numel() * 4

    def replay(self) -> None:
        if self.graph is None:
            self.capture()
        self.graph.replay()

    def replay_burst(self, steps: int, stop=None, ahead: int = 3) -> List[List[int]]:
        """Queue up to ``steps`` replays of a self-feeding graph - every step's input is the step before's
        output, on the device - and return the sampled tokens of the steps that ran.  No more than ``ahead``
        replays are queued beyond the one the device is working on; before each further one the host asks
        ``stop()`` and ends the run early when it says so (a request has arrived or been aborted meanwhile)."""
        if not self.self_feeding:
            raise RuntimeError("a run of replays needs a self-feeding graph")
        if self.host_burst is None or self.host_burst.shape[0] < steps:
            self.host_burst = torch.zeros((max(steps, 8), self.bs), dtype=torch.int32, pin_memory=True)
        while len(self._events) < steps:
            self._events.append(torch.cuda.Event())
        ran = 0
        for j in range(steps):
            if j >= ahead:
                self._events[j - ahead].synchronize()
                if stop is not None and stop():
                    break
            self.replay()
            self.host_burst[j].copy_(self.sampled, non_blocking=True)   # in stream order, before the next replay overwrites it
            self._events[j].record()
            ran += 1
        self.host_out[:1].copy_(self.status, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        raise_on_status(int(self.host_out[0]))
        return self.host_burst[:ran].tolist()

    def fetch(self) -> List[int]:
        """Sampled tokens of the last replay (one device-to-host copy, then a wait)."""
        self.host_out.copy_(self.ints[4 * self.bs:], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        out = self.host_out.tolist()
        raise_on_status(out[0])
        return out[1:]


class DecodeGraphs:
    """Captured steps by batch size, made when first needed.  ``self_feeding`` graphs end
    with the kernel that turns the sampled tokens into the next step's input, so several
    replays can be queued without the host in between."""

    def __init__(self, runner, max_batch_size: int, self_feeding: bool = False):
        self.runner, self.max_bs, self.self_feeding = runner, max_batch_size, self_feeding
        self.graphs: Dict[int, DecodeGraph] = {}

    def usable(self, batch_size: int, longest: int) -> bool:
        cache = self.runner.cache
        return (1 <= batch_size <= self.max_bs and bool(cache.device_tables)
                and longest <= cache.table_width * cache.page_size)

    def get(self, batch_size: int) -> DecodeGraph:
        g = self.graphs.get(batch_size)
        if g is None:
            g = self.graphs[batch_size] = DecodeGraph(self.runner, batch_size, self_feeding=self.self_feeding)
        return g
