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
from .batch import StepBatch
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
        # int32 block: tokens | positions | slots | logit_rows(arange) | cu_q(arange) | status
        self.n_int = 3 * bs
        self.ints = torch.zeros(5 * bs + 2, dtype=torch.int32, device=dev)
        self.ints[3 * bs:4 * bs] = torch.arange(bs, dtype=torch.int32, device=dev)
        self.ints[4 * bs:5 * bs + 1] = torch.arange(bs + 1, dtype=torch.int32, device=dev)
        self.tokens, self.positions, self.slots = self.ints[0:bs], self.ints[bs:2 * bs], self.ints[2 * bs:3 * bs]
        self.status = self.ints[5 * bs + 1:5 * bs + 2]
        self.temps = torch.zeros(bs, dtype=torch.float32, device=dev)
        self.seeds = torch.zeros(bs, dtype=torch.int64, device=dev)
        self.counters = torch.zeros(bs, dtype=torch.int64, device=dev)
        self.sampled = torch.zeros(bs, dtype=torch.int32, device=dev)
        self.host_ints = torch.zeros(3 * bs, dtype=torch.int32, pin_memory=True)
        self.host_samp = torch.zeros(3 * bs, dtype=torch.int64, pin_memory=True)   # temps bits | seeds | counters
        self.dev_samp = torch.zeros(3 * bs, dtype=torch.int64, device=dev)
        self.host_out = torch.zeros(bs + 1, dtype=torch.int32, pin_memory=True)
        self.host_burst: Optional[torch.Tensor] = None      # [steps, bs] sampled tokens of a queued run of replays
        self.batch = StepBatch(
            n_tokens=bs, n_seqs=bs, token_ids=self.tokens, positions=self.positions, token_seq=self.slots,
            cu_q=self.ints[4 * bs:5 * bs + 1], q_start=self.positions, kv_len=self.positions,
            state_slots=self.slots, logit_rows=self.ints[3 * bs:4 * bs], block_tables=dict(cache.device_tables),
            status=self.status, q_lens=np.ones(bs, np.int32), max_q_len=1, decode_only=True)
        self.batch.extras["captured"] = True
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches = 0
        self.logits: Optional[torch.Tensor] = None

    def _body(self) -> None:
        # temps travel as the low 32 bits of an int64 word
        self.temps.copy_(self.dev_samp[:self.bs].to(torch.int32).view(torch.float32))
        self.seeds.copy_(self.dev_samp[self.bs:2 * self.bs])
        self.counters.copy_(self.dev_samp[2 * self.bs:])
        self.logits = self.runner.model.forward(self.batch, self.runner.caches)
        out = K.sample(self.logits, self.temps, self.seeds, self.counters)
        self.sampled.copy_(out)
        if self.self_feeding:
            K.decode_advance(self.tokens, self.positions, None, self.sampled, self.runner.model.spec.max_positions)
            self.dev_samp[2 * self.bs:] += 1

    def capture(self) -> None:
        """Warm up once eagerly on the current buffer contents, then capture."""
        from ..ops import library
        saved, saved_samp = self.ints.clone(), self.dev_samp.clone()
        stream = torch.cuda.Stream(device=self.runner.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            self._body()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        self.ints.copy_(saved)          # a self-feeding warm-up has moved tokens, positions and counters
        self.dev_samp.copy_(saved_samp)
        before = library.launch_count
        graph = torch.cuda.CUDAGraph()
        with no_collection(), torch.cuda.graph(graph):
            self._body()
        self.launches = library.launch_count - before
        self.graph = graph
        self.ints.copy_(saved)
        self.dev_samp.copy_(saved_samp)

    def load(self, tokens: Sequence[int], positions: Sequence[int], slots: Sequence[int],
             temperatures: Sequence[float], seeds: Sequence[int], counters: Sequence[int]) -> None:
        """Fill the fixed buffers for the next replay (two small host-to-device copies)."""
        bs = self.bs
        h = self.host_ints.numpy()
        h[0:bs], h[bs:2 * bs], h[2 * bs:3 * bs] = tokens, positions, slots
        s = self.host_samp.numpy()
        s[0:bs] = np.asarray(temperatures, dtype=np.float32).view(np.int32).astype(np.int64)
        s[bs:2 * bs] = [x & (2**63 - 1) for x in seeds]
        s[2 * bs:] = counters
        self.ints[:3 * bs].copy_(self.host_ints, non_blocking=True)
        self.dev_samp.copy_(self.host_samp, non_blocking=True)

    @property
    def h2d_bytes(self) -> int:
        return self.host_ints.numel() * 4 + self.host_samp.numel() * 8

    @property
    def d2h_bytes(self) -> int:
        return self.host_out.numel() * 4

    def replay(self) -> None:
        if self.graph is None:
            self.capture()
        self.graph.replay()

    def replay_burst(self, steps: int) -> List[List[int]]:
        """Queue ``steps`` replays of a self-feeding graph - every step's input is the step before's
        output, on the device - and return the sampled tokens of every step.  The host waits once."""
        if not self.self_feeding:
            raise RuntimeError("a run of replays needs a self-feeding graph")
        if self.host_burst is None or self.host_burst.shape[0] < steps:
            self.host_burst = torch.zeros((max(steps, 8), self.bs), dtype=torch.int32, pin_memory=True)
        for j in range(steps):
            self.replay()
            self.host_burst[j].copy_(self.sampled, non_blocking=True)   # in stream order, before the next replay overwrites it
        self.host_out[self.bs:].copy_(self.status, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        if int(self.host_out[self.bs]) != 0:
            raise RuntimeError(f"a kernel met a bad page id or position during the step (code {int(self.host_out[self.bs])})")
        return self.host_burst[:steps].tolist()

    def fetch(self) -> List[int]:
        """Sampled tokens of the last replay (one device-to-host copy, then a wait)."""
        self.host_out[:self.bs].copy_(self.sampled, non_blocking=True)
        self.host_out[self.bs:].copy_(self.status, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        out = self.host_out.tolist()
        if out[-1] != 0:
            raise RuntimeError(f"a kernel met a bad page id or position during the step (code {out[-1]})")
        return out[:-1]


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
