"""Steps with prompt tokens, captured piece by piece.

A step that brings prompt portions is several hundred launches; launched one
by one from Python they cost about 160 microseconds of host time a layer, more
than the kernels of a few hundred tokens take.  Everything in such a step has
the shape of its token count alone - except attention, whose grids follow how
the tokens are spread over requests, and the output head, which runs at the
wanted rows.  So the layers are captured once per token count as a chain of
CUDA graphs cut at the attention calls: a step replays piece, launches that
layer's attention, replays the next piece, ... and runs the head as usual.
(The reference captures decode steps only, crates/prelude-cuda/src/cuda_graph.rs:45-339;
cutting a step's graph at attention is what lets prompt steps be replayed too.)

Token counts are rounded up to a bucket; the rows after the real tokens are
padding: their token id and position are 0 and their request is -1, which the
kernel that writes the cache takes as "nothing to write".  Rows never mix, so
what the padding rows compute is never read.

What changes between steps lives at fixed addresses: token ids, positions, each
token's row of the device-resident block table (its request's state slot),
cumulative lengths, start positions.  One host-to-device copy fills them.
All pieces of all buckets allocate from one memory pool; after the capture only
the tensors that the launches between the pieces read and write are kept, so
the buckets share their memory.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from .batch import StepBatch, StepItem, pack_items
from .capture import no_collection


def bucket_of(n_tokens: int) -> int:
    """The token count a step of ``n_tokens`` is captured at."""
    step = 32 if n_tokens <= 256 else 64 if n_tokens <= 1024 else 128 if n_tokens <= 4096 else 256
    return -(-n_tokens // step) * step


class _Recorder:
    """Cuts the capture of a step into pieces at the calls that must run eagerly."""

    def __init__(self, pool, stream: torch.cuda.Stream):
        self.pool, self.stream = pool, stream
        self.pieces: List[torch.cuda.CUDAGraph] = []
        self.between: List[Callable[[], None]] = []      # between[i] runs after pieces[i]
        self.capturing = False
        self._graph: Optional[torch.cuda.CUDAGraph] = None

    def begin_piece(self) -> None:
        self._graph = torch.cuda.CUDAGraph()
        self._graph.capture_begin(pool=self.pool)
        self.capturing = True

    def end_piece(self) -> None:
        self._graph.capture_end()
        self.capturing = False
        self.pieces.append(self._graph)
        self._graph.replay()                              # a capture runs nothing: what follows needs the piece's results
        self._graph = None

    def abandon(self) -> None:
        """A launch failed while a piece was being captured: close the capture and drop what was recorded."""
        if self.capturing and self._graph is not None:
            try:
                self._graph.capture_end()
            except Exception:
                pass
        self.capturing, self._graph = False, None
        self.pieces.clear()
        self.between.clear()

    def run_between_pieces(self, fn: Callable[[], None]) -> None:
        self.end_piece()
        fn()
        self.between.append(fn)
        self.begin_piece()


class StepGraph:
    """The captured layers of a step of ``bucket`` tokens."""

    def __init__(self, runner, bucket: int, pool, stream: torch.cuda.Stream):
        self.runner, self.bucket, self.stream = runner, bucket, stream
        cache = runner.cache
        dev = runner.device
        R = cache.max_slots
        self.max_requests = R
        # int32 block: tokens | positions | token rows | cu_q | q_start | kv_len | slots | logit rows | status | token requests
        sizes = [bucket, bucket, bucket, R + 1, R, R, R, bucket, 1, bucket]
        self.offsets = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        self.ints = torch.zeros(int(self.offsets[-1]), dtype=torch.int32, device=dev)
        self.host = torch.zeros(int(self.offsets[-1]), dtype=torch.int32, pin_memory=True)
        v = [self.ints[int(self.offsets[i]):int(self.offsets[i + 1])] for i in range(len(sizes))]
        self.batch = StepBatch(
            n_tokens=bucket, n_seqs=0, token_ids=v[0], positions=v[1], token_seq=v[9], cu_q=v[3], q_start=v[4],
            kv_len=v[5], state_slots=v[6], logit_rows=v[7][:0], block_tables=dict(cache.device_tables), status=v[8],
            token_table_row=v[2])
        self._logit_rows = v[7]
        self.recorder = _Recorder(pool, stream)
        self.delta = self.res = None
        self.captured = False
        self.failed = False                 # a capture that raised: the bucket's steps are launched from then on
        self.replays = 0

    # -- the step's inputs --------------------------------------------------------------
    def load(self, items: Sequence[StepItem], slots: Sequence[int], vocab_size: int, max_positions: int) -> None:
        b, o, h = self.batch, self.offsets, self.host.numpy()
        R = len(items)
        q_lens, q_start, kv_len, cu_q, tokens, positions, rows = pack_items(items, vocab_size, max_positions)
        T = int(cu_q[-1])
        slots = np.asarray(list(slots), dtype=np.int32)
        h[:] = 0
        h[o[0]:o[0] + T] = tokens
        h[o[1]:o[1] + T] = positions
        h[o[2]:o[3]] = -1                                  # padding rows belong to no request
        h[o[2]:o[2] + T] = np.repeat(slots, q_lens)        # a token's row of the device-resident block table
        h[o[3]:o[3] + R + 1] = cu_q
        h[o[4]:o[4] + R] = q_start
        h[o[5]:o[5] + R] = kv_len
        h[o[6]:o[6] + R] = slots
        h[o[7]:o[7] + len(rows)] = rows
        h[o[9]:o[10]] = -1
        h[o[9]:o[9] + T] = np.repeat(np.arange(R, dtype=np.int32), q_lens)   # a token's request, as in a launched step
        self.ints.copy_(self.host, non_blocking=True)
        keep = {k: val for k, val in b.extras.items() if k == "recorder" or (isinstance(k, tuple) and k and k[0] == "workspace")}
        b.extras.clear()
        b.extras.update(keep)                              # the plans of the step before do not fit this one
        b.n_seqs, b.real_tokens, b.h2d_bytes = R, T, self.host.numel() * 4
        b.logit_rows = self._logit_rows[:len(rows)]
        b.q_lens, b.q_start_host, b.kv_len_host, b.state_slots_host = q_lens, q_start, kv_len, slots
        b.max_q_len, b.max_kv_len, b.decode_only = int(q_lens.max()), int(kv_len.max()), False

    # -- capture and replay ---------------------------------------------------------------
    def run(self) -> torch.Tensor:
        """The layers on the loaded inputs, then the head: float32 logits at the wanted rows."""
        model, caches = self.runner.model, self.runner.caches
        current = torch.cuda.current_stream()
        self.stream.wait_stream(current)
        with torch.cuda.stream(self.stream):
            if not self.captured:
                rec = self.recorder
                self.batch.extras["recorder"] = rec
                try:
                    with no_collection():
                        rec.begin_piece()
                        self.delta, self.res = model.forward_hidden(self.batch, caches)
                        rec.end_piece()
                except BaseException:
                    rec.abandon()                          # never leave the stream capturing
                    self.failed = True
                    raise
                self.captured = True
            else:
                for i, piece in enumerate(self.recorder.pieces):
                    piece.replay()
                    if i < len(self.recorder.between):
                        self.recorder.between[i]()
                self.replays += 1
            logits = model.head_logits(self.delta, self.res, self.batch)
        current.wait_stream(self.stream)
        return logits


class StepGraphs:
    """Captured prompt steps by token bucket, made when first needed; the least recently used go first."""

    def __init__(self, runner, max_tokens: int, max_graphs: int = 48):
        self.runner, self.max_tokens, self.max_graphs = runner, max_tokens, max_graphs
        self.graphs: "OrderedDict[int, StepGraph]" = OrderedDict()
        self.pool = torch.cuda.graph_pool_handle()
        self.stream = torch.cuda.Stream(device=runner.device)
        # the library behind torch.mm makes its handle and workspace for a stream at the first product on it, which
        # a capture does not allow: have one here
        with torch.cuda.stream(self.stream):
            a = torch.zeros((64, 64), dtype=runner.model.ctx.dtype, device=runner.device)
            torch.mm(a, a)
        self.stream.synchronize()

    def usable(self, n_tokens: int, n_requests: int, longest: int) -> bool:
        cache = self.runner.cache
        g = self.graphs.get(bucket_of(n_tokens))
        return (bool(cache.device_tables) and bucket_of(n_tokens) <= self.max_tokens and n_requests <= cache.max_slots
                and longest <= cache.table_width * cache.page_size and not (g is not None and g.failed))

    def get(self, n_tokens: int) -> StepGraph:
        b = bucket_of(n_tokens)
        g = self.graphs.get(b)
        if g is None:
            while len(self.graphs) >= self.max_graphs:
                self.graphs.popitem(last=False)
            g = self.graphs[b] = StepGraph(self.runner, b, self.pool, self.stream)
        self.graphs.move_to_end(b)
        return g
