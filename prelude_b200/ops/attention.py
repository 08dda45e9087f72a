"""Paged attention over a step's batch: picks the kernel for the type and shape.

float32 always runs the plain warp-per-row kernel.  bfloat16 runs the
tensor-core kernels where they take the shape (head sizes in multiples of 16
up to 256; at most 16 query heads per key/value head for decode steps, 64 for
prompt portions) and the plain kernel otherwise.  Which one ran changes the
rounding, never what is computed.
"""
from __future__ import annotations

import os
from typing import Optional

import numpy as np
import torch

from . import kernels as K
from . import library as _l
from .library import check

# Which kernel prompt portions run on: "auto" gives the tcgen05 kernel the portions that fill its blocks well
# (where it takes the shape) and the mma.sync kernel the rest, "tc" gives the tcgen05 kernel everything it
# takes, "mma" nothing.
PREFILL_KERNEL = os.environ.get("PRELUDE_PREFILL_ATTN", "auto")
TC_MIN_FILL = float(os.environ.get("PRELUDE_PREFILL_TC_MIN_FILL", "0.5"))
# Whether the single tokens of a mixed step run on the decode kernel (PRELUDE_DECODE_IN_MIXED=0: on the prompt kernels).
DECODE_IN_MIXED = os.environ.get("PRELUDE_DECODE_IN_MIXED", "1") != "0"

SM_COUNT = 148          # refreshed from the device at first use
_sm_count_known = False


def _sm_count(device) -> int:
    global SM_COUNT, _sm_count_known
    if not _sm_count_known:
        SM_COUNT = torch.cuda.get_device_properties(device).multi_processor_count
        _sm_count_known = True
    return SM_COUNT


_counters = {}


def _decode_counters(device) -> torch.Tensor:
    """Arrival counters of the split decode kernel: zero before the first call,
    left at zero by every call, so one buffer serves all calls on a stream."""
    buf = _counters.get(device)
    if buf is None:
        buf = _counters[device] = torch.zeros(1 << 16, dtype=torch.int32, device=device)
    return buf


def decode_splits(n_tokens: int, n_kv_heads: int, head_dim: int, max_context: int, device, page_size: int = 16,
                  swizzled: bool = True):
    """(parts, cluster): over how many blocks a decode step spreads the keys of one (token, key/value head), and
    whether those blocks add their parts up inside a thread-block cluster (through each other's shared memory)
    or through scratch memory.  The library's plan: what fills the device, what the device holds as clusters at
    one time, and what adding the parts up costs either way (``pb_attention_decode_plan``)."""
    plan = int(_l.library().pb_attention_decode_plan(n_tokens, n_kv_heads, head_dim, page_size, 1 if swizzled else 0,
                                                     max(1, int(max_context))))
    return plan & 255, bool(plan & 256)


def _prefill_plan(batch, tpt: int, min_len: int = 0, max_len: Optional[int] = None):
    """Tiles of ``tpt`` tokens of the requests whose portion has min_len <= tokens (< max_len), as device
    arrays (made once per step and choice)."""
    key = ("attn_tiles", tpt, min_len, max_len)
    plan = batch.extras.get(key)
    if plan is None:
        seqs, toks = [np.zeros(0, dtype=np.int32)], [np.zeros(0, dtype=np.int32)]
        for r, n in enumerate(batch.q_lens.tolist()):
            if n < min_len or (max_len is not None and n >= max_len):
                continue
            starts = np.arange(0, n, tpt, dtype=np.int32)
            seqs.append(np.full(starts.shape, r, dtype=np.int32))
            toks.append(starts)
        seqs, toks = np.concatenate(seqs), np.concatenate(toks)
        if seqs.shape[0] == 0:
            plan = (None, None, 0)
        else:
            # longest tiles first: a tile late in a portion walks more keys
            order = np.argsort(-(toks + batch.q_start_host[seqs]), kind="stable")
            host = torch.from_numpy(np.stack([seqs[order], toks[order]]))
            dev = host.to(batch.token_ids.device, non_blocking=True)
            plan = (dev[0], dev[1], int(seqs.shape[0]))
        batch.extras[key] = plan
    return plan


def _single_token_runs(batch):
    """(first token, tokens, longest context) of every run of consecutive requests that bring one token each."""
    runs = batch.extras.get("single_token_runs")
    if runs is None:
        runs = []
        single = batch.q_lens == 1
        r, R = 0, int(single.shape[0])
        while r < R:
            if not single[r]:
                r += 1
                continue
            e = r
            while e < R and single[e]:
                e += 1
            runs.append((int(batch.q_lens[:r].sum()), e - r, int(batch.kv_len_host[r:e].max())))
            r = e
        batch.extras["single_token_runs"] = runs
    return runs


def tensor_core_shape_ok(n_heads: int, n_kv_heads: int, head_dim: int, decode: bool, page_size: int = 16) -> bool:
    group = n_heads // n_kv_heads
    if not (head_dim % 16 == 0 and 16 <= head_dim <= 256):
        return False
    return group <= (16 if decode else 64)


def paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, batch, group: int,
                    scale: float, window: Optional[int], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, nH, D] of the batch's tokens against the pages of cache group ``group``; the result goes to ``out``
    when given.  While a step is being captured piece by piece (``batch.extras["recorder"]``), attention is what
    the pieces are cut at: its grids depend on how the step's tokens are spread over requests, so it is launched
    at every step anew, between the replays of the pieces."""
    recorder = batch.extras.get("recorder")
    if recorder is not None and recorder.capturing:
        if out is None:
            out = torch.empty_like(q)
        recorder.run_between_pieces(lambda: paged_attention(q, k_pages, v_pages, batch, group, scale, window, out))
        return out
    table = batch.block_tables[group]
    T, nH, D = q.shape
    num_pages, nKV, page_size, _ = k_pages.shape
    if out is None:
        out = torch.empty_like(q)
    if q.dtype != torch.bfloat16 or not tensor_core_shape_ok(nH, nKV, D, batch.decode_only, page_size):
        n = batch.n_real                                   # the rows after them are padding of a captured step
        out[:n] = K.paged_attention_ref(q[:n], k_pages, v_pages, batch.positions[:n], batch.table_row_of_token[:n], table, scale,
                                        window, batch.status)
        return out
    lib = _l.library()
    stream = _l.current_stream_ptr(q.device)
    win = int(window) if window else 0
    swizzled = 1 if K.kv_swizzled(q.dtype, D) else 0

    def decode(t0: int, n: int, max_ctx: int) -> None:
        """Tokens t0 .. t0 + n of the batch, one per request, on the kernel that spreads a token's keys over blocks."""
        row = nH * D * q.element_size()
        if window:
            max_ctx = min(max_ctx, window + 64)
        plan = decode_splits(n, nKV, D, max_ctx, q.device, page_size, bool(swizzled))
        splits, cluster = plan if isinstance(plan, tuple) else (int(plan), True)
        if n * nKV > (1 << 16):
            splits = 1
        # the partial results of the splits: one buffer per step and size, shared by the layers (a layer's attention
        # has finished long before the next layer's starts)
        key = ("attn_decode_scratch", n, nH, D, splits)
        scratch = batch.extras.get(key)
        if scratch is None:
            floats = lib.pb_attention_decode_scratch_floats(n, nH, D, splits)
            scratch = torch.empty(max(floats, 1), dtype=torch.float32, device=q.device)
            batch.extras[key] = scratch
        check(lib.pb_attention_decode_bf16(
            q.data_ptr() + t0 * row, k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr() + t0 * row, table.data_ptr(),
            table.shape[1], batch.positions.data_ptr() + 4 * t0, batch.table_row_of_token.data_ptr() + 4 * t0, page_size, num_pages,
            n, nH, nKV, D, float(scale), win, swizzled, splits, 1 if cluster else 0, scratch.data_ptr() if splits > 1 else None,
            _decode_counters(q.device).data_ptr() if splits > 1 else None, batch.status.data_ptr(), stream), "attention_decode")

    if batch.decode_only:
        decode(0, T, batch.max_kv_len if batch.max_kv_len else table.shape[1] * page_size)
        return out
    # A mixed step: runs of requests with a single token each (decode steps beside prompt portions) go to the decode
    # kernel, as they would in a step of their own, where that kernel takes the shape.
    mma_min = 0
    if DECODE_IN_MIXED and tensor_core_shape_ok(nH, nKV, D, True, page_size):
        for t0, n, max_ctx in _single_token_runs(batch):
            decode(t0, n, max_ctx)
        mma_min = 2
    # The tcgen05 kernel works on 256 query rows at a time and pays for all of them: it takes the portions that
    # fill at least TC_MIN_FILL of a block's tokens, the mma.sync kernel (64 rows at a time) the shorter ones
    # and the single tokens of a mixed step.  Both write disjoint rows of `out`.
    tc_min = None
    if PREFILL_KERNEL != "mma" and lib.pb_attention_prefill_tc_supported(nH, nKV, D, page_size, swizzled):
        tc_tokens = lib.pb_attention_prefill_tc_tile_tokens(nH, nKV)
        tc_min = max(mma_min, 1 if PREFILL_KERNEL == "tc" else max(1, int(tc_tokens * TC_MIN_FILL)))
        tile_seq, tile_tok0, n_tiles = _prefill_plan(batch, tc_tokens, tc_min, None)
        if n_tiles:
            check(lib.pb_attention_prefill_tc_bf16(
                q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), table.data_ptr(), table.shape[1],
                batch.positions.data_ptr(), batch.table_row_of_token.data_ptr(), batch.cu_q.data_ptr(), batch.q_start.data_ptr(),
                tile_seq.data_ptr(), tile_tok0.data_ptr(), n_tiles, page_size, num_pages, T, nH, nKV, D, float(scale), win,
                swizzled, batch.status.data_ptr(), stream), "attention_prefill_tc")
    tile_seq, tile_tok0, n_tiles = _prefill_plan(batch, 64 // (nH // nKV), mma_min, tc_min)
    if n_tiles:
        check(lib.pb_attention_prefill_bf16(
            q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), table.data_ptr(), table.shape[1],
            batch.positions.data_ptr(), batch.table_row_of_token.data_ptr(), batch.cu_q.data_ptr(), batch.q_start.data_ptr(),
            tile_seq.data_ptr(), tile_tok0.data_ptr(), n_tiles, page_size, num_pages, T, nH, nKV, D, float(scale), win,
            swizzled, batch.status.data_ptr(), stream), "attention_prefill")
    return out
