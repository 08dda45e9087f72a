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

# Which kernel prompt portions run on: "auto" takes the tcgen05 kernel where it takes the shape and the step
# has at least TC_MIN_TOKENS tokens, "tc" takes it wherever it takes the shape, "mma" never.
PREFILL_KERNEL = os.environ.get("PRELUDE_PREFILL_ATTN", "auto")
TC_MIN_TOKENS = int(os.environ.get("PRELUDE_PREFILL_TC_MIN_TOKENS", "1"))

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


def decode_splits(n_tokens: int, n_kv_heads: int, head_dim: int, max_context: int, device) -> int:
    """Over how many blocks a decode step spreads the keys of one (token, key/value head):
    as many as the device holds at one time, never more than there are 64-key tiles."""
    resident = _sm_count(device) * _l.library().pb_attention_decode_blocks_per_sm(head_dim)
    blocks = max(1, n_tokens * n_kv_heads)
    tiles = max(1, -(-max_context // 64))
    return max(1, min(resident // blocks, tiles, 64))


def _prefill_plan(batch, tpt: int):
    """Tiles of ``tpt`` tokens per request, as device arrays (made once per step and tile size)."""
    key = ("attn_tiles", tpt)
    plan = batch.extras.get(key)
    if plan is None:
        seqs, toks = [], []
        for r, n in enumerate(batch.q_lens.tolist()):
            starts = np.arange(0, n, tpt, dtype=np.int32)
            seqs.append(np.full(starts.shape, r, dtype=np.int32))
            toks.append(starts)
        seqs, toks = np.concatenate(seqs), np.concatenate(toks)
        # longest tiles first: a tile late in a portion walks more keys
        order = np.argsort(-(toks + batch.q_start_host[seqs]), kind="stable")
        host = torch.from_numpy(np.stack([seqs[order], toks[order]]))
        dev = host.to(batch.token_ids.device, non_blocking=True)
        plan = (dev[0], dev[1], int(seqs.shape[0]))
        batch.extras[key] = plan
    return plan


def tensor_core_shape_ok(n_heads: int, n_kv_heads: int, head_dim: int, decode: bool, page_size: int = 16) -> bool:
    group = n_heads // n_kv_heads
    if not (head_dim % 16 == 0 and 16 <= head_dim <= 256):
        return False
    return group <= (16 if decode else 64)


def paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, batch, group: int,
                    scale: float, window: Optional[int]) -> torch.Tensor:
    """q [T, nH, D] of the batch's tokens against the pages of cache group ``group``."""
    table = batch.block_tables[group]
    T, nH, D = q.shape
    num_pages, nKV, page_size, _ = k_pages.shape
    if q.dtype != torch.bfloat16 or not tensor_core_shape_ok(nH, nKV, D, batch.decode_only, page_size):
        return K.paged_attention_ref(q, k_pages, v_pages, batch.positions, batch.token_seq, table, scale, window,
                                     batch.status)
    out = torch.empty_like(q)
    lib = _l.library()
    stream = torch.cuda.current_stream().cuda_stream
    win = int(window) if window else 0
    if batch.decode_only:
        max_ctx = batch.max_kv_len if batch.max_kv_len else table.shape[1] * page_size
        if window:
            max_ctx = min(max_ctx, window + 64)
        splits = decode_splits(T, nKV, D, max_ctx, q.device)
        if T * nKV > (1 << 16):
            splits = 1
        n = lib.pb_attention_decode_scratch_floats(T, nH, D, splits)
        scratch = torch.empty(n, dtype=torch.float32, device=q.device) if n else None
        counters = _decode_counters(q.device) if n else None
        check(lib.pb_attention_decode_bf16(
            q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), table.data_ptr(), table.shape[1],
            batch.positions.data_ptr(), batch.token_seq.data_ptr(), page_size, num_pages, T, nH, nKV, D, float(scale),
            win, 1 if K.kv_swizzled(q.dtype, D) else 0, splits, None if scratch is None else scratch.data_ptr(),
            None if counters is None else counters.data_ptr(), batch.status.data_ptr(), stream),
            "attention_decode")
        return out
    swizzled = 1 if K.kv_swizzled(q.dtype, D) else 0
    if PREFILL_KERNEL != "mma" and lib.pb_attention_prefill_tc_supported(nH, nKV, D, page_size, swizzled) \
            and (PREFILL_KERNEL == "tc" or T >= TC_MIN_TOKENS):
        tile_seq, tile_tok0, n_tiles = _prefill_plan(batch, lib.pb_attention_prefill_tc_tile_tokens(nH, nKV))
        check(lib.pb_attention_prefill_tc_bf16(
            q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), table.data_ptr(), table.shape[1],
            batch.positions.data_ptr(), batch.token_seq.data_ptr(), batch.cu_q.data_ptr(), batch.q_start.data_ptr(),
            tile_seq.data_ptr(), tile_tok0.data_ptr(), n_tiles, page_size, num_pages, T, nH, nKV, D, float(scale), win,
            swizzled, batch.status.data_ptr(), stream), "attention_prefill_tc")
        return out
    tile_seq, tile_tok0, n_tiles = _prefill_plan(batch, 64 // (nH // nKV))
    check(lib.pb_attention_prefill_bf16(
        q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), table.data_ptr(), table.shape[1],
        batch.positions.data_ptr(), batch.token_seq.data_ptr(), batch.cu_q.data_ptr(), batch.q_start.data_ptr(),
        tile_seq.data_ptr(), tile_tok0.data_ptr(), n_tiles, page_size, num_pages, T, nH, nKV, D, float(scale), win,
        1 if K.kv_swizzled(q.dtype, D) else 0, batch.status.data_ptr(), stream), "attention_prefill")
    return out
