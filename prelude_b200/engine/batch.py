"""The batch of one step, as the model's parts see it.

``StepItem`` is the step function's input for one request: its next tokens,
the position of the first of them, and the places (indices into these tokens)
whose logits are wanted.  ``build_step_batch`` packs the items of a step into
flat device arrays with one host-to-device copy.  The reference builds the same
arrays in ``batch_mixed_paged`` (crates/prelude-core/src/engine/model_runner/paged_mixed.rs:32-117):
packed tokens, positions, cumulative query lengths, context lengths and padded
block tables; the slot of a token is not shipped but recomputed by the kernels
from (request, position) and the block table.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


class StepError(RuntimeError):
    """A kernel raised the step's status word: it met a bad page id or position, or gave up a bounded wait."""


_STATUS = {2: "a token's page id lies outside the pool (cache write)", 3: "a position lies outside the rotation tables",
           4: "a page id lies outside the pool (plain attention)", 5: "a block-table update points outside the table",
           6: "a page id lies outside the pool (attention)", 7: "an attention kernel gave up waiting for a copy",
           8: "the tensor-core product gave up waiting for a copy", 9: "a tensor-core kernel gave up waiting for its products",
           10: "a tensor-core kernel gave up waiting for its accumulator", 11: "a streaming product's loader gave up waiting for a free stage",
           12: "a streaming product gave up waiting for its input or weights"}


def status_message(code: int) -> str:
    return f"a kernel raised the step's status word: {_STATUS.get(code, 'unknown reason')} (code {code})"


def raise_on_status(code: int) -> None:
    if code != 0:
        raise StepError(status_message(code))


@dataclass
class StepItem:
    request_id: object
    tokens: Sequence[int]
    position_start: int
    want: Sequence[int] = ()            # indices into ``tokens``


@dataclass
class LayerCache:
    """What one entry of the run order reads and writes: pages of a cache
    group, or per-request state, or nothing."""
    kind: Optional[str] = None          # "kv" | "state" | None
    group: int = -1
    k_pages: Optional[torch.Tensor] = None     # [num_pages, n_kv_heads, page_size, head_dim]
    v_pages: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None       # [max_slots, *shape]


@dataclass
class StepBatch:
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor             # [T] int32
    positions: torch.Tensor             # [T] int32, absolute position of each token
    token_seq: torch.Tensor             # [T] int32, index of the token's request in this batch
    cu_q: torch.Tensor                  # [R + 1] int32
    q_start: torch.Tensor               # [R] int32, position of the request's first token in this step
    kv_len: torch.Tensor                # [R] int32, tokens in the cache after this step
    state_slots: torch.Tensor           # [R] int32
    logit_rows: torch.Tensor            # [W] int32, rows of the packed batch whose logits are wanted
    block_tables: Dict[int, torch.Tensor]   # cache group -> [R, max_blocks] int32 (-1 where no page)
    status: torch.Tensor                # [1] int32, raised by kernels that met a bad page or position, or gave up a wait
    # [T] int32, the row of ``block_tables`` that holds the pages of each token's request.  A launched step packs
    # one table row per request, so this is ``token_seq`` itself (None); a captured step reads the
    # device-resident tables, which have one row per state slot.  -1 marks a padding row of a captured step.
    token_table_row: Optional[torch.Tensor] = None
    # host copies, for planning and for mixers that loop on the host
    q_lens: np.ndarray = field(default_factory=lambda: np.zeros(0, np.int32))
    q_start_host: np.ndarray = field(default_factory=lambda: np.zeros(0, np.int32))
    kv_len_host: np.ndarray = field(default_factory=lambda: np.zeros(0, np.int32))
    state_slots_host: np.ndarray = field(default_factory=lambda: np.zeros(0, np.int32))
    max_q_len: int = 0
    max_kv_len: int = 0
    decode_only: bool = False
    extras: Dict[str, object] = field(default_factory=dict)    # per-kernel plans made once per step
    real_tokens: int = -1               # tokens that exist; a captured step is padded to n_tokens (-1: all exist)
    h2d_bytes: int = 0                  # bytes of the host-to-device copy that brought this step's inputs

    @property
    def table_row_of_token(self) -> torch.Tensor:
        """What the kernels that walk block tables take for every token (see ``token_table_row``)."""
        return self.token_seq if self.token_table_row is None else self.token_table_row

    @property
    def n_real(self) -> int:
        return self.n_tokens if self.real_tokens < 0 else self.real_tokens

    def workspace(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        """A tensor that lives as long as the step and is handed out again for the same name, shape and type:
        what one layer's mixer puts there is dead by the time the next layer's asks (the stream orders them),
        so the layers share it instead of allocating each their own."""
        key = ("workspace", name, tuple(shape), dtype)
        t = self.extras.get(key)
        if t is None:
            t = self.extras[key] = torch.empty(tuple(shape), dtype=dtype, device=self.token_ids.device)
        return t


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def pack_items(items: Sequence[StepItem], vocab_size: int, max_positions: int):
    """The host arrays of a step, checked: (q_lens [R], q_start [R], kv_len [R], cu_q [R + 1], tokens [T] int64,
    positions [T], logit_rows [W]), the requests' tokens packed one after the other."""
    R = len(items)
    if R == 0:
        raise ValueError("a step needs at least one request")
    q_lens = np.array([len(it.tokens) for it in items], dtype=np.int32)
    if (q_lens <= 0).any():
        raise ValueError("every request of a step brings at least one token")
    T = int(q_lens.sum())
    q_start = np.array([it.position_start for it in items], dtype=np.int32)
    kv_len = q_start + q_lens
    if (q_start < 0).any() or int(kv_len.max()) > max_positions:
        raise ValueError(f"positions must lie in [0, {max_positions}); a request would reach {int(kv_len.max())}")
    cu_q = np.zeros(R + 1, dtype=np.int32)
    np.cumsum(q_lens, out=cu_q[1:])
    tokens = np.concatenate([np.asarray(it.tokens, dtype=np.int64) for it in items])
    if tokens.min() < 0 or tokens.max() >= vocab_size:
        raise ValueError(f"token ids must lie in [0, {vocab_size})")
    positions = (np.arange(T, dtype=np.int32) - np.repeat(cu_q[:-1], q_lens)) + np.repeat(q_start, q_lens)
    rows = []
    for i, it in enumerate(items):
        for wi in it.want:
            if not 0 <= wi < q_lens[i]:
                raise ValueError(f"request {it.request_id!r}: wanted place {wi} outside its {q_lens[i]} tokens")
            rows.append(int(cu_q[i]) + int(wi))
    return q_lens, q_start, kv_len, cu_q, tokens, positions.astype(np.int32), np.asarray(rows, dtype=np.int32)


def build_step_batch(items: Sequence[StepItem], block_tables: Dict[int, List[List[int]]],
                     state_slots: Sequence[int], device: torch.device, vocab_size: int,
                     max_positions: int, min_table_width: int = 1) -> StepBatch:
    """Pack ``items``; ``block_tables[group][i]`` is the page list of item i in
    that cache group (-1 for a page that a window has passed)."""
    R = len(items)
    q_lens, q_start, kv_len, cu_q, tokens, positions, logit_rows = pack_items(items, vocab_size, max_positions)
    T = int(cu_q[-1])
    token_seq = np.repeat(np.arange(R, dtype=np.int32), q_lens)
    slots = np.asarray(list(state_slots), dtype=np.int32)
    if slots.shape[0] != R:
        raise ValueError("one state slot per request")

    tables_np = {}
    for g, tabs in block_tables.items():
        width = max(min_table_width, max(len(t) for t in tabs))
        arr = np.full((R, width), -1, dtype=np.int32)
        for i, t in enumerate(tabs):
            arr[i, :len(t)] = t
        tables_np[g] = arr

    # one pinned staging buffer, one copy
    parts = [tokens.astype(np.int32), positions.astype(np.int32), token_seq, cu_q, q_start, kv_len, slots, logit_rows]
    parts += [tables_np[g].reshape(-1) for g in sorted(tables_np)]
    offsets = np.cumsum([0] + [p.size for p in parts])
    flat = torch.empty(int(offsets[-1]) + 1, dtype=torch.int32, pin_memory=(device.type == "cuda"))
    flat_np = flat.numpy()
    for p, o in zip(parts, offsets[:-1]):
        flat_np[o:o + p.size] = p
    flat_np[-1] = 0                                   # the status word
    dev = flat.to(device, non_blocking=True)

    def cut(i):
        return dev[int(offsets[i]):int(offsets[i + 1])]

    tables_dev = {}
    for n, g in enumerate(sorted(tables_np)):
        tables_dev[g] = cut(8 + n).view(R, tables_np[g].shape[1])
    return StepBatch(
        n_tokens=T, n_seqs=R, token_ids=cut(0), positions=cut(1), token_seq=cut(2), cu_q=cut(3), q_start=cut(4),
        kv_len=cut(5), state_slots=cut(6), logit_rows=cut(7), block_tables=tables_dev, status=dev[-1:],
        q_lens=q_lens, q_start_host=q_start, kv_len_host=kv_len, state_slots_host=slots,
        max_q_len=int(q_lens.max()), max_kv_len=int(kv_len.max()), decode_only=bool((q_lens == 1).all()),
        h2d_bytes=flat.numel() * 4)
