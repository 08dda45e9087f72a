"""Paged attention over a step's batch: picks the kernel for the type and shape.

float32 always runs the plain warp-per-row kernel.  bfloat16 runs the fast
kernels where they take the shape and the plain kernel otherwise; which one ran
never changes what is computed, only how fast.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import kernels as K


def paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, batch, group: int,
                    scale: float, window: Optional[int]) -> torch.Tensor:
    """q [T, nH, D] of the batch's tokens against the pages of cache group ``group``."""
    table = batch.block_tables[group]
    return K.paged_attention_ref(q, k_pages, v_pages, batch.positions, batch.token_seq, table, scale, window,
                                 batch.status)
