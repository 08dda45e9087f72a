"""The two ends of a decoder: token embedding and output head.

``TokenEmbedding`` gathers the rows of the step's tokens into the float32
residual stream (crates/prelude-core/src/models/commons/embedding.rs:29-35,
qwen3.rs:555-558, 602).  ``LinearHead`` multiplies the wanted rows, after the
final norm, with the vocabulary matrix; tied, it takes the embedding's table
itself, the same memory (qwen3.rs:637-660).  Both are parts like any other: an
architecture whose embedding is scaled, or whose logits are capped, registers
its own kind and names its spec in ``ModelSpec.embedding`` / ``ModelSpec.head``.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.spec import LinearHeadSpec, TokenEmbeddingSpec
from ..ops import kernels as K
from ..ops.linear import linear
from ..weights.loader import TensorReq
from .registry import RunContext, register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding:
    def __init__(self, spec: TokenEmbeddingSpec, prefix: str = ""):
        self.spec = spec
        self.table: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorReq]:
        return {self.spec.name: TensorReq((self.spec.vocab_size, self.spec.hidden_size))}

    def load(self, get, ctx: RunContext) -> None:
        self.table = get(self.spec.name).to(device=ctx.device, dtype=ctx.dtype).contiguous()

    def forward(self, batch) -> torch.Tensor:
        return K.embed_gather(batch.token_ids, self.table)


@register_part("head", "linear_head")
class LinearHead:
    def __init__(self, spec: LinearHeadSpec, prefix: str = ""):
        self.spec = spec
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Tuple[Dict[str, TensorReq], Dict[str, TensorReq]]:
        """(required, optional): a tied model may still carry a copy of the head; it is not read."""
        req = {self.spec.name: TensorReq((self.spec.vocab_size, self.spec.hidden_size))}
        return ({}, req) if self.spec.tied else (req, {})

    def load(self, get, ctx: RunContext, embedding) -> None:
        if self.spec.tied:
            table = getattr(embedding, "table", None)
            if table is None or tuple(table.shape) != (self.spec.vocab_size, self.spec.hidden_size):
                raise ValueError("a tied head needs an embedding part with a [vocab, hidden] table")
            self.weight = table                          # the same memory
        else:
            self.weight = get(self.spec.name).to(device=ctx.device, dtype=ctx.dtype).contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, None, out_dtype=torch.float32)
