"""The decoder: embedding, blocks run in the order the spec lists, final norm,
output head (crates/prelude-core/src/models/qwen3.rs:534-678).

``DecoderModel(spec)`` is cheap; ``tensors()`` says what it needs;
``load(store, ctx)`` checks the store against that list in one go and moves the
tensors to the device; ``forward(batch, caches)`` runs one step and returns the
float32 logits of the rows the batch asks for.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config.spec import ModelSpec
from ..ops import kernels as K
from ..ops.linear import linear
from ..weights.loader import TensorReq, WeightStore
from . import attention as _attention  # noqa: F401  (registers the part)
from . import block as _block  # noqa: F401
from . import mlp as _mlp  # noqa: F401
from . import norm as _norm  # noqa: F401
from . import rope as _rope  # noqa: F401
from .registry import RunContext, make_part


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.order = spec.resolved_order()
        self.blocks = [make_part("block", b, b.prefix) for b in spec.blocks]
        self.final_norm = make_part("norm", spec.final_norm, spec.final_norm_name)
        self.embed: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.ctx: Optional[RunContext] = None

    # -- weights ------------------------------------------------------------------
    def tensors(self) -> Tuple[Dict[str, TensorReq], Dict[str, TensorReq]]:
        """(required, optional) tensors by name."""
        s = self.spec
        req: Dict[str, TensorReq] = {s.embed_name: TensorReq((s.vocab_size, s.hidden_size))}
        opt: Dict[str, TensorReq] = {}
        for b in self.blocks:
            req.update(b.tensors())
        req.update(self.final_norm.tensors())
        # a tied model may still carry a copy of the head; it is not read
        (opt if s.tie_embeddings else req)[s.head_name] = TensorReq((s.vocab_size, s.hidden_size))
        return req, opt

    def load(self, store: WeightStore, ctx: RunContext) -> "DecoderModel":
        req, opt = self.tensors()
        store.check(req, opt)
        self.ctx = ctx
        s = self.spec
        self.embed = store.get(s.embed_name).to(device=ctx.device, dtype=ctx.dtype).contiguous()
        for b in self.blocks:
            b.load(store.get, ctx)
        self.final_norm.load(store.get, ctx)
        if s.tie_embeddings:
            self.head = self.embed                      # the same memory (qwen3.rs:639-641)
        else:
            self.head = store.get(s.head_name).to(device=ctx.device, dtype=ctx.dtype).contiguous()
        return self

    # -- cache needs, one per entry of the run order ---------------------------------
    def cache_needs(self) -> List[object]:
        """For each entry of the order: what its own cache must hold, or None
        when it has none of its own (it reads an earlier entry's, or needs none)."""
        return [self.blocks[c.block].cache_need() if c.writes_cache else None for c in self.order]

    def weight_bytes(self) -> int:
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.is_cuda and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
                elif hasattr(v, "__dict__") and not isinstance(v, (type, torch.device)) and id(v) not in seen:
                    seen.add(id(v))
                    visit(v)
                elif isinstance(v, (list, tuple)):
                    for e in v:
                        if hasattr(e, "__dict__") and id(e) not in seen:
                            seen.add(id(e))
                            visit(e)
        visit(self)
        return total

    # -- one step -------------------------------------------------------------------
    def forward(self, batch, caches) -> torch.Tensor:
        """``caches[n]`` is the LayerCache that entry n of the order owns.
        Returns float32 logits [len(batch.logit_rows), vocab]."""
        delta, res = self.forward_hidden(batch, caches)
        return self.head_logits(delta, res, batch)

    def forward_hidden(self, batch, caches):
        """The layers: returns (delta, res), the last layer's output and the residual it has yet to be added to.
        Every launch in here has the shape of the step's token count alone, except what a mixer runs through
        ``batch.extras["recorder"]``; that is what lets a step be captured piece by piece."""
        res = K.embed_gather(batch.token_ids, self.embed)
        delta = None
        for call in self.order:
            delta = self.blocks[call.block].forward(delta, res, batch, caches[call.cache], call.writes_cache)
        return delta, res

    def head_logits(self, delta, res, batch) -> torch.Tensor:
        """Final norm and output head at the rows whose logits are wanted."""
        if batch.logit_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=res.device)
        x = self.final_norm.gather_add_forward(delta, res, batch.logit_rows)
        return linear(x, self.head, None, out_dtype=torch.float32)
