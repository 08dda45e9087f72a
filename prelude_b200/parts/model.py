"""The decoder: embedding, blocks run in the order the spec lists, final norm,
output head (crates/prelude-core/src/models/qwen3.rs:534-678).  All four are
parts chosen by the spec; this file only says in which order they run.

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
from ..ops.linear import step_status
from ..weights.loader import TensorReq, WeightStore
from . import attention as _attention  # noqa: F401  (registers the part)
from . import block as _block  # noqa: F401
from . import ends as _ends  # noqa: F401
from . import mlp as _mlp  # noqa: F401
from . import norm as _norm  # noqa: F401
from . import rope as _rope  # noqa: F401
from .registry import KvPagesNeed, RunContext, RuntimeCaps, StateNeed, capturable, make_part


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.order = spec.resolved_order()
        self.blocks = [make_part("block", b, b.prefix) for b in spec.blocks]
        self.final_norm = make_part("norm", spec.final_norm, spec.final_norm_name)
        self.embedding = make_part("embedding", spec.embedding_spec(), "")
        self.head = make_part("head", spec.head_spec(), "")
        self.ctx: Optional[RunContext] = None

    # -- weights ------------------------------------------------------------------
    def tensors(self) -> Tuple[Dict[str, TensorReq], Dict[str, TensorReq]]:
        """(required, optional) tensors by name."""
        req: Dict[str, TensorReq] = dict(self.embedding.tensors())
        for b in self.blocks:
            req.update(b.tensors())
        req.update(self.final_norm.tensors())
        head_req, opt = self.head.tensors()
        req.update(head_req)
        return req, dict(opt)

    def load(self, store: WeightStore, ctx: RunContext) -> "DecoderModel":
        req, opt = self.tensors()
        store.check(req, opt, self.spec.ignored_tensors)
        self.ctx = ctx
        self.embedding.load(store.get, ctx)
        for b in self.blocks:
            b.load(store.get, ctx)
        self.final_norm.load(store.get, ctx)
        self.head.load(store.get, ctx, self.embedding)
        return self

    def all_parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def runtime_caps(self) -> RuntimeCaps:
        """What the engine may do with this model, from what its parts say."""
        needs = self.cache_needs()
        pages = any(isinstance(n, KvPagesNeed) for n in needs)
        return RuntimeCaps(kv_cache=pages, paged_attention=pages, varlen=True,
                           state_slots=any(isinstance(n, StateNeed) for n in needs),
                           cuda_graph=all(capturable(p) for p in self.all_parts()))

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
        with step_status(batch.status):
            res = self.embedding.forward(batch)
            delta = None
            for call in self.order:
                delta = self.blocks[call.block].forward(delta, res, batch, caches[call.cache], call.writes_cache)
        return delta, res

    def head_logits(self, delta, res, batch) -> torch.Tensor:
        """Final norm and output head at the rows whose logits are wanted."""
        if batch.logit_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=res.device)
        x = self.final_norm.gather_add_forward(delta, res, batch.logit_rows)
        with step_status(batch.status):
            return self.head.forward(x)
