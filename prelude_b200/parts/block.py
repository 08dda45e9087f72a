"""Arrangement of a mixer and a feed-forward in one layer.

Pre-norm residual block with the add fused into the next norm, as the
reference's decoder layer (crates/prelude-core/src/models/qwen3.rs:486-502):

    res += delta ; x = norm1(res) ; a = mixer(x)
    res += a     ; x = norm2(res) ; return feed_forward(x)      (added by whoever comes next)

``res`` is the float32 residual stream and is updated in place.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import BlockSpec
from ..weights.loader import TensorReq
from .registry import RunContext, make_part, register_part


@register_part("block", "prenorm_residual")
class PreNormResidualBlock:
    def __init__(self, spec: BlockSpec, prefix: str = ""):
        self.spec = spec
        p = spec.prefix
        self.mixer_norm = make_part("norm", spec.mixer_norm, f"{p}.{spec.mixer_norm_name}")
        self.mixer = make_part("mixer", spec.mixer, f"{p}.{spec.mixer_name}")
        self.ff_norm = make_part("norm", spec.ff_norm, f"{p}.{spec.ff_norm_name}")
        self.feed_forward = make_part("feed_forward", spec.feed_forward, f"{p}.{spec.ff_name}")

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward)

    def tensors(self) -> Dict[str, TensorReq]:
        out: Dict[str, TensorReq] = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, get, ctx: RunContext) -> None:
        for part in self.parts():
            part.load(get, ctx)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, delta: Optional[torch.Tensor], res: torch.Tensor, batch, cache, write_cache: bool) -> torch.Tensor:
        x = self.mixer_norm.add_forward(delta, res)
        a = self.mixer.forward(x, batch, cache, write_cache)
        x = self.ff_norm.add_forward(a, res)
        return self.feed_forward.forward(x)
