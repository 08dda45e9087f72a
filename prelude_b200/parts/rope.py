"""Position encodings.  A position part owns its tables; the mixer hands them
to its kernel together with each token's absolute position.

Rotary tables follow the reference (crates/prelude-core/src/models/commons/attn_utils.rs:32-50):
inv_freq_j = float32(1 / theta^(2j / rotary_dim)) with the power in float64,
angle[p, j] = float32(p) * inv_freq_j, cos and sin taken in float32.  The
tables stay float32 in every mode (the reference rounds them to the model's
type); they are computed once on the host.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

from ..config.spec import NoPositionSpec, RopeSpec
from ..weights.loader import TensorReq
from .registry import RunContext, register_part

_TABLE_CACHE: Dict[tuple, Tuple[torch.Tensor, torch.Tensor]] = {}


@register_part("position", "rope_half")
class RotaryHalf:
    """Pairs element j with j + rotary_dim/2 (attn_utils.rs:52-59)."""

    def __init__(self, spec: RopeSpec, prefix: str = ""):
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ValueError(f"rotary_dim={spec.rotary_dim} must be even and in (0, head_dim={spec.head_dim}]")
        self.spec = spec
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorReq]:
        return {}

    def load(self, get, ctx: RunContext) -> None:
        s = self.spec
        key = (s.rotary_dim, s.theta, s.max_positions, str(ctx.device))
        if key not in _TABLE_CACHE:       # the layers of a model share one pair of tables
            inv = [1.0 / math.pow(float(s.theta), i / float(s.rotary_dim)) for i in range(0, s.rotary_dim, 2)]
            inv_freq = torch.tensor(inv, dtype=torch.float64).to(torch.float32)
            pos = torch.arange(s.max_positions, dtype=torch.float32).reshape(-1, 1)
            ang = pos * inv_freq.reshape(1, -1)
            _TABLE_CACHE[key] = (ang.cos().contiguous().to(ctx.device), ang.sin().contiguous().to(ctx.device))
        self.cos, self.sin = _TABLE_CACHE[key]

    @property
    def rotary_dim(self) -> int:
        return self.spec.rotary_dim


@register_part("position", "none")
class NoPosition:
    def __init__(self, spec: NoPositionSpec, prefix: str = ""):
        self.spec = spec
        self.cos = self.sin = None
        self.rotary_dim = 0

    def tensors(self) -> Dict[str, TensorReq]:
        return {}

    def load(self, get, ctx: RunContext) -> None:
        pass
