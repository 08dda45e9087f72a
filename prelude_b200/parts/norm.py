"""RMSNorm with a learned scale, alone or fused with the residual add.

y = x / sqrt(mean(x^2) + eps) * w in float32
(crates/prelude-core/src/ops/traits/norm.rs:5-12; fused add+norm protocol
crates/prelude-core/src/models/commons/linear.rs:435-501).  The scale is kept
in float32 whatever the run's type: a bfloat16 scale converts exactly, and one
stored in 32-bit keeps its bits.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import NormSpec
from ..ops import kernels as K
from ..weights.loader import TensorReq
from .registry import RunContext, register_part


@register_part("norm", "rmsnorm")
class RmsNorm:
    def __init__(self, spec: NormSpec, prefix: str):
        self.spec, self.prefix = spec, prefix
        self.weight: Optional[torch.Tensor] = None
        self.dtype = None

    def tensors(self) -> Dict[str, TensorReq]:
        return {f"{self.prefix}.weight": TensorReq((self.spec.dim,), "norm")}

    def load(self, get, ctx: RunContext) -> None:
        self.weight = get(f"{self.prefix}.weight").to(device=ctx.device, dtype=torch.float32).contiguous()
        self.dtype = ctx.dtype

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Norm of a tensor of the run's type over its last axis."""
        return K.rmsnorm(x, self.weight, self.spec.eps)

    def add_forward(self, x: Optional[torch.Tensor], res: torch.Tensor) -> torch.Tensor:
        """res += x in place (float32), then the norm of res in the run's type."""
        return K.add_rmsnorm(x, res, self.weight, self.spec.eps, self.dtype)

    def gather_add_forward(self, x: Optional[torch.Tensor], res: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """norm(res[rows] + x[rows]) for the chosen rows only; res is left alone."""
        return K.gather_add_rmsnorm(x, res, rows, self.weight, self.spec.eps, self.dtype)
