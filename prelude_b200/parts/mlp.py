"""Gated feed-forward: down(act(gate(x)) * up(x)), no biases
(crates/prelude-core/src/models/qwen3.rs:383-448).

Gate and up rows are stored one below the other so that one product feeds the
activation kernel; the reference merges them the same way where its kernels
take the merged layout (qwen3.rs:411-419).  The activation comes from the spec;
the reference parses ``hidden_act`` and then applies SiLU regardless.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import GatedMlpSpec
from ..ops import kernels as K
from ..ops.linear import gated_linear_silu, linear
from ..weights.loader import TensorReq
from .registry import RunContext, register_part

_ACTIVATIONS = {"silu": K.silu_mul}


@register_part("feed_forward", "gated_mlp")
class GatedMlp:
    def __init__(self, spec: GatedMlpSpec, prefix: str):
        if spec.activation not in _ACTIVATIONS:
            raise ValueError(f"gated feed-forward: no kernel for activation {spec.activation!r}; known: {sorted(_ACTIVATIONS)}")
        self.spec, self.prefix = spec, prefix
        self.w_gate_up = self.w_down = None

    def tensors(self) -> Dict[str, TensorReq]:
        s, p = self.spec, self.prefix
        return {
            f"{p}.gate_proj.weight": TensorReq((s.intermediate_size, s.hidden_size)),
            f"{p}.up_proj.weight": TensorReq((s.intermediate_size, s.hidden_size)),
            f"{p}.down_proj.weight": TensorReq((s.hidden_size, s.intermediate_size)),
        }

    def load(self, get, ctx: RunContext) -> None:
        p = self.prefix

        def mat(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=ctx.dtype)

        self.w_gate_up = torch.cat([mat("gate_proj.weight"), mat("up_proj.weight")], dim=0).contiguous()
        self.w_down = mat("down_proj.weight").contiguous()

    def activation_bytes_per_token(self, elem: int) -> int:
        """The merged gate/up projection, the activation, the output (as float32 partial sums at most)."""
        return 3 * self.spec.intermediate_size * elem + 4 * self.spec.hidden_size * 4

    def forward(self, x: torch.Tensor):
        """The feed-forward of x; what comes back goes to a fused residual add, which also takes
        the partial sums of a product whose K was cut into parts."""
        act = gated_linear_silu(x, self.w_gate_up) if self.spec.activation == "silu" else None
        if act is None:
            act = _ACTIVATIONS[self.spec.activation](linear(x, self.w_gate_up))
        return linear(act, self.w_down, partial_sums_ok=True)
