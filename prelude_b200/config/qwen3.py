"""Typed configuration of Qwen3 dense, read from its own config.json keys.

Fields and their required/optional status follow the reference's
``Qwen3Config`` (crates/prelude-core/src/models/config.rs:4-22): every size,
``rope_theta``, ``rms_norm_eps``, ``tie_word_embeddings`` and
``max_position_embeddings`` must be present.  Four switches that published
Qwen3 folders always carry with the same value may be absent and then take
that value (``attention_bias`` false, ``use_sliding_window`` false,
``max_window_layers`` 0, ``hidden_act`` "silu"); this is a deliberate
relaxation so that a minimal random-weights folder is valid.

What the reference's model code refuses is refused here with the same reason:
``use_sliding_window: true`` (crates/prelude-core/src/models/qwen3.rs:50-52).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, fields
from typing import Optional, Tuple

from .registry import ConfigError, extract_eos_token_ids, register_architecture
from .spec import (AttentionSpec, BlockSpec, GatedMlpSpec, LayerCall, ModelSpec, NormSpec, RopeSpec)

_REQUIRED_INT = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                 "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings")
_REQUIRED_FLOAT = ("rope_theta", "rms_norm_eps")


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


@register_architecture("Qwen3", aliases=("Qwen3", "Qwen3Model"), model_types=("qwen3",))
@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    attention_bias: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    hidden_act: str = "silu"
    eos_token_ids: Tuple[int, ...] = ()

    # -- parsing ------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        problems = []
        kw = {}
        for key in _REQUIRED_INT:
            v = raw.get(key)
            if v is None:
                problems.append(f"missing field `{key}`")
            elif not _is_int(v) or v <= 0:
                problems.append(f"`{key}` must be a positive integer, got {v!r}")
            else:
                kw[key] = v
        for key in _REQUIRED_FLOAT:
            v = raw.get(key)
            if v is None:
                problems.append(f"missing field `{key}`")
            elif isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
                problems.append(f"`{key}` must be a positive number, got {v!r}")
            else:
                kw[key] = float(v)
        v = raw.get("tie_word_embeddings")
        if v is None:
            problems.append("missing field `tie_word_embeddings`")
        elif not isinstance(v, bool):
            problems.append(f"`tie_word_embeddings` must be true or false, got {v!r}")
        else:
            kw["tie_word_embeddings"] = v
        for key in ("attention_bias", "use_sliding_window"):
            v = raw.get(key)
            if v is not None:
                if not isinstance(v, bool):
                    problems.append(f"`{key}` must be true or false, got {v!r}")
                else:
                    kw[key] = v
        v = raw.get("sliding_window")
        if v is not None:
            if not _is_int(v) or v <= 0:
                problems.append(f"`sliding_window` must be a positive integer or null, got {v!r}")
            else:
                kw["sliding_window"] = v
        v = raw.get("max_window_layers")
        if v is not None:
            if not _is_int(v) or v < 0:
                problems.append(f"`max_window_layers` must be a non-negative integer, got {v!r}")
            else:
                kw["max_window_layers"] = v
        v = raw.get("hidden_act")
        if v is not None:
            if not isinstance(v, str):
                problems.append(f"`hidden_act` must be a string, got {v!r}")
            else:
                kw["hidden_act"] = v
        try:
            kw["eos_token_ids"] = extract_eos_token_ids(raw)
        except ConfigError as e:
            problems.append(str(e))
        if problems:
            raise ConfigError("failed to parse Qwen3 config: " + "; ".join(problems))
        cfg = cls(**kw)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        problems = []
        if self.use_sliding_window:
            problems.append("sliding window is not supported yet (use_sliding_window=true)")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            problems.append(f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                            f"num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            problems.append(f"head_dim={self.head_dim} must be even for rotary pairs")
        if self.hidden_act != "silu":
            # The reference parses the key and then applies SiLU whatever it says
            # (crates/prelude-core/src/models/qwen3.rs:391-447); a different value
            # would silently compute something else, so it is refused instead.
            problems.append(f"hidden_act={self.hidden_act!r}: Qwen3's feed-forward is SiLU-gated")
        if problems:
            raise ConfigError("failed to parse Qwen3 config: " + "; ".join(problems))

    def to_dict(self) -> dict:
        out = {f.name: getattr(self, f.name) for f in fields(self) if f.name != "eos_token_ids"}
        out["architectures"] = ["Qwen3ForCausalLM"]
        out["model_type"] = "qwen3"
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return out

    # -- what the model builder reads --------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        """Layer by layer description (crates/prelude-core/src/models/qwen3.rs:45-131,
        391-409, 462-484, 545-571): every layer is GQA attention with per-head q/k
        RMSNorm and full rotary, then a SiLU-gated MLP, pre-norm residual."""
        rope = RopeSpec(head_dim=self.head_dim, rotary_dim=self.head_dim, theta=self.rope_theta,
                        max_positions=self.max_position_embeddings)
        attn = AttentionSpec(hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                             num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                             softmax_scale=1.0 / math.sqrt(self.head_dim), position=rope,
                             qk_norm_eps=self.rms_norm_eps, bias=self.attention_bias, window=None)
        mlp = GatedMlpSpec(hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
                           activation=self.hidden_act)
        norm = NormSpec(dim=self.hidden_size, eps=self.rms_norm_eps)
        blocks = tuple(BlockSpec(mixer=attn, feed_forward=mlp, mixer_norm=norm, ff_norm=norm,
                                 prefix=f"model.layers.{i}") for i in range(self.num_hidden_layers))
        order = tuple(LayerCall(block=i) for i in range(self.num_hidden_layers))
        return ModelSpec(architecture="Qwen3ForCausalLM", vocab_size=self.vocab_size,
                         hidden_size=self.hidden_size, max_positions=self.max_position_embeddings,
                         blocks=blocks, order=order, final_norm=norm,
                         tie_embeddings=self.tie_word_embeddings, eos_token_ids=self.eos_token_ids)
