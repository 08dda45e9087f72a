"""Architecture-neutral description of a decoder: what the model builder reads.

An architecture's typed configuration (for instance ``Qwen3Config``) turns its
config.json keys into one ``ModelSpec``.  Everything below the configuration —
parts, cache manager, step function, scheduler — sees only these records, so a
part never knows which model it is in, and another architecture is another
function from config.json to a ``ModelSpec``.

Every spec class carries a ``kind`` string; ``prelude_b200.parts.registry`` maps
(part family, kind) to the class that implements it.  A new kind of mixer,
feed-forward, norm or position encoding is a new spec dataclass plus a part
class registered under its kind.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """Root-mean-square norm over ``dim`` with a learned scale."""
    dim: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding, half-split pairing (j, j + rotary_dim/2)."""
    head_dim: int
    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rope_half"


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding inside the mixer."""
    kind: str = "none"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a paged key/value cache."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    softmax_scale: float
    position: object                      # RopeSpec | NoPositionSpec | ...
    qk_norm_eps: Optional[float] = None   # per-head RMSNorm of q and k when set
    bias: bool = False
    window: Optional[int] = None          # keys visible: pos_q - window < pos_k <= pos_q
    kind: str = "attention"


@dataclass(frozen=True)
class GatedMlpSpec:
    """down(act(gate(x)) * up(x)), no biases."""
    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: which mixer, which feed-forward, which norms, how arranged.

    ``prefix`` is the layer's tensor-name prefix; the four ``*_name`` fields are
    the sub-prefixes of its parts below it.
    """
    mixer: object
    feed_forward: object
    mixer_norm: NormSpec
    ff_norm: NormSpec
    prefix: str
    mixer_name: str = "self_attn"
    ff_name: str = "mlp"
    mixer_norm_name: str = "input_layernorm"
    ff_norm_name: str = "post_attention_layernorm"
    kind: str = "prenorm_residual"


@dataclass(frozen=True)
class TokenEmbeddingSpec:
    """A table of ``vocab_size`` rows of ``hidden_size``: the residual stream starts as the rows of the step's tokens."""
    vocab_size: int
    hidden_size: int
    name: str = "model.embed_tokens.weight"
    kind: str = "token_embedding"


@dataclass(frozen=True)
class LinearHeadSpec:
    """logits = x W^T over the vocabulary; ``tied`` takes the embedding's table for W."""
    vocab_size: int
    hidden_size: int
    tied: bool
    name: str = "lm_head.weight"
    kind: str = "linear_head"


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``block`` indexes ``ModelSpec.blocks`` (a block may be named more than once:
    its weights are shared).  ``cache`` names the cache this call uses; by
    default every call has a cache of its own, numbered by its place in the
    order.  A call with ``writes_cache=False`` reads the cache of the earlier
    call that owns it and stores nothing.
    """
    block: int
    cache: Optional[int] = None
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    blocks: Tuple[BlockSpec, ...]
    order: Tuple[LayerCall, ...]
    final_norm: NormSpec
    tie_embeddings: bool
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm"
    head_name: str = "lm_head.weight"
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)
    # The two ends of the model are parts as well.  Left at None they are the plain ones that the fields above
    # describe (a table gather; a linear head, tied or not); an architecture with a scaled embedding, learned
    # positions added to it, or a capped or scaled head names its own spec here.
    embedding: Optional[object] = None
    head: Optional[object] = None
    # name patterns (shell style) of tensors that checkpoints of the architecture carry and the model does not read
    ignored_tensors: Tuple[str, ...] = field(default_factory=tuple)

    def embedding_spec(self) -> object:
        return self.embedding or TokenEmbeddingSpec(self.vocab_size, self.hidden_size, self.embed_name)

    def head_spec(self) -> object:
        return self.head or LinearHeadSpec(self.vocab_size, self.hidden_size, self.tie_embeddings, self.head_name)

    def resolved_order(self) -> Tuple[LayerCall, ...]:
        """The run order with every ``cache`` filled in and checked."""
        out = []
        for n, call in enumerate(self.order):
            if not 0 <= call.block < len(self.blocks):
                raise ValueError(f"order[{n}] names block {call.block}, model has {len(self.blocks)}")
            cache = n if call.cache is None else call.cache
            if call.writes_cache:
                if cache != n:
                    raise ValueError(f"order[{n}] writes a cache, so it must own it (cache={cache})")
            else:
                if not (0 <= cache < n and out[cache].writes_cache):
                    raise ValueError(f"order[{n}] reads cache {cache}, which no earlier call owns")
            out.append(LayerCall(call.block, cache, call.writes_cache))
        return tuple(out)
