"""Plain, slow, whole-sequence implementation of the Qwen3 dense decoder.

This file is the oracle of the test-suite.  It shares no code with the
``prelude_b200`` package: it takes a plain ``dict`` (the parsed config.json)
and a ``dict`` of tensors keyed by safetensors name, runs a whole sequence at
once with no cache, and returns the logits of every position.

It rests on the reference's formulas (Virtue-Research/prelude); every function
cites the file and lines it was written from (paths relative to the
reference's project root).  The reference's own model code is Rust on a forked
tensor crate and cannot be built or imported here, so there is no golden output
produced by it; ``tests/golden`` holds outputs of *this* file instead, to pin
it against accidental edits.

All arithmetic is done in ``dtype`` (float32 by default, float64 for tie
analysis).  Weights are converted to ``dtype`` on entry, so a bfloat16
checkpoint is evaluated exactly (bfloat16 -> float32 is lossless).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------
def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h[t, :] = E[ids[t], :].

    crates/prelude-core/src/models/commons/embedding.rs:29-35
    """
    return table[ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * w over the last axis.

    crates/prelude-core/src/ops/traits/norm.rs:5-12
    crates/prelude-cuda/src/kernels/kernels_src/normalization/rmsnorm.cu:33-51
    """
    var = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(var + eps) * weight


def rope_tables(head_dim: int, n_positions: int, theta: float, dtype=torch.float32):
    """cos/sin tables [n_positions, head_dim/2].

    inv_freq_j = (float32)(1 / theta^(2j/D)) with the power taken in float64,
    angle[p, j] = float32(p) * inv_freq_j, in float32.

    crates/prelude-core/src/models/commons/attn_utils.rs:32-50
    """
    inv = [1.0 / math.pow(float(theta), i / float(head_dim)) for i in range(0, head_dim, 2)]
    inv_freq = torch.tensor(inv, dtype=torch.float64).to(torch.float32)
    pos = torch.arange(n_positions, dtype=torch.float32).reshape(-1, 1)
    ang = pos * inv_freq.reshape(1, -1)          # float32 product, as the reference
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split rotation.  x: [L, heads, D]; cos, sin: [L, D/2].

    out[..., :D/2] = x1*cos - x2*sin ; out[..., D/2:] = x2*cos + x1*sin

    crates/prelude-core/src/models/commons/attn_utils.rs:52-59
    """
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: Optional[int] = None) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence.

    q: [L, nH, D]; k, v: [L, nKV, D].  Query head h reads kv head h // (nH/nKV).
    Key j is visible to query i iff j <= i (and i - j < window when a window is
    given).  scores = (q.k) * scale, masked = -inf, softmax over keys, times v.

    crates/prelude-core/src/models/qwen3.rs:335-365 (matmul_cross_attention)
    crates/prelude-core/src/ops/traits/attention.rs:30-81
    """
    L, nH, D = q.shape
    nKV = k.shape[1]
    group = nH // nKV
    kx = k.repeat_interleave(group, dim=1)       # [L, nH, D]
    vx = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kx) * scale
    i = torch.arange(L).reshape(L, 1)
    j = torch.arange(L).reshape(1, L)
    visible = j <= i
    if window is not None:
        visible = visible & ((i - j) < window)
    scores = scores.masked_fill(~visible[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, vx)


def attention_block(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict,
                    cos: torch.Tensor, sin: torch.Tensor,
                    kv_from: Optional[tuple] = None, window: Optional[int] = None):
    """q/k/v projections, per-head q/k RMSNorm, RoPE, attention, output projection.

    Returns (output [L, H], (k, v)) so that a later layer may read this layer's
    keys and values instead of making its own (``kv_from``).

    crates/prelude-core/src/models/qwen3.rs:161-231 (forward), 54-131 (shapes)
    """
    L = x.shape[0]
    nH, nKV, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]

    def lin(name, inp):
        y = inp @ w[f"{prefix}.{name}.weight"].T
        b = w.get(f"{prefix}.{name}.bias")
        return y if b is None else y + b

    q = lin("q_proj", x).reshape(L, nH, D)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], eps)
    q = apply_rope(q, cos, sin)
    if kv_from is None:
        k = lin("k_proj", x).reshape(L, nKV, D)
        v = lin("v_proj", x).reshape(L, nKV, D)
        k = rms_norm(k, w[f"{prefix}.k_norm.weight"], eps)
        k = apply_rope(k, cos, sin)
    else:
        k, v = kv_from
    scale = 1.0 / math.sqrt(D)                  # qwen3.rs:126
    o = causal_attention(q, k, v, scale, window)
    return lin("o_proj", o.reshape(L, nH * D)), (k, v)


def swiglu_mlp(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down( silu(gate(x)) * up(x) ), silu(g) = g / (1 + exp(-g)); no biases.

    crates/prelude-core/src/models/qwen3.rs:391-447
    crates/prelude-cuda/src/kernels/kernels_src/elementwise/silu_mul.cu:27-32
    """
    g = x @ w[f"{prefix}.gate_proj.weight"].T
    u = x @ w[f"{prefix}.up_proj.weight"].T
    m = (g / (1.0 + torch.exp(-g))) * u
    return m @ w[f"{prefix}.down_proj.weight"].T


def decoder_block(res: torch.Tensor, w, i: int, cfg: dict, cos, sin, kv_from=None, window=None):
    """Pre-norm residual block: res += attn(norm(res)); res += mlp(norm(res)).

    The reference carries (hidden, residual) pairs and fuses the add into the
    next norm; the value of the residual stream is the same.

    crates/prelude-core/src/models/qwen3.rs:486-502
    crates/prelude-core/src/models/commons/linear.rs:471-488
    """
    p = f"model.layers.{i}"
    eps = cfg["rms_norm_eps"]
    a, kv = attention_block(rms_norm(res, w[f"{p}.input_layernorm.weight"], eps), w,
                            f"{p}.self_attn", cfg, cos, sin, kv_from, window)
    res = res + a
    m = swiglu_mlp(rms_norm(res, w[f"{p}.post_attention_layernorm.weight"], eps), w, f"{p}.mlp")
    return res + m, kv


# ----------------------------------------------------------------------------
# whole model
# ----------------------------------------------------------------------------
def forward_logits(cfg: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int],
                   dtype=torch.float32, order: Optional[List[tuple]] = None,
                   windows: Optional[Dict[int, int]] = None, rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits [L, V] of every position of one whole sequence (or of the positions ``rows`` alone: the head of
    a large vocabulary is most of the work, and a test that looks at a few positions need not pay for all).

    ``order`` is an optional list of (layer index, index in ``order`` of the call
    whose keys/values are read, or None); the default runs layers 0..L-1 once,
    each with keys and values of its own.  ``windows`` maps a position in
    ``order`` to a sliding-window length.

    crates/prelude-core/src/models/qwen3.rs:601-623 (backbone), 637-673 (head)
    """
    w = weights if all(v.dtype == dtype for v in weights.values()) else {k: v.to(dtype) for k, v in weights.items()}
    ids_t = torch.as_tensor(list(ids), dtype=torch.long)
    L = ids_t.numel()
    cos, sin = rope_tables(cfg["head_dim"], L, cfg["rope_theta"], dtype)
    res = embedding(ids_t, w["model.embed_tokens.weight"])
    if order is None:
        order = [(i, None) for i in range(cfg["num_hidden_layers"])]
    kvs = []
    for n, (layer, src) in enumerate(order):
        kv_from = None if src is None else kvs[src]
        win = None if windows is None else windows.get(n)
        res, kv = decoder_block(res, w, layer, cfg, cos, sin, kv_from, win)
        kvs.append(kv)
    if rows is not None:
        res = res[torch.as_tensor(list(rows), dtype=torch.long)]
    x = rms_norm(res, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return x @ head.T


def greedy_generate(cfg: dict, weights, prompt: Sequence[int], n_new: int,
                    dtype=torch.float32) -> List[int]:
    """Greedy continuation by re-running the whole sequence for every token.

    Ties go to the smaller index, as the reference's argmax kernel does
    (crates/prelude-cuda/src/kernels/kernels_src/sample/fast_argmax_vocab.cu:15-16,43).
    """
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward_logits(cfg, weights, ids, dtype)[-1]
        tok = int(torch.argmax(logits))          # first maximal index
        out.append(tok)
        ids.append(tok)
    return out


def softmax_temperature(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """p = softmax(logits / T) in float32.

    crates/prelude-core/src/engine/sampling/logits_processor.rs:100-110
    """
    return torch.softmax(logits.to(torch.float32) / temperature, dim=-1)
