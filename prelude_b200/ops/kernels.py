"""Thin tensor wrappers over the C launchers of the kernel library.

Each function checks what the C side cannot see (devices, types, contiguity),
allocates the output with torch, and launches on torch's current stream, so the
calls can be captured in a CUDA graph.  Nothing here computes: if the library
is missing the call raises.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import library as _l
from .library import KernelLibraryError, check

F32, BF16 = 0, 1


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelLibraryError(f"kernels take float32 or bfloat16, not {dtype}")


def _stream() -> int:
    return _l.current_stream_ptr()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def kv_swizzled(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether key/value pages of this type and head size store the 16-byte chunks
    of a token row permuted (chunk c of token r at position c ^ (r & 7)).  The rule
    is a function of the page tensor alone, so the kernel that writes a page and
    the kernels that read it always agree."""
    return dtype == torch.bfloat16 and head_dim % 64 == 0


def _need(t: torch.Tensor, name: str, dtype=None, contiguous=True) -> None:
    if not t.is_cuda:
        raise KernelLibraryError(f"{name} must live on a CUDA device")
    if dtype is not None and t.dtype != dtype:
        raise KernelLibraryError(f"{name} must be {dtype}, is {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelLibraryError(f"{name} must be contiguous")


def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """res[t, :] = table[ids[t], :] as float32 (the residual stream)."""
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    T, (V, H) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    check(_l.library().pb_embed_gather(ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype), out.data_ptr(),
                                       T, H, V, _stream()), "embed_gather")
    return out


class PartialSums:
    """The output of a product whose K was cut into parts: ``parts`` is float32
    [n, rows, width] and the value is their sum.  The residual add takes it as
    it is and adds the parts up in float32; anyone else calls ``materialize``."""

    def __init__(self, parts: torch.Tensor):
        if parts.dim() != 3 or parts.dtype != torch.float32 or not parts.is_contiguous():
            raise KernelLibraryError("PartialSums: a dense float32 [parts, rows, width] tensor is needed")
        self.parts = parts

    @property
    def shape(self):
        return self.parts.shape[1:]

    def materialize(self, dtype: torch.dtype) -> torch.Tensor:
        return self.parts.sum(dim=0).to(dtype)


def _x_args(x, out_dtype: torch.dtype, what: str):
    """(pointer, parts, stride) of the addend of a fused add: a tensor of the run's type, partial sums, or nothing."""
    if x is None:
        return None, 0, 0
    if isinstance(x, PartialSums):
        _need(x.parts, what)
        return x.parts.data_ptr(), x.parts.shape[0], x.parts.stride(0)
    _need(x, what, out_dtype)
    return x.data_ptr(), 0, 0


def add_rmsnorm(x, res: torch.Tensor, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """res += x (when x is given: a tensor of ``out_dtype`` or ``PartialSums``); returns
    rmsnorm(res) * weight in ``out_dtype``."""
    _need(res, "res", torch.float32)
    _need(weight, "weight", torch.float32)
    rows, width = res.shape
    if x is not None and tuple(x.shape) != tuple(res.shape):
        raise KernelLibraryError(f"add_rmsnorm: x {tuple(x.shape)} against residual {tuple(res.shape)}")
    if weight.numel() != width:
        raise KernelLibraryError(f"add_rmsnorm: weight has {weight.numel()} elements, rows have {width}")
    ptr, parts, stride = _x_args(x, out_dtype, "x")
    if out is None:
        out = torch.empty((rows, width), dtype=out_dtype, device=res.device)
    check(_l.library().pb_add_rmsnorm(ptr, parts, stride, res.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                      dtype_code(out_dtype), rows, width, float(eps), _stream()), "add_rmsnorm")
    return out


def gather_add_rmsnorm(x, res: torch.Tensor, rows: torch.Tensor, weight: torch.Tensor,
                       eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """rmsnorm(res[rows] + x[rows]) * weight for the chosen rows; res is not changed."""
    _need(res, "res", torch.float32)
    _need(rows, "rows", torch.int32)
    _need(weight, "weight", torch.float32)
    if x is not None and tuple(x.shape) != tuple(res.shape):
        raise KernelLibraryError(f"gather_add_rmsnorm: x {tuple(x.shape)} against residual {tuple(res.shape)}")
    ptr, parts, stride = _x_args(x, out_dtype, "x")
    total, width = res.shape
    out = torch.empty((rows.numel(), width), dtype=out_dtype, device=res.device)
    check(_l.library().pb_gather_add_rmsnorm(ptr, parts, stride, res.data_ptr(), rows.data_ptr(), weight.data_ptr(),
                                             out.data_ptr(), dtype_code(out_dtype), rows.numel(), total, width,
                                             float(eps), _stream()), "gather_add_rmsnorm")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    _need(x, "x")
    _need(weight, "weight", torch.float32)
    width = x.shape[-1]
    rows = x.numel() // width
    if weight.numel() != width:
        raise KernelLibraryError(f"rmsnorm: weight has {weight.numel()} elements, rows have {width}")
    out = torch.empty_like(x)
    check(_l.library().pb_rmsnorm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), dtype_code(x.dtype), rows, width,
                                  float(eps), _stream()), "rmsnorm")
    return out


def qknorm_rope_kvwrite(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                        q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                        cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                        positions: torch.Tensor, token_seq: Optional[torch.Tensor],
                        block_table: Optional[torch.Tensor], k_pages: Optional[torch.Tensor],
                        v_pages: Optional[torch.Tensor], write_kv: bool,
                        status: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                        interleaved: bool = False) -> torch.Tensor:
    """q/k norm + rotation, q to a dense [T, nH, D] tensor (``out`` if given), k and v into their pages.
    Angle j turns the pair (j, j + rotary_dim / 2), or with ``interleaved`` the pair (2 j, 2 j + 1).

    ``qkv`` is the merged projection [T, (nH + 2 nKV) D] (or [T, nH D] when
    nothing is written).  Pages are [num_pages, nKV, page_size, D].
    """
    _need(qkv, "qkv", contiguous=False)
    if qkv.dim() != 2 or qkv.stride(1) != 1:
        raise KernelLibraryError("qknorm_rope_kvwrite: the projection must be [tokens, columns] with dense rows")
    T = qkv.shape[0]
    q_cols, kv_cols = n_heads * head_dim, n_kv_heads * head_dim
    want = q_cols + (2 * kv_cols if write_kv else 0)
    if qkv.shape[1] < want:
        raise KernelLibraryError(f"qknorm_rope_kvwrite: projection has {qkv.shape[1]} columns, needs {want}")
    esz = qkv.element_size()
    base = qkv.data_ptr()
    if out is None:
        q_out = torch.empty((T, n_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    else:
        _need(out, "out", qkv.dtype)
        if tuple(out.shape) != (T, n_heads, head_dim):
            raise KernelLibraryError(f"qknorm_rope_kvwrite: out is {tuple(out.shape)}, q is {(T, n_heads, head_dim)}")
        q_out = out
    max_pos, page_size, num_pages, stride = 0, 0, 0, 0
    if cos is not None:
        _need(cos, "cos", torch.float32)
        _need(sin, "sin", torch.float32)
        max_pos = cos.shape[0]
        if cos.shape[1] * 2 != rotary_dim:
            raise KernelLibraryError("qknorm_rope_kvwrite: table width does not match rotary_dim")
    if write_kv:
        _need(k_pages, "k_pages", qkv.dtype)
        _need(v_pages, "v_pages", qkv.dtype)
        _need(block_table, "block_table", torch.int32)
        _need(token_seq, "token_seq", torch.int32)
        num_pages, page_size = k_pages.shape[0], k_pages.shape[2]
        if (k_pages.shape[1], k_pages.shape[3]) != (n_kv_heads, head_dim) or k_pages.shape != v_pages.shape:
            raise KernelLibraryError(f"qknorm_rope_kvwrite: pages {tuple(k_pages.shape)} do not fit "
                                     f"{n_kv_heads} heads of {head_dim}")
        stride = block_table.shape[1]
    for w, n in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            _need(w, n, torch.float32)
            if w.numel() != head_dim:
                raise KernelLibraryError(f"qknorm_rope_kvwrite: {n} has {w.numel()} elements, heads have {head_dim}")
    _need(positions, "positions", torch.int32)
    check(_l.library().pb_qknorm_rope_kvwrite(
        base, base + q_cols * esz, base + (q_cols + kv_cols) * esz, qkv.stride(0), q_out.data_ptr(),
        _ptr(k_pages) if write_kv else None, _ptr(v_pages) if write_kv else None, dtype_code(qkv.dtype),
        _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin), rotary_dim if cos is not None else 0,
        1 if interleaved else 0, max_pos, positions.data_ptr(), _ptr(token_seq), _ptr(block_table), stride, page_size, num_pages, T, n_heads,
        n_kv_heads, head_dim, 1 if write_kv else 0, 1 if (write_kv and kv_swizzled(qkv.dtype, head_dim)) else 0,
        _ptr(status), _stream()), "qknorm_rope_kvwrite")
    return q_out


def paged_attention_ref(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, positions: torch.Tensor,
                        token_seq: torch.Tensor, block_table: torch.Tensor, scale: float,
                        window: Optional[int] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Plain paged attention, q [T, nH, D] -> [T, nH, D]."""
    _need(q, "q")
    _need(k_pages, "k_pages", q.dtype)
    _need(v_pages, "v_pages", q.dtype)
    _need(positions, "positions", torch.int32)
    _need(token_seq, "token_seq", torch.int32)
    _need(block_table, "block_table", torch.int32)
    T, nH, D = q.shape
    num_pages, nKV, page_size, Dk = k_pages.shape
    if Dk != D or v_pages.shape != k_pages.shape:
        raise KernelLibraryError("paged_attention_ref: q and pages disagree on the head size")
    out = torch.empty_like(q)
    check(_l.library().pb_paged_attention_ref(
        q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), dtype_code(q.dtype),
        positions.data_ptr(), token_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size,
        num_pages, T, nH, nKV, D, float(scale), int(window) if window else 0, 1 if kv_swizzled(q.dtype, D) else 0,
        _ptr(status), _stream()), "paged_attention_ref")
    return out


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[T, 2I] (gate columns first) -> silu(gate) * up, [T, I]."""
    _need(gate_up, "gate_up")
    T, two_i = gate_up.shape
    if two_i % 2:
        raise KernelLibraryError("silu_mul: merged projection must have an even number of columns")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    check(_l.library().pb_silu_mul(gate_up.data_ptr(), out.data_ptr(), dtype_code(gate_up.dtype), T, two_i // 2,
                                   _stream()), "silu_mul")
    return out


def gemm_ref(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
             out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M, K] times w [N, K] transposed (+ bias) on the float32 units."""
    _need(a, "a", contiguous=False)
    _need(w, "w", a.dtype, contiguous=False)
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1]:
        raise KernelLibraryError(f"gemm: a {tuple(a.shape)} against w {tuple(w.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1:
        raise KernelLibraryError("gemm: rows must be dense")
    M, K = a.shape
    N = w.shape[0]
    out_dtype = out_dtype or a.dtype
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != N:
            raise KernelLibraryError(f"gemm: bias has {bias.numel()} elements, output has {N} columns")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    check(_l.library().pb_gemm_ref(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), dtype_code(a.dtype),
                                   dtype_code(out_dtype), M, N, K, a.stride(0), w.stride(0), out.stride(0), _stream()),
          "gemm_ref")
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Row-wise argmax of float32 logits, ties to the smaller index; int32 [rows]."""
    _need(logits, "logits", torch.float32, contiguous=False)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelLibraryError("argmax: logits must be [rows, vocab] with dense rows")
    rows, vocab = logits.shape
    out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    lib = _l.library()
    scratch = torch.empty(max(1, lib.pb_sample_scratch_floats(rows, vocab)), dtype=torch.float32, device=logits.device)
    check(lib.pb_argmax(logits.data_ptr(), logits.stride(0), rows, vocab, out.data_ptr(), scratch.data_ptr(), _stream()),
          "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row: greedy where temperature < 1e-7, else a Philox draw from softmax(logits / T).
    The tokens go to ``out`` (int32 [rows]) when given."""
    _need(logits, "logits", torch.float32, contiguous=False)
    _need(temperature, "temperature", torch.float32)
    _need(seeds, "seeds", torch.int64)
    _need(counters, "counters", torch.int64)
    rows, vocab = logits.shape
    if not (temperature.numel() == seeds.numel() == counters.numel() == rows):
        raise KernelLibraryError("sample: one temperature, seed and counter per row")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    else:
        _need(out, "out", torch.int32)
        if out.numel() != rows:
            raise KernelLibraryError("sample: out holds one token per row")
    lib = _l.library()
    scratch = torch.empty(max(1, lib.pb_sample_scratch_floats(rows, vocab)), dtype=torch.float32, device=logits.device)
    check(lib.pb_sample(logits.data_ptr(), logits.stride(0), rows, vocab, temperature.data_ptr(), seeds.data_ptr(),
                        counters.data_ptr(), out.data_ptr(), scratch.data_ptr(), _stream()), "sample")
    return out


def softmax_temperature(logits: torch.Tensor, temperature: torch.Tensor) -> torch.Tensor:
    _need(logits, "logits", torch.float32, contiguous=False)
    _need(temperature, "temperature", torch.float32)
    rows, vocab = logits.shape
    out = torch.empty((rows, vocab), dtype=torch.float32, device=logits.device)
    check(_l.library().pb_softmax_temperature(logits.data_ptr(), logits.stride(0), rows, vocab,
                                              temperature.data_ptr(), out.data_ptr(), _stream()), "softmax_temperature")
    return out


def philox_uniform(seed: int, counter: int) -> float:
    """The uniform number in [0, 1) the sampler draws for (seed, counter); host-side, for tests."""
    return float(_l.library().pb_philox_uniform(seed & (2**64 - 1), counter & (2**64 - 1)))


def scatter_i32(dst: torch.Tensor, idx: torch.Tensor, val: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """dst.view(-1)[idx[i]] = val[i] on the device (block-table updates before a captured step)."""
    _need(dst, "dst", torch.int32)
    _need(idx, "idx", torch.int32)
    _need(val, "val", torch.int32)
    if idx.numel() != val.numel():
        raise KernelLibraryError("scatter_i32: one value per index")
    check(_l.library().pb_scatter_i32(dst.data_ptr(), dst.numel(), idx.data_ptr(), val.data_ptr(), idx.numel(),
                                      _ptr(status), _stream()), "scatter_i32")


def decode_advance(tokens: torch.Tensor, positions: torch.Tensor, kv_len: Optional[torch.Tensor],
                   counters: Optional[torch.Tensor], sampled: torch.Tensor, max_positions: int) -> None:
    """tokens = sampled; positions += 1; kv_len = positions + 1; counters += 1: a decode step that feeds itself."""
    _need(tokens, "tokens", torch.int32)
    _need(positions, "positions", torch.int32)
    _need(sampled, "sampled", torch.int32)
    if kv_len is not None:
        _need(kv_len, "kv_len", torch.int32)
    if counters is not None:
        _need(counters, "counters", torch.int64)
    check(_l.library().pb_decode_advance(tokens.data_ptr(), positions.data_ptr(), _ptr(kv_len), _ptr(counters),
                                         sampled.data_ptr(), tokens.numel(), int(max_positions), _stream()), "decode_advance")
