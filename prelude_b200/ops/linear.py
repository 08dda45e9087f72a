"""y = x W^T (+ b) with W stored [out, in], in the run's type.

float32: the plain kernel on the float32 units, every output element summed
in ascending k by one thread; no reduced-precision matrix mode exists on this
path.

bfloat16, float32 accumulation:
  * up to 16 rows (decode steps): the weight-streaming kernel of this library
    (bulk copies into a shared-memory ring that start before the previous kernel
    has finished, mma.sync, every block owning whole output features);
  * the merged gate/up projection of a prompt step (from ``PAIR_MIN_ROWS`` rows): the paired-block tcgen05
    kernel of this library with silu(gate) * up in its epilogue (measured on B200 at 2,048 x 19,456 x 2,560:
    135 us against 159 us for cuBLAS followed by the activation kernel); the merged q/k/v projection of a long
    prompt step (from ``PAIR_QKV_MIN_ROWS`` rows) there too, with the per-head norm, the rotation and the cache
    write in its epilogue (``qkv_heads``);
  * cuBLAS through torch.mm for the other products above 16 rows, which is where the reference's own
    dispatch ends as well (crates/prelude-cuda/src/ops/gemm.rs:35-137, 340-433); PRELUDE_PREFILL_GEMM=pair
    sends them to the paired-block kernel too (on a par at 2,048 rows and more where the tiles fill the
    multiprocessors' waves, slower where they do not), =cublas none.
"""
from __future__ import annotations

import contextlib
import os
from typing import Dict, Optional

import torch

from . import kernels as K
from . import library as _l
from .library import KernelLibraryError, check

# rows up to which the streaming kernel is used (0 turns it off; it takes 16 at most)
STREAM_MAX_ROWS = int(os.environ.get("PRELUDE_STREAM_MAX_ROWS", "16"))
# which products of prompt steps run on the paired-block tcgen05 kernel: "auto" the gated one, "pair" all, "cublas" none
PREFILL_GEMM = os.environ.get("PRELUDE_PREFILL_GEMM", "auto")
if PREFILL_GEMM not in ("auto", "pair", "cublas"):
    raise KernelLibraryError(f"PRELUDE_PREFILL_GEMM={PREFILL_GEMM!r} is not auto, pair or cublas")
# rows from which they do (below, a 256-row tile is mostly empty or the tiles are too few for the device)
PAIR_MIN_ROWS = int(os.environ.get("PRELUDE_PAIR_MIN_ROWS", "768"))
# rows from which the merged q/k/v projection runs there with norm, rotation and cache write in its epilogue
PAIR_QKV_MIN_ROWS = int(os.environ.get("PRELUDE_PAIR_QKV_MIN_ROWS", "1536"))


def stream_takes(x: torch.Tensor, weight: torch.Tensor, splits: int = 1) -> bool:
    """Whether the streaming kernel takes x [M, K] against weight [N, K], K cut into ``splits`` parts."""
    M, Kdim = x.shape
    if splits > 1 and Kdim % (16 * splits):
        return False
    return (0 < M <= min(STREAM_MAX_ROWS, 16) and x.stride(1) == 1 and weight.stride(1) == 1
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and bool(_l.library().pb_gemm_stream_supported(M, weight.shape[0], Kdim // splits, weight.stride(0), x.stride(0))))


def gemm_stream(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                out_dtype: torch.dtype = torch.bfloat16, splits: int = 1, gated: bool = False) -> torch.Tensor:
    """The weight-streaming product for up to 16 rows of x; raises when the shape is not taken.
    With ``splits`` > 1, K is cut into that many parts and the result is the float32 partial
    sums [splits, M, N], for a reader that adds them up (``PartialSums``).  With ``gated``,
    weight is [2 N, K] (N gate rows, then N up rows) and the result is silu(gate) * up, [M, N]."""
    M, Kdim = x.shape
    N = weight.shape[0] // 2 if gated else weight.shape[0]
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelLibraryError("gemm_stream: output must be bfloat16 or float32")
    if x.stride(1) != 1 or weight.stride(1) != 1:
        raise KernelLibraryError("gemm_stream: rows must be dense")
    if gated and weight.shape[0] % 2:
        raise KernelLibraryError("gemm_stream: a gated weight has as many up rows as gate rows")
    if splits > 1:
        out = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
    else:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    check(_l.library().pb_gemm_stream_bf16(
        x.data_ptr(), weight.data_ptr(), None if bias is None else bias.data_ptr(), out.data_ptr(), M, N, Kdim,
        x.stride(0), weight.stride(0), N, 1 if out.dtype == torch.float32 else 0, splits, M * N, 1 if gated else 0,
        tc_status(x.device).data_ptr(), _l.current_stream_ptr(x.device)), "gemm_stream")
    return out


def gated_linear_silu(x: torch.Tensor, weight_gate_up: torch.Tensor) -> Optional[torch.Tensor]:
    """silu(x Wg^T) * (x Wu^T) for the merged [gate; up] weight in one kernel: the streaming kernel where it
    takes the shape (a decode step), the paired-block kernel for the many rows of a prompt step; None
    otherwise - the caller then multiplies and activates in two steps."""
    if x.dtype == torch.bfloat16 and weight_gate_up.dtype == torch.bfloat16:
        if stream_takes(x, weight_gate_up):
            return gemm_stream(x, weight_gate_up, gated=True)
        if PREFILL_GEMM != "cublas" and x.shape[0] >= PAIR_MIN_ROWS and pair_takes(x, weight_gate_up, gated=True):
            return gemm_pair(x, weight_gate_up, gated=True)
    return None


def pair_takes(x: torch.Tensor, weight: torch.Tensor, gated: bool = False) -> bool:
    """Whether the paired-block tcgen05 kernel takes x [M, K] against weight [N, K]."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.stride(1) == 1 and weight.stride(1) == 1
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and bool(_l.library().pb_gemm_pair_supported(x.shape[0], weight.shape[0], x.shape[1], x.stride(0),
                                                         weight.stride(0), 1 if gated else 0)))


def gemm_pair(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, gated: bool = False,
              out: Optional[torch.Tensor] = None, max_pairs: int = 0) -> torch.Tensor:
    """The product on paired blocks of the fifth-generation tensor cores (prompt steps); bfloat16 out.
    With ``gated``, weight is [2 N, K] (N gate rows, then N up rows) and the result is silu(gate) * up, [M, N].
    ``max_pairs`` (tests): fewer pairs of blocks than the device has."""
    M, Kdim = x.shape
    N = weight.shape[0] // 2 if gated else weight.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    elif out.shape != (M, N) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise KernelLibraryError("gemm_pair: out must be bfloat16 [M, N] with dense rows")
    check(_l.library().pb_gemm_pair_bf16(
        x.data_ptr(), weight.data_ptr(), None if bias is None else bias.data_ptr(), out.data_ptr(), M, weight.shape[0],
        Kdim, x.stride(0), weight.stride(0), out.stride(0), 1 if gated else 0, 1, max_pairs,
        tc_status(x.device).data_ptr(), _l.current_stream_ptr(x.device)), "gemm_pair")
    return out


def qkv_heads(x: torch.Tensor, w_qkv: torch.Tensor, bias: Optional[torch.Tensor], n_heads: int, n_kv_heads: int, head_dim: int,
              q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
              cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int, interleaved: bool,
              positions: torch.Tensor, token_seq: Optional[torch.Tensor], block_table: Optional[torch.Tensor],
              k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], write_kv: bool,
              status: Optional[torch.Tensor], out: torch.Tensor, force: Optional[bool] = None) -> torch.Tensor:
    """The merged q/k/v projection of x, per-head norm of queries and keys, rotation, queries to ``out``
    [T, n_heads, head_dim] and keys and values into their pages: one paired-block product with all of it in the
    epilogue for the many rows of a prompt step where the layer's shape allows (``force``: tests say which way),
    else the product followed by ``kernels.qknorm_rope_kvwrite``."""
    rows = (n_heads + (2 * n_kv_heads if write_kv else 0)) * head_dim
    w = w_qkv if w_qkv.shape[0] == rows else w_qkv[:rows]
    fused = (PREFILL_GEMM != "cublas" and x.shape[0] >= PAIR_QKV_MIN_ROWS) if force is None else force
    if (fused and bias is None and cos is not None and not interleaved and x.dtype == torch.bfloat16 and pair_takes(x, w)
            and bool(_l.library().pb_gemm_pair_heads_supported(x.shape[0], x.shape[1], x.stride(0), w.stride(0), n_heads,
                                                              n_kv_heads if write_kv else 0, head_dim, rotary_dim))):
        T = x.shape[0]
        if tuple(out.shape) != (T, n_heads, head_dim) or out.dtype != torch.bfloat16 or not out.is_contiguous():
            raise KernelLibraryError(f"qkv_heads: out is {tuple(out.shape)} {out.dtype}, q is {(T, n_heads, head_dim)} bfloat16")
        for t_, n_ in ((cos, "cos"), (sin, "sin"), (q_weight, "q_weight"), (k_weight, "k_weight")):
            if t_ is not None and (t_.dtype != torch.float32 or not t_.is_contiguous()):
                raise KernelLibraryError(f"qkv_heads: {n_} must be dense float32")
        if cos.shape[1] * 2 != rotary_dim or positions.dtype != torch.int32:
            raise KernelLibraryError("qkv_heads: table width does not match rotary_dim, or positions are not int32")
        page_size = num_pages = stride = 0
        if write_kv:
            if (k_pages.dtype != torch.bfloat16 or k_pages.shape != v_pages.shape or not k_pages.is_contiguous() or not v_pages.is_contiguous()
                    or (k_pages.shape[1], k_pages.shape[3]) != (n_kv_heads, head_dim) or block_table.dtype != torch.int32
                    or token_seq.dtype != torch.int32 or not block_table.is_contiguous()):
                raise KernelLibraryError(f"qkv_heads: pages {tuple(k_pages.shape)} or tables do not fit {n_kv_heads} heads of {head_dim}")
            num_pages, page_size, stride = k_pages.shape[0], k_pages.shape[2], block_table.shape[1]
        st = status if status is not None else tc_status(x.device)
        check(_l.library().pb_gemm_pair_heads_bf16(
            x.data_ptr(), w.data_ptr(), T, x.shape[1], x.stride(0), w.stride(0), out.data_ptr(),
            k_pages.data_ptr() if write_kv else None, v_pages.data_ptr() if write_kv else None,
            None if q_weight is None else q_weight.data_ptr(), None if k_weight is None else k_weight.data_ptr(), float(eps),
            cos.data_ptr(), sin.data_ptr(), cos.shape[0], positions.data_ptr(), token_seq.data_ptr() if write_kv else None,
            block_table.data_ptr() if write_kv else None, stride, page_size, num_pages, n_heads, n_kv_heads if write_kv else 0,
            head_dim, 1 if (write_kv and K.kv_swizzled(x.dtype, head_dim)) else 0, 0, st.data_ptr(), _l.current_stream_ptr(x.device)),
            "gemm_pair (q/k/v)")
        return out
    qkv = linear(x, w, None if bias is None else bias[:rows])
    return K.qknorm_rope_kvwrite(qkv, n_heads, n_kv_heads, head_dim, q_weight, k_weight, eps, cos, sin, rotary_dim, positions,
                                 token_seq, block_table, k_pages, v_pages, write_kv, status, out=out, interleaved=interleaved)


_tc_status: Dict[torch.device, torch.Tensor] = {}
_step_status: Optional[torch.Tensor] = None


@contextlib.contextmanager
def step_status(status: Optional[torch.Tensor]):
    """While this is open, the products raise ``status`` (the status word of the step being run, which the engine
    reads after every step) instead of the device's own word: a product that gave up a wait then fails the step
    like any other kernel's complaint, instead of passing unseen."""
    global _step_status
    before, _step_status = _step_status, status
    try:
        yield
    finally:
        _step_status = before


def tc_status(device: torch.device) -> torch.Tensor:
    """The status word that this library's products raise (non-zero: a block gave up waiting): the running step's
    while a model runs one, else one word per device for products called on their own."""
    if _step_status is not None:
        return _step_status
    st = _tc_status.get(device)
    if st is None:
        st = _tc_status[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return st


def stream_splits(M: int, N: int, Kdim: int) -> int:
    """Into how many parts the streaming kernel cuts K when its reader takes partial sums: 4 where
    K is long and the output narrow (measured on B200 at 8 rows, 2,560 x 9,728: 10.9 us against
    19.5 uncut; 2,560 x 4,096 and 6,144 x 2,560 gain nothing)."""
    return 4 if (Kdim >= 8192 and Kdim % 64 == 0 and N <= Kdim) else 1


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, partial_sums_ok: bool = False):
    """x [M, K], weight [N, K] (both of the run's type), bias float32 [N] or None.
    With ``partial_sums_ok`` the result may be ``PartialSums`` (float32 parts whose sum is
    the product): say so only when the reader is a fused residual add."""
    if x.dtype != weight.dtype:
        raise KernelLibraryError(f"linear: input is {x.dtype}, weight is {weight.dtype}")
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32:
        if out_dtype != torch.float32:
            raise KernelLibraryError("linear: the 32-bit path has 32-bit outputs")
        return K.gemm_ref(x, weight, bias, torch.float32)
    if x.dtype == torch.bfloat16:
        if x.shape[0] == 0:
            return torch.empty((0, weight.shape[0]), dtype=out_dtype, device=x.device)
        splits = stream_splits(x.shape[0], weight.shape[0], x.shape[1]) if partial_sums_ok else 1
        if splits > 1 and stream_takes(x, weight, splits):      # a row of x too long for shared memory may still fit in parts
            return K.PartialSums(gemm_stream(x, weight, bias, out_dtype, splits=splits))
        if stream_takes(x, weight):
            return gemm_stream(x, weight, bias, out_dtype)
        if PREFILL_GEMM == "pair" and out_dtype == torch.bfloat16 and x.shape[0] >= PAIR_MIN_ROWS and pair_takes(x, weight):
            return gemm_pair(x, weight, bias)
        if out_dtype == torch.bfloat16:
            y = torch.mm(x, weight.t())
        else:
            y = torch.mm(x, weight.t(), out_dtype=out_dtype)
        if bias is not None:
            y += bias.to(y.dtype)
        return y
    raise KernelLibraryError(f"linear: unsupported type {x.dtype}")
