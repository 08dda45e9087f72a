"""y = x W^T (+ b) with W stored [out, in], in the run's type.

float32: the plain kernel on the float32 units, every output element summed
in ascending k by one thread; no reduced-precision matrix mode exists on this
path.

bfloat16, float32 accumulation:
  * few rows (decode steps): the weight-streaming kernel of this library, which
    reads every weight byte once and balances the stream over all blocks;
  * many rows (prompt portions), outputs in float32 (logits) and shapes the
    streaming kernel does not take: cuBLAS through torch.mm, which is where the
    reference's own dispatch ends as well
    (crates/prelude-cuda/src/ops/gemm.rs:35-137, 340-433).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from . import kernels as K
from . import library as _l
from .library import KernelLibraryError, check

# rows up to which the streaming kernel is used (0 turns it off)
SKINNY_MAX_ROWS = int(os.environ.get("PRELUDE_SKINNY_MAX_ROWS", "16"))

_scratch: Dict[torch.device, torch.Tensor] = {}
_retired: List[torch.Tensor] = []          # outgrown buffers that captured graphs may still use


def _skinny_scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    """One zero-initialised scratch buffer per device, shared by all calls (they
    run one after the other on a stream and leave the counters at zero)."""
    buf = _scratch.get(device)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _retired.append(buf)
        buf = torch.zeros(max(nbytes, 4 << 20), dtype=torch.uint8, device=device)
        _scratch[device] = buf
    return buf


def gemm_skinny(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The weight-streaming product for up to 64 rows of x; raises when the shape is not taken."""
    M, Kdim = x.shape
    N = weight.shape[0]
    lib = _l.library()
    if x.stride(1) != 1 or weight.stride(1) != 1:
        raise KernelLibraryError("gemm_skinny: rows must be dense")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    scratch = _skinny_scratch(x.device, lib.pb_gemm_skinny_scratch_bytes(M, N, Kdim))
    check(lib.pb_gemm_skinny_bf16(x.data_ptr(), weight.data_ptr(), None if bias is None else bias.data_ptr(),
                                  out.data_ptr(), M, N, Kdim, x.stride(0), weight.stride(0), out.stride(0),
                                  scratch.data_ptr(), torch.cuda.current_stream().cuda_stream), "gemm_skinny")
    return out


def skinny_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    M, Kdim = x.shape
    return (0 < M <= SKINNY_MAX_ROWS and x.stride(1) == 1 and weight.stride(1) == 1
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and bool(_l.library().pb_gemm_skinny_supported(M, weight.shape[0], Kdim, weight.stride(0), x.stride(0))))


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """x [M, K], weight [N, K] (both of the run's type), bias float32 [N] or None."""
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
        if out_dtype == torch.bfloat16 and skinny_takes(x, weight):
            return gemm_skinny(x, weight, bias)
        if out_dtype == torch.bfloat16:
            y = torch.mm(x, weight.t())
        else:
            y = torch.mm(x, weight.t(), out_dtype=out_dtype)
        if bias is not None:
            y += bias.to(y.dtype)
        return y
    raise KernelLibraryError(f"linear: unsupported type {x.dtype}")
