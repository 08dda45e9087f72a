"""y = x W^T (+ b) with W stored [out, in], in the run's type.

float32: the plain kernel on the float32 units, every output element summed
in ascending k by one thread; no reduced-precision matrix mode exists on this
path.

bfloat16, float32 accumulation:
  * the tcgen05 kernel of this library (TMA, tensor memory, a persistent grid that
    balances the stream of weight bytes over all blocks) where it is the fastest:
    with few rows (decode steps) the output head and the long-K projections;
    PRELUDE_TC_GEMM=all sends every product there;
  * cuBLAS through torch.mm elsewhere, which is where the reference's own
    dispatch ends as well (crates/prelude-cuda/src/ops/gemm.rs:35-137, 340-433);
  * a second kernel of this library that streams weights through registers
    (mma.sync) is kept for comparison and is off unless PRELUDE_SKINNY_MAX_ROWS is set.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from . import kernels as K
from . import library as _l
from .library import KernelLibraryError, check

# rows up to which the streaming kernel is used (0 turns it off)
SKINNY_MAX_ROWS = int(os.environ.get("PRELUDE_SKINNY_MAX_ROWS", "0"))
# which products go to the tcgen05 kernel: "auto" (where it is the fastest measured), "all", "none"
TC_POLICY = os.environ.get("PRELUDE_TC_GEMM", "auto")

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


_tc_scratch: Dict[torch.device, torch.Tensor] = {}
_tc_status: Dict[torch.device, torch.Tensor] = {}
TC_SWAP_MAX_ROWS = 64          # up to this many rows of x the weights are the 128-row operand


def tc_status(device: torch.device) -> torch.Tensor:
    """The status word of the tensor-core product on this device (non-zero: a block gave up waiting)."""
    st = _tc_status.get(device)
    if st is None:
        st = _tc_status[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return st


def _tc_scratch_for(device: torch.device, nbytes: int) -> torch.Tensor:
    buf = _tc_scratch.get(device)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _retired.append(buf)
        buf = torch.zeros(max(nbytes, 48 << 20), dtype=torch.uint8, device=device)
        _tc_scratch[device] = buf
    return buf


def tc_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    M, Kdim = x.shape
    if x.stride(1) != 1 or weight.stride(1) != 1 or x.data_ptr() % 16 or weight.data_ptr() % 16:
        return False
    lib = _l.library()
    if M <= TC_SWAP_MAX_ROWS:
        return bool(lib.pb_gemm_tc_supported(weight.shape[0], M, Kdim, weight.stride(0), x.stride(0)))
    return bool(lib.pb_gemm_tc_supported(M, weight.shape[0], Kdim, x.stride(0), weight.stride(0)))


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
            out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """x W^T on tcgen05: for few rows the weights are the 128-row operand and the
    result is stored transposed; for many rows x is."""
    M, Kdim = x.shape
    N = weight.shape[0]
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelLibraryError("gemm_tc: output must be bfloat16 or float32")
    lib = _l.library()
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    swap = M <= TC_SWAP_MAX_ROWS
    a, b = (weight, x) if swap else (x, weight)
    scratch = _tc_scratch_for(x.device, lib.pb_gemm_tc_scratch_bytes(a.shape[0], b.shape[0], Kdim))
    check(lib.pb_gemm_tc_bf16(a.data_ptr(), b.data_ptr(), None if bias is None else bias.data_ptr(), out.data_ptr(),
                              a.shape[0], b.shape[0], Kdim, a.stride(0), b.stride(0), out.stride(0), 1 if swap else 0,
                              1 if out_dtype == torch.float32 else 0, scratch.data_ptr(), tc_status(x.device).data_ptr(),
                              torch.cuda.current_stream().cuda_stream), "gemm_tc")
    return out


def skinny_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    M, Kdim = x.shape
    return (0 < M <= SKINNY_MAX_ROWS and x.stride(1) == 1 and weight.stride(1) == 1
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and bool(_l.library().pb_gemm_skinny_supported(M, weight.shape[0], Kdim, weight.stride(0), x.stride(0))))


def _tc_wanted(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> bool:
    """Measured on B200 against cuBLAS: with few rows the tcgen05 kernel wins where the
    weight stream is long (the output head; projections with K at least three times N)."""
    if TC_POLICY == "all":
        return True
    if TC_POLICY == "none" or x.shape[0] > TC_SWAP_MAX_ROWS:
        return False
    N, Kdim = weight.shape
    return out_dtype == torch.float32 or Kdim >= 3 * N


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
        if _tc_wanted(x, weight, out_dtype) and tc_takes(x, weight):
            return gemm_tc(x, weight, bias, out_dtype)
        if out_dtype == torch.bfloat16:
            y = torch.mm(x, weight.t())
        else:
            y = torch.mm(x, weight.t(), out_dtype=out_dtype)
        if bias is not None:
            y += bias.to(y.dtype)
        return y
    raise KernelLibraryError(f"linear: unsupported type {x.dtype}")
