"""y = x W^T (+ b) with W stored [out, in], in the run's type.

float32: the plain kernel on the float32 units, every output element summed
in ascending k by one thread; no reduced-precision matrix mode exists on this
path.  bfloat16: the tensor-core product, float32 accumulation; it is cuBLAS
through torch.mm, which is where the reference's own dispatch ends for shapes
its other libraries refuse (crates/prelude-cuda/src/ops/gemm.rs:35-137, 340-433).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import kernels as K
from .library import KernelLibraryError


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
        if out_dtype == torch.bfloat16:
            y = torch.mm(x, weight.t())
        else:
            y = torch.mm(x, weight.t(), out_dtype=out_dtype)
        if bias is not None:
            y += bias.to(y.dtype)
        return y
    raise KernelLibraryError(f"linear: unsupported type {x.dtype}")
