"""Loads the sm_100a kernel library and declares the C signatures.

There is no fallback: if the library cannot be built or loaded, or the device
is not sm_100, every kernel call raises ``KernelLibraryError``.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_float, c_int, c_longlong, c_uint64, c_void_p
from typing import Optional

ABI_VERSION = 16


class KernelLibraryError(RuntimeError):
    """The CUDA kernel library is missing, stale, or refused a call."""


P = c_void_p
I = c_int
L = c_longlong
F = c_float

_SIGNATURES = {
    "pb_abi_version": ([], I),
    "pb_built_for_sm": ([], I),
    "pb_check_device": ([], I),
    "pb_embed_gather": ([P, P, I, P, I, I, I, P], I),
    "pb_add_rmsnorm": ([P, I, L, P, P, P, I, I, I, F, P], I),
    "pb_rmsnorm": ([P, P, P, I, I, I, F, P], I),
    "pb_gather_add_rmsnorm": ([P, I, L, P, P, P, P, I, I, I, I, F, P], I),
    "pb_qknorm_rope_kvwrite": ([P, P, P, L, P, P, P, I, P, P, F, P, P, I, I, I, P, P, P, I, I, I, I, I, I, I, I, I, P, P], I),
    "pb_rope_set_heads_min_tokens": ([I], I),
    "pb_paged_attention_ref": ([P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, P, P], I),
    "pb_silu_mul": ([P, P, I, I, I, P], I),
    "pb_gemm_ref": ([P, P, P, P, I, I, I, I, I, L, L, L, P], I),
    "pb_sample_scratch_floats": ([I, I], L),
    "pb_argmax": ([P, L, I, I, P, P, P], I),
    "pb_sample": ([P, L, I, I, P, P, P, P, P, P], I),
    "pb_softmax_temperature": ([P, L, I, I, P, P, P], I),
    "pb_philox_uniform": ([c_uint64, c_uint64], F),
    "pb_attention_prefill_bf16": ([P, P, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P, P], I),
    "pb_attention_prefill_tc_supported": ([I, I, I, I, I], I),
    "pb_attention_prefill_tc_tile_tokens": ([I, I], I),
    "pb_attention_prefill_tc_bf16": ([P, P, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P, P], I),
    "pb_attention_decode_scratch_floats": ([I, I, I, I], L),
    "pb_attention_decode_blocks_per_sm": ([I], I),
    "pb_attention_decode_bf16": ([P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, I, I, I, I, P, P, P, P], I),
    "pb_attention_decode_cluster_max": ([], I),
    "pb_attention_decode_plan": ([I, I, I, I, I, I], I),
    "pb_attention_decode_set_cluster": ([I], None),
    "pb_gemm_pair_supported": ([I, I, I, L, L, I], I),
    "pb_gemm_pair_bf16": ([P, P, P, P, I, I, I, L, L, L, I, I, I, P, P], I),
    "pb_gemm_pair_heads_supported": ([I, I, L, L, I, I, I, I], I),
    "pb_gemm_pair_heads_bf16": ([P, P, I, I, L, L, P, P, P, P, P, F, P, P, I, P, P, P, I, I, I, I, I, I, I, I, P, P], I),
    "pb_gemm_stream_supported": ([I, I, I, L, L], I),
    "pb_gemm_stream_bf16": ([P, P, P, P, I, I, I, L, L, L, I, I, L, I, P, P], I),
    "pb_scatter_i32": ([P, L, P, P, I, P, P], I),
    "pb_decode_advance": ([P, P, P, P, P, I, I, P], I),
}

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None
_lib_path: Optional[str] = None
_device_checked = False


def declare(lib: ctypes.CDLL, name: str, argtypes, restype) -> None:
    try:
        fn = getattr(lib, name)
    except AttributeError:
        raise KernelLibraryError(f"kernel library {_lib_path} has no symbol {name}: it is stale, rebuild it") from None
    fn.argtypes = argtypes
    fn.restype = restype


def register_signatures(table: dict) -> None:
    """Add C signatures (used by kernel files added after this one was written)."""
    _SIGNATURES.update(table)
    if _lib is not None:
        for name, (args, res) in table.items():
            declare(_lib, name, args, res)


def library() -> ctypes.CDLL:
    """The loaded library; builds it at the first call if need be."""
    global _lib, _lib_path
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from ..csrc import build as _build
        try:
            path = _build.build()
        except Exception as e:   # noqa: BLE001 - turned into the one error type callers expect
            raise KernelLibraryError(f"cannot build the CUDA kernel library: {e}") from e
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelLibraryError(f"cannot load {path}: {e}") from e
        _lib_path = path
        lib.pb_last_error.argtypes = []
        lib.pb_last_error.restype = c_char_p
        for name, (args, res) in _SIGNATURES.items():
            declare(lib, name, args, res)
        if lib.pb_abi_version() != ABI_VERSION:
            raise KernelLibraryError(f"{path} has interface version {lib.pb_abi_version()}, expected {ABI_VERSION}")
        _lib = lib
    return _lib


def library_path() -> Optional[str]:
    return _lib_path


def last_error() -> str:
    return (library().pb_last_error() or b"").decode(errors="replace")


launch_count = 0     # launcher calls so far in this process (a launcher issues one kernel)


def current_stream_ptr(device=None) -> int:
    """The raw handle of the current CUDA stream of ``device`` (the current device if None).  One call into torch's
    C module: the launch path asks for it several times per layer, and ``torch.cuda.current_stream()`` costs
    about 10 microseconds a call."""
    import torch
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    return torch._C._cuda_getCurrentRawStream(index)


def check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if code != 0:
        raise KernelLibraryError(f"{what}: {last_error()}")


def require_device() -> None:
    """Raise unless the current CUDA device can run the library."""
    global _device_checked
    if _device_checked:
        return
    import torch
    if not torch.cuda.is_available():
        raise KernelLibraryError("no CUDA device: this engine runs on sm_100a GPUs only and has no CPU path")
    check(library().pb_check_device(), "device check")
    _device_checked = True
