"""From a model folder to a model on the device with its cache and runner.

The order is the reference's (crates/prelude-core/src/engine/loading.rs:34-75,
165-264): read config.json, resolve the architecture through the registry,
open the safetensors files, build the model from its parts, size the cache.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from ..cache.manager import CacheManager
from ..config.registry import load_model_config
from ..config.spec import ModelSpec
from ..parts.model import DecoderModel
from ..parts.registry import RunContext
from ..weights.loader import WeightStore
from .runner import ModelRunner

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "f32": torch.float32,
           "fp32": torch.float32}


def parse_dtype(dtype: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype in (torch.bfloat16, torch.float32):
            return dtype
        raise ValueError(f"dtype must be bfloat16 or float32, not {dtype}")
    try:
        return _DTYPES[dtype.lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}") from None


def load_model(model_dir: str, dtype: Union[str, torch.dtype] = "bfloat16",
               device: Union[str, torch.device] = "cuda:0", random_weights_seed: Optional[int] = None) -> DecoderModel:
    """config.json -> registry -> typed configuration -> model spec -> parts -> weights by name.  With
    ``random_weights_seed`` the folder needs its config.json only: the tensors the model asks for are drawn on the
    device (linear ~N(0, 0.02), norm scales 1 + U(-0.05, 0.05), each tensor seeded by (seed, name)) and go through
    the same loading by name."""
    config = load_model_config(model_dir)
    if random_weights_seed is not None:
        from ..weights.random_init import random_tensors
        run_dtype = parse_dtype(dtype)
        tensors = random_tensors(config, seed=int(random_weights_seed), std=0.02, norm_jitter=0.05,
                                 dtype=torch.bfloat16 if run_dtype == torch.bfloat16 else torch.float32, device=device)
        store = WeightStore.from_tensors(tensors)
    else:
        store = WeightStore.open(model_dir)
    return build_model(config.to_model_spec(), store, dtype, device)


def build_model(spec: ModelSpec, store: WeightStore, dtype: Union[str, torch.dtype] = "bfloat16",
                device: Union[str, torch.device] = "cuda:0") -> DecoderModel:
    ctx = RunContext(torch.device(device), parse_dtype(dtype))
    return DecoderModel(spec).load(store, ctx)


def make_runner(model: DecoderModel, page_size: int = 16, num_pages: Optional[int] = None,
                max_tokens: Optional[int] = None, max_slots: int = 256,
                max_request_tokens: Optional[int] = None) -> ModelRunner:
    """A cache of ``num_pages`` pages (or enough for ``max_tokens`` tokens) and the runner over it.  With
    ``max_request_tokens`` the block tables also live on the device (what captured steps read)."""
    if num_pages is None:
        if max_tokens is None:
            raise ValueError("give num_pages or max_tokens")
        num_pages = -(-max_tokens // page_size)
    cache = CacheManager(model.cache_needs(), page_size, num_pages, max_slots, model.ctx.device, model.ctx.dtype,
                         max_request_tokens=max_request_tokens)
    return ModelRunner(model, cache)
