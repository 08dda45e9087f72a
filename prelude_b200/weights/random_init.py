"""Random weights: write a model folder from a configuration and a seed.

The folder holds config.json and model.safetensors and is read back through
the ordinary by-name loader, so random models exercise the same path as real
ones.  (The reference can only make all-zero weights,
crates/prelude-core/src/engine/weight_loader.rs:317-333.)

The list of tensors comes from the model itself (``DecoderModel.tensors()``),
so this works for any registered architecture.  Each tensor is drawn from a
generator seeded by (seed, tensor name): the values of a tensor do not depend
on which other tensors the model has.  Matrices and biases are N(0, std);
norm scales are 1 + U(-jitter, jitter).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Union

import torch

from ..config.registry import load_model_config
from ..parts.model import DecoderModel
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str, device="cpu") -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(digest[:8], "little") & (2**63 - 1))
    return g


def random_tensors(config: Union[dict, object], seed: int = 0, std: float = 0.02, norm_jitter: float = 0.1,
                   dtype: torch.dtype = torch.float32, device="cpu") -> Dict[str, torch.Tensor]:
    """Tensors by name for the model that ``config`` (a config.json dict or a
    typed configuration) describes.  With a CUDA ``device`` the numbers are drawn
    on the GPU (another stream of numbers than on the CPU): for benchmarks at
    sizes where a folder on disk would be tens of gigabytes."""
    cfg = load_model_config(config) if isinstance(config, dict) else config
    required, _ = DecoderModel(cfg.to_model_spec()).tensors()
    out = {}
    for name, req in required.items():
        g = _generator(seed, name, device)
        if req.role == "norm":
            t = 1.0 + (torch.rand(req.shape, generator=g, dtype=torch.float32, device=device) * 2.0 - 1.0) * norm_jitter
        else:
            t = torch.randn(req.shape, generator=g, dtype=torch.float32, device=device) * std
        out[name] = t.to(dtype)
    return out


def write_random_model(model_dir: str, config: dict, seed: int = 0, std: float = 0.02, norm_jitter: float = 0.1,
                       dtype: torch.dtype = torch.float32) -> str:
    """Create ``model_dir`` with config.json and model.safetensors; returns the folder."""
    os.makedirs(model_dir, exist_ok=True)
    load_model_config(config)                 # refuse a bad configuration before writing anything
    tensors = random_tensors(config, seed, std, norm_jitter, dtype)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config, f, indent=1, sort_keys=True)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      {"format": "pt", "seed": seed, "std": std, "norm_jitter": norm_jitter})
    return model_dir
