"""Weights by tensor name, with one error for everything that does not fit.

The model states which tensors it needs (name, shape, role); ``WeightStore.check``
compares that list with what the files hold and raises a single ``WeightError``
that lists missing tensors, unexpected tensors and wrong shapes together.  The
reference looks names up one by one through prefix paths and fails at the first
that is absent or misshapen (crates/prelude-core/src/engine/weight_loader.rs:188-285,
335-404); the names and the shape rule are the same, the report is whole.

Storage types: a tensor stored in bfloat16 is kept in bfloat16; one stored in
32-bit floating point stays 32-bit; float16 becomes bfloat16 and float64 becomes
float32; integer tensors of any width become int32.  What a part then does with
its tensors (for instance matrices in the run's type, norm scales in float32)
is the part's business.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

import torch

from .safetensors_io import SafetensorsFile, find_shards


class WeightError(ValueError):
    """The weight files do not fit the model.  ``missing``, ``unexpected`` and
    ``wrong_shape`` hold the details that the message lists."""

    def __init__(self, source: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]], wrong_type: List[Tuple[str, str]] = ()):
        self.missing, self.unexpected, self.wrong_shape, self.wrong_type = missing, unexpected, wrong_shape, list(wrong_type)
        lines = [f"weights in {source} do not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + ", ".join(
                f"{n} expected {list(e)} got {list(g)}" for n, e, g in wrong_shape))
        if self.wrong_type:
            lines.append(f"  wrong type ({len(self.wrong_type)}): " + ", ".join(f"{n} is {t}" for n, t in self.wrong_type))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorReq:
    """What a part needs: the shape, and a role that tells the random-weights
    writer how to fill it ("matrix", "norm", "bias")."""
    shape: Tuple[int, ...]
    role: str = "matrix"


def normalize_storage(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.float32, torch.bfloat16, torch.int32):
        return t
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool):
        return t.to(torch.int32)
    raise ValueError(f"unsupported tensor type {t.dtype}")


class WeightStore:
    """All tensors of a model folder (or of a dict), by name."""

    def __init__(self, source: str, files: Iterable[SafetensorsFile] = (), tensors: Optional[Mapping[str, torch.Tensor]] = None):
        self.source = source
        self._where: Dict[str, SafetensorsFile] = {}
        self._tensors: Dict[str, torch.Tensor] = dict(tensors or {})
        for f in files:
            for name in f.names():
                self._where.setdefault(name, f)

    @classmethod
    def open(cls, model_dir: str) -> "WeightStore":
        return cls(model_dir, files=[SafetensorsFile(p) for p in find_shards(model_dir)])

    @classmethod
    def from_tensors(cls, tensors: Mapping[str, torch.Tensor], source: str = "<memory>") -> "WeightStore":
        return cls(source, tensors=tensors)

    def names(self) -> List[str]:
        return sorted(set(self._where) | set(self._tensors))

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        if name in self._tensors:
            t = self._tensors[name]
            return t.dtype, tuple(t.shape)
        return self._where[name].info(name)

    def __contains__(self, name: str) -> bool:
        return name in self._tensors or name in self._where

    def get(self, name: str) -> torch.Tensor:
        """The tensor on the CPU in its storage type (see the module text)."""
        if name in self._tensors:
            return normalize_storage(self._tensors[name])
        if name not in self._where:
            raise WeightError(self.source, [name], [], [])
        return normalize_storage(self._where[name].tensor(name))

    def check(self, required: Mapping[str, TensorReq], optional: Mapping[str, TensorReq] = None,
              ignored: Iterable[str] = ()) -> None:
        """Raise one WeightError unless the store holds exactly the required
        tensors (plus any of the optional ones) with the stated shapes.  ``ignored``
        are name patterns (shell style: ``*.rotary_emb.inv_freq``) of tensors that a
        checkpoint of the architecture may carry and the model never reads; they are
        passed over instead of counting as unexpected."""
        import fnmatch
        optional = optional or {}
        patterns = list(ignored)
        have = set(self.names())
        missing = sorted(n for n in required if n not in have)
        unexpected = sorted(n for n in have if n not in required and n not in optional
                            and not any(fnmatch.fnmatchcase(n, pat) for pat in patterns))
        wrong, wrong_type = [], []
        for name, req in list(required.items()) + list(optional.items()):
            if name in have:
                dtype, shape = self.info(name)
                if tuple(shape) != tuple(req.shape):
                    wrong.append((name, tuple(req.shape), tuple(shape)))
                if not dtype.is_floating_point:
                    wrong_type.append((name, str(dtype)))
        if missing or unexpected or wrong or wrong_type:
            raise WeightError(self.source, missing, unexpected, wrong, wrong_type)
