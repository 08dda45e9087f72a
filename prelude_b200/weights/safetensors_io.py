"""Reading and writing safetensors files, and finding a model folder's shards.

A safetensors file is an 8-byte little-endian header length, a JSON header
{name: {"dtype", "shape", "data_offsets": [begin, end]}} and the raw data.  The
reader maps the file and hands out torch views of it without copying.

Shard discovery follows the reference (crates/prelude-core/src/engine/weights.rs:57-144):
``model.safetensors.index.json`` names the shards (absolute paths and ``..``
are refused); else ``model.safetensors``; else every ``*.safetensors`` in name
order; none at all is an error.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, List, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# safetensors dtype name -> (numpy dtype used to view the bytes, torch dtype, bytes per element)
_DTYPES = {
    "F64": (np.float64, torch.float64, 8),
    "F32": (np.float32, torch.float32, 4),
    "F16": (np.float16, torch.float16, 2),
    "BF16": (np.uint16, torch.bfloat16, 2),
    "I64": (np.int64, torch.int64, 8),
    "I32": (np.int32, torch.int32, 4),
    "I16": (np.int16, torch.int16, 2),
    "I8": (np.int8, torch.int8, 1),
    "U8": (np.uint8, torch.uint8, 1),
    "BOOL": (np.uint8, torch.bool, 1),
}
_TORCH_TO_NAME = {torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
                  torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8",
                  torch.uint8: "U8", torch.bool: "BOOL"}


class SafetensorsFile:
    """One mapped file: ``names()``, ``info(name)`` and ``tensor(name)``."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {path}: {e}") from None
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + hlen
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, ent in header.items():
            try:
                dtype, shape, (b, e) = ent["dtype"], tuple(int(s) for s in ent["shape"]), ent["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for {name!r}") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype}")
            n = 1
            for s in shape:
                n *= s
            if e - b != n * _DTYPES[dtype][2] or b < 0 or self._data_start + e > size:
                raise SafetensorsError(f"{path}: tensor {name!r}: offsets [{b}, {e}) do not fit shape {shape} {dtype}")
            self._entries[name] = (dtype, shape, b, e)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self._entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dtype, shape, _, _ = self._entries[name]
        return _DTYPES[dtype][1], shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (read-only: copy before writing)."""
        dtype, shape, b, e = self._entries[name]
        np_dtype, t_dtype, _ = _DTYPES[dtype]
        if e == b:
            return torch.empty(shape, dtype=t_dtype)
        arr = np.frombuffer(self._map, dtype=np_dtype, count=(e - b) // np.dtype(np_dtype).itemsize,
                            offset=self._data_start + b)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # torch warns that the buffer is not writable
            t = torch.from_numpy(arr)
        if t_dtype == torch.bfloat16:
            t = t.view(torch.bfloat16)
        elif t_dtype == torch.bool:
            t = t.view(torch.bool)
        return t.reshape(shape)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write ``tensors`` (CPU, any supported dtype) in name order."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"cannot store {name!r} of dtype {t.dtype}")
        if t.dtype == torch.bfloat16:
            raw = t.view(torch.int16).numpy().tobytes()
        elif t.dtype == torch.bool:
            raw = t.view(torch.uint8).numpy().tobytes()
        else:
            raw = t.numpy().tobytes()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)      # keep the data 8-byte aligned
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)


def find_shards(model_dir: str) -> List[str]:
    """Paths of the safetensors files of a model folder, in load order."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        try:
            with open(index, "r", encoding="utf-8") as f:
                weight_map = json.load(f)["weight_map"]
        except (OSError, ValueError, KeyError, TypeError) as e:
            raise SafetensorsError(f"{index}: cannot read the shard index: {e}") from None
        shards: List[str] = []
        for shard in weight_map.values():
            if not isinstance(shard, str) or os.path.isabs(shard) or ".." in shard.replace("\\", "/").split("/"):
                raise SafetensorsError(f"{index}: shard name {shard!r} leaves the model folder")
            if shard not in shards:
                shards.append(shard)
        paths = [os.path.join(model_dir, s) for s in shards]
        missing = [p for p in paths if not os.path.isfile(p)]
        if missing:
            raise SafetensorsError(f"{index} names shards that do not exist: {missing}")
        if paths:
            return paths
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    try:
        found = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    except OSError as e:
        raise SafetensorsError(f"cannot list model folder {model_dir!r}: {e}") from None
    if not found:
        raise SafetensorsError(f"no .safetensors files were resolved for model load in {model_dir!r}")
    return [os.path.join(model_dir, f) for f in found]
