"""One registry from an architecture's name to its configuration class.

Resolution follows the reference (crates/prelude-core/src/models/registry.rs:79-196,
crates/prelude-core/src/engine/config.rs:85-120): each entry of config.json's
``architectures`` is split at the first "For"; the part before it is matched
against the registered architecture aliases after dropping everything that is
not an ASCII letter or digit and lower-casing; the part after it names the task
and must be a text-generation suffix.  If no entry resolves, ``model_type`` is
matched against the model-type aliases.  Otherwise an error names both.

An architecture registers a class with

    @register_architecture("Qwen3", aliases=("Qwen3", "Qwen3Model"), model_types=("qwen3",))
    class Qwen3Config: ...

The class needs ``from_dict(raw: dict) -> config`` and ``config.to_model_spec()
-> ModelSpec``; nothing else in the framework is touched.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

from .spec import ModelSpec


class ConfigError(ValueError):
    """config.json cannot be read, resolved or parsed."""


_GENERATE_SUFFIXES = ("causallm", "conditionalgeneration", "textgeneration", "generation")
_OTHER_TASK_SUFFIXES = {"sequenceclassification": "Classify", "embedding": "Embed", "textembedding": "Embed"}


def normalize_identifier(text: str) -> str:
    return "".join(ch.lower() for ch in text if ch.isascii() and ch.isalnum())


@dataclass(frozen=True)
class ArchEntry:
    name: str
    aliases: Tuple[str, ...]
    model_types: Tuple[str, ...]
    config_cls: type


_REGISTRY: Dict[str, ArchEntry] = {}


def register_architecture(name: str, aliases: Tuple[str, ...] = (), model_types: Tuple[str, ...] = ()) -> Callable:
    def deco(cls):
        entry = ArchEntry(name, tuple(aliases) or (name,), tuple(model_types), cls)
        _REGISTRY[name] = entry
        return cls
    return deco


def unregister_architecture(name: str) -> None:
    _REGISTRY.pop(name, None)


def registered_architectures() -> List[str]:
    return sorted(_REGISTRY)


def _find_by_alias(prefix: str) -> Optional[ArchEntry]:
    key = normalize_identifier(prefix)
    for entry in _REGISTRY.values():
        if any(normalize_identifier(a) == key for a in entry.aliases):
            return entry
    return None


def _find_by_model_type(model_type: str) -> Optional[ArchEntry]:
    key = normalize_identifier(model_type)
    for entry in _REGISTRY.values():
        if any(normalize_identifier(a) == key for a in entry.model_types):
            return entry
    return None


def resolve_architecture(raw: dict) -> ArchEntry:
    """The registry entry that config.json's ``architectures`` / ``model_type`` name."""
    names = raw.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    model_type = raw.get("model_type")
    for name in names:
        if not isinstance(name, str) or "For" not in name:
            continue
        prefix, suffix = name.split("For", 1)
        entry = _find_by_alias(prefix)
        if entry is None:
            continue
        task = normalize_identifier(suffix)
        if task in _GENERATE_SUFFIXES:
            return entry
        if task in _OTHER_TASK_SUFFIXES:
            raise ConfigError(
                f"task {_OTHER_TASK_SUFFIXES[task]!r} is not supported for architecture {entry.name!r}: "
                "this engine generates text only")
    if isinstance(model_type, str):
        entry = _find_by_model_type(model_type)
        if entry is not None:
            return entry
    raise ConfigError(
        "unable to resolve model architecture from config metadata: "
        f"architectures={list(names)!r}, model_type={model_type!r}; known: {registered_architectures()}")


def extract_eos_token_ids(raw: dict, required: bool = False) -> Tuple[int, ...]:
    """``eos_token_id`` as a tuple: an integer, a list of integers, or nested
    under ``text_config`` (crates/prelude-core/src/engine/config.rs:122-170).

    The reference refuses a generation model without it; here it is optional
    unless ``required``, because replay and random-weight folders stop on no
    token.
    """
    value = raw.get("eos_token_id")
    if value is None and isinstance(raw.get("text_config"), dict):
        value = raw["text_config"].get("eos_token_id")
    if value is None:
        if required:
            raise ConfigError("generation model config is missing required field `eos_token_id`")
        return ()
    if isinstance(value, bool):
        raise ConfigError("generation model config has invalid `eos_token_id` type")
    if isinstance(value, int):
        if value < 0:
            raise ConfigError("generation model config has invalid non-integer `eos_token_id`")
        return (value,)
    if isinstance(value, list):
        ids = []
        for v in value:
            if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                raise ConfigError("generation model config has non-integer entry in `eos_token_id`")
            ids.append(v)
        if not ids:
            raise ConfigError("generation model config has empty `eos_token_id`")
        return tuple(ids)
    raise ConfigError("generation model config has invalid `eos_token_id` type")


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json in model folder {model_dir!r}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return raw


def load_model_config(model_dir_or_dict):
    """Typed configuration of a model folder (or of an already parsed dict)."""
    raw = model_dir_or_dict if isinstance(model_dir_or_dict, dict) else read_config_json(model_dir_or_dict)
    entry = resolve_architecture(raw)
    return entry.config_cls.from_dict(raw)


def load_model_spec(model_dir_or_dict) -> ModelSpec:
    return load_model_config(model_dir_or_dict).to_model_spec()
