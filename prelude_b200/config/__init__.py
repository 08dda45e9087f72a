"""Typed configurations and the architecture registry."""
from .registry import (ConfigError, load_model_config, load_model_spec, read_config_json, register_architecture,
                       registered_architectures, resolve_architecture, unregister_architecture)
from . import qwen3 as _qwen3  # noqa: F401  (registers Qwen3)
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "Qwen3Config", "load_model_config", "load_model_spec", "read_config_json",
           "register_architecture", "registered_architectures", "resolve_architecture", "unregister_architecture"]
