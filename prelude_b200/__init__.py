"""prelude_b200: a small, whole inference engine for one GPU (sm_100a).

    from prelude_b200 import Engine, SamplingParams
    engine = Engine("/path/to/model_dir")
    result = engine.generate([1, 2, 3], temperature=0.0, max_new_tokens=16)

Importing the package touches neither CUDA nor the kernel library; both come
in when an Engine (or anything else that runs on the device) is made.
"""
from .config import ConfigError, Qwen3Config, load_model_config, register_architecture  # noqa: F401

__all__ = ["Engine", "SamplingParams", "GenerateResult", "StepEntry", "ConfigError", "Qwen3Config",
           "load_model_config", "register_architecture"]


def __getattr__(name):
    if name in ("Engine", "GenerateResult"):
        from .engine import engine as _e
        return getattr(_e, name)
    if name == "SamplingParams":
        from .engine.scheduler import SamplingParams
        return SamplingParams
    if name == "StepEntry":
        from .engine.runner import StepEntry
        return StepEntry
    raise AttributeError(f"module 'prelude_b200' has no attribute {name!r}")
