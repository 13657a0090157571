"""A B200-native inference engine for the Qwen2.5 dense decoder, after jiamumuzhao/vllm-cpp.

Importing the package registers the built-in architecture and parts; nothing that
needs a GPU happens until an engine is built.
"""
from .config.engine_config import ConfigError, EngineConfig  # noqa: F401
from .config.registry import known_architectures, register_architecture, resolve_architecture  # noqa: F401
from . import models as _models  # noqa: F401  (registers the architectures)

__version__ = "0.1.0"


def __getattr__(name):
    # the entry points import the kernel library; load them only when asked for
    if name == "LLM":
        from .engine.llm import LLM
        return LLM
    if name == "Engine":
        from .engine.llm_engine import Engine
        return Engine
    if name == "SamplingParams":
        from .sampling.params import SamplingParams
        return SamplingParams
    raise AttributeError(name)
