"""A small, whole inference engine for the dense Llama-style decoder on one B200."""

from .config import (ConfigError, DenseLlamaConfig, EngineOptions, build_model,
                     config_from_dict, config_from_folder, register_architecture)

__all__ = ["ConfigError", "DenseLlamaConfig", "EngineOptions", "build_model",
           "config_from_dict", "config_from_folder", "register_architecture",
           "LLM", "Engine"]


def __getattr__(name):
    if name == "LLM":
        from .engine.llm import LLM
        return LLM
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)
