"""name -> model class registry (reference: xllm/models/model_registry.h `REGISTER_CAUSAL_MODEL`)."""
from __future__ import annotations

from typing import Callable, Dict

_MODELS: Dict[str, Callable] = {}


def register_model(*names: str):
    def deco(cls):
        for n in names:
            _MODELS[n] = cls
        return cls
    return deco


def get_model_class(model_type: str):
    if model_type not in _MODELS:
        from . import qwen, deepseek  # noqa: F401  (populate the registry)
    if model_type not in _MODELS:
        raise KeyError(f"model_type '{model_type}' is not registered; known: {sorted(_MODELS)}")
    return _MODELS[model_type]


def registered_models():
    from . import qwen, deepseek  # noqa: F401
    return sorted(_MODELS)
