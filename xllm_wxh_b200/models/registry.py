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
        _populate()
    if model_type not in _MODELS:
        raise KeyError(f"model_type '{model_type}' is not registered; known: {sorted(_MODELS)}")
    return _MODELS[model_type]


def _populate():
    import importlib
    for mod in ("qwen", "deepseek_impl"):
        importlib.import_module(f"{__package__}.{mod}")


def registered_models():
    _populate()
    return sorted(_MODELS)
