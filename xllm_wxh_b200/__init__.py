"""B200-native LLM serving engine with the capabilities and public API of xLLM.

    from xllm_wxh_b200 import LLM, SamplingParams      # or: from xllm import LLM, SamplingParams
"""
from __future__ import annotations

__version__ = "0.1.0"


def _ensure_core():
    """Build the C++ host runtime on first import if the shared object is missing or stale.  `XLLM_CORE_SO` names an
    alternative build of the same extension (the AddressSanitizer / UBSan build of `build_ext.build_core_sanitized`)."""
    import os
    alt = os.environ.get("XLLM_CORE_SO")
    if alt:
        import importlib.util
        import sys
        spec = importlib.util.spec_from_file_location(__name__ + "._core", alt)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules[__name__ + "._core"] = mod
        globals()["_core"] = mod
        return
    try:
        from . import _core  # noqa: F401
    except ImportError:
        from .build_ext import build_core
        build_core()
        from . import _core  # noqa: F401


_ensure_core()

from .api.llm import LLM, ArgumentParser, Embedding  # noqa: E402
from .config import Options  # noqa: E402
from .framework.params import (BeamSearchParams, LogProb, PoolingParams, RequestOutput, RequestParams,  # noqa: E402
                               SamplingParams, SequenceOutput, Status, StatusCode, Usage)

__all__ = ["LLM", "Embedding", "ArgumentParser", "Options", "SamplingParams", "BeamSearchParams", "PoolingParams",
           "RequestParams", "RequestOutput", "SequenceOutput", "Status", "StatusCode", "Usage", "LogProb"]
