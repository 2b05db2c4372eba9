"""B200-native LLM serving engine with the capabilities and public API of xLLM.

    from xllm_wxh_b200 import LLM, SamplingParams      # or: from xllm import LLM, SamplingParams
"""
from __future__ import annotations

__version__ = "0.1.0"


def _ensure_core():
    """Build the C++ host runtime on first import if the shared object is missing or stale."""
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
