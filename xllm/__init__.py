"""Drop-in name: `from xllm import LLM, SamplingParams, ArgumentParser` keeps working for code written
against the reference's Python package (xllm/__init__.py:13-83 of the reference re-exports the same names)."""
from xllm_wxh_b200 import *  # noqa: F401,F403
from xllm_wxh_b200 import __all__, __version__  # noqa: F401
