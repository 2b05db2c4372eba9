"""DeepSeek-V2/V3 (MLA + MoE) and the MTP draft model: see `deepseek_impl` (registered on import)."""
from .deepseek_impl import *  # noqa: F401,F403
