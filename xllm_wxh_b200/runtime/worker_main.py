"""Entry point of a rank process other than rank 0 (the reference's `spawn_worker` binary /
LLMAssistantMaster, llm_master.cpp:560-592): build the engine shard and serve steps until stopped."""
from __future__ import annotations

import json
import os
import sys

from ..config import Options
from .launcher import make_engine


def main() -> int:
    opts = Options(**json.loads(os.environ["XLLM_WORKER_OPTIONS"]))
    engine = make_engine(opts)
    engine.worker_loop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
