"""Starts the rank processes of one instance.

The reference's DistManager spawns one worker server per device (threads, or `spawn_worker` processes
for offline ranks > 0; xllm/core/distributed_runtime/dist_manager.cpp:144-318, worker_server.cpp:180-242).
Here every device gets its own process: under `torchrun` (RANK / WORLD_SIZE in the environment) the
processes already exist and rank 0 simply becomes the driver; otherwise rank 0 spawns ranks 1..N-1 as
`python -m xllm_wxh_b200.runtime.worker_main` children that join the same rendez-vous.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import List, Tuple

from ..config import Options
from .engine import LLMEngine


def make_engine(options: Options, **kw) -> LLMEngine:
    """The engine class the options call for (plain, or speculative when draft tokens are requested)."""
    if options.num_speculative_tokens > 0:
        from .speculative import SpeculativeEngine
        return SpeculativeEngine(options, **kw)
    return LLMEngine(options, **kw)


def launch_engine(options: Options) -> Tuple[LLMEngine, List[subprocess.Popen]]:
    devices = options.device_list()
    env_world = int(os.environ.get("WORLD_SIZE", "1"))
    procs: List[subprocess.Popen] = []
    if env_world > 1 or len(devices) <= 1:
        return make_engine(options), procs
    world = len(devices)
    addr, port = options.master_node_addr.rsplit(":", 1)
    import dataclasses
    payload = json.dumps(dataclasses.asdict(options))
    for r in range(1, world):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR=addr, MASTER_PORT=port,
                   XLLM_WORKER_OPTIONS=payload)
        procs.append(subprocess.Popen([sys.executable, "-m", "xllm_wxh_b200.runtime.worker_main"], env=env))
    os.environ.update(RANK="0", LOCAL_RANK="0", WORLD_SIZE=str(world), MASTER_ADDR=addr, MASTER_PORT=port)
    engine = make_engine(options, rank=0, world_size=world)
    return engine, procs
