"""`xllm` command: start one serving instance (the reference's `xllm` binary, xllm/xllm.cpp:111-347).

    xllm --model /path/to/Qwen3-8B --devices cuda:0,cuda:1 --port 8010 [--enable_prefix_cache=false ...]

Flag names and defaults are the reference's (core/common/global_flags.cpp).  One process is started per device.  With
`--nnodes > 1`, `--node_rank 0` hosts the API and the scheduler; the other nodes only run their rank processes
(xllm.cpp:327-340).  `--instance_role PREFILL|DECODE --enable_disagg_pd` joins a prefill/decode pair over the control
port `--disagg_pd_port` (DECODE listens, PREFILL connects to `--decode_addr`).
"""
from __future__ import annotations

import argparse
import asyncio
import logging
import os
import signal
import sys
from typing import List, Optional

from .config import Options, add_flags, options_from_namespace

log = logging.getLogger("xllm")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="xllm", description="B200-native LLM serving engine", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    add_flags(p)
    p.add_argument("--decode_addr", default="", help="host:port of the DECODE instance's control service (PREFILL role).")
    p.add_argument("--log_level", default="INFO")
    return p


def _node_worker_only(options: Options) -> int:
    """Nodes other than node 0: run this node's rank processes and wait (no API, no scheduler)."""
    import subprocess
    import json
    import dataclasses
    devices = options.device_list()
    per_node = len(devices)
    world = per_node * options.nnodes
    addr, port = options.master_node_addr.rsplit(":", 1)
    payload = json.dumps(dataclasses.asdict(options))
    procs = []
    for i in range(per_node):
        r = options.node_rank * per_node + i
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(i), WORLD_SIZE=str(world), MASTER_ADDR=addr, MASTER_PORT=port,
                   XLLM_WORKER_OPTIONS=payload)
        procs.append(subprocess.Popen([sys.executable, "-m", "xllm_wxh_b200.runtime.worker_main"], env=env))
    rc = 0
    for pr in procs:
        rc = pr.wait() or rc
    return rc


def main(argv: Optional[List[str]] = None) -> int:
    ns = build_parser().parse_args(argv)
    logging.basicConfig(level=getattr(logging, str(ns.log_level).upper(), logging.INFO),
                        format="%(asctime)s %(levelname).1s %(name)s: %(message)s")
    options = options_from_namespace(ns)
    if not options.model:
        print("--model is required", file=sys.stderr)
        return 2
    if options.nnodes > 1 and options.node_rank != 0:
        return _node_worker_only(options)

    from .runtime.launcher import launch_engine
    from .runtime.master import LLMMaster
    from .utils.health import HEALTH
    engine, procs = launch_engine(options)
    master = LLMMaster(options, engine=engine)
    coordinator = None
    if options.enable_disagg_pd and options.instance_role in ("PREFILL", "DECODE"):
        from .runtime import disagg_pd
        if options.instance_role == "DECODE":
            coordinator = disagg_pd.DecodeCoordinator(master)
            coordinator.serve(options.disagg_pd_port)
            log.info("DECODE instance: control service on port %d", options.disagg_pd_port)
        else:
            if ns.decode_addr:
                h, pt = ns.decode_addr.rsplit(":", 1)
                coordinator = disagg_pd.PrefillCoordinator(master, disagg_pd.SocketTransport.connect(h, int(pt)))
                log.info("PREFILL instance: linked to decode instance %s", ns.decode_addr)
            elif master.xservice is not None:
                # no fixed partner: follow the DECODE instances that are registered with the service layer
                from .runtime.pd_discovery import DecodeLinker
                coordinator = disagg_pd.PrefillCoordinator(master)
                linker = DecodeLinker(coordinator, master.xservice)
                linker.start()
                log.info("PREFILL instance: decode instances are taken from the service at %s", options.etcd_addr)
            else:
                print("--instance_role PREFILL needs --decode_addr, or --enable_service_routing with --etcd_addr",
                      file=sys.stderr)
                return 2

    if options.enable_xtensor:
        from .runtime.weight_transfer import WeightServer
        try:
            master.weight_server = WeightServer(master)
            master.weight_server.serve(options.transfer_listen_port)
            log.info("weight service on port %d", options.transfer_listen_port)
        except OSError as e:
            master.weight_server = None
            log.warning("weight service not started: %s", e)

    def child_alive():
        dead = [p.pid for p in procs if p.poll() is not None]
        return (not dead, f"rank process exited: {dead}" if dead else "")
    HEALTH.register("rank_processes", child_alive)
    HEALTH.start(options.health_check_interval_ms)
    master.run()

    from .api.openai_service import serve
    loop = asyncio.new_event_loop()
    asyncio.set_event_loop(loop)
    task = loop.create_task(serve(master, options))
    for sig in (signal.SIGINT, signal.SIGTERM):
        try:
            loop.add_signal_handler(sig, task.cancel)
        except (NotImplementedError, RuntimeError):
            pass
    log.info("serving %s on %s:%d", master.model_id, options.host or "0.0.0.0", options.port)
    try:
        loop.run_until_complete(task)
    except asyncio.CancelledError:
        pass
    finally:
        HEALTH.stop()
        master.stop()
        for p in procs:
            try:
                p.wait(timeout=10)
            except Exception:
                p.kill()
    return 0


if __name__ == "__main__":
    sys.exit(main())
