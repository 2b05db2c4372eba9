"""Host-side cost of serving, measured without a GPU: a one-layer model whose attention is replaced by a copy runs on the
CPU, so that what is timed is the scheduler, the batch builder, output emission and - in the second part - the HTTP
streaming path (event loop, JSON chunks, socket writes).  The figures bound the token rate one process can serve
whatever the GPUs deliver.

    python -m xllm_wxh_b200.runtime.bench_host_overhead [--concurrency 256] [--tokens 64] [--no-http]

Part 1: `LLM.generate` on a wave of `concurrency` requests: milliseconds of host time per engine step.
Part 2: the same wave as streaming `/v1/completions` requests from a client process (aiohttp): streamed tokens per second.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import subprocess
import sys
import threading
import time

import torch

_CLIENT = r"""
import asyncio, json, sys, time, aiohttp
port, conc, ntok = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
async def one(s, i):
    n = 0
    body = {"prompt": " ".join(str((i * 7 + j) % 1000) for j in range(16)), "max_tokens": ntok, "temperature": 0,
            "ignore_eos": True, "stream": True}
    async with s.post(f"http://127.0.0.1:{port}/v1/completions", json=body) as r:
        async for line in r.content:
            n += line.startswith(b"data: {")
    return n
async def main():
    async with aiohttp.ClientSession(connector=aiohttp.TCPConnector(limit=0)) as s:
        await asyncio.gather(*[one(s, i) for i in range(8)])
        t0 = time.time()
        ns = await asyncio.gather(*[one(s, i) for i in range(conc)])
        print(json.dumps({"chunks": int(sum(ns)), "start": t0, "end": time.time()}))
asyncio.run(main())
"""


def _engine(concurrency: int, port: int = 0):
    from .. import ops
    from ..config import Options
    from ..models.args import ModelArgs
    from ..models.qwen import QwenForCausalLM
    from .engine import LLMEngine
    ops.paged_attention = lambda q, kc, vc, inp, scale, w=-1: q.reshape(q.shape[0], -1)      # no attention: host cost only
    args = ModelArgs(model_type="qwen3", dtype="float32", vocab_size=1024, hidden_size=64, n_layers=1, n_heads=2, n_kv_heads=1,
                     head_dim=32, intermediate_size=64, qk_norm=True, max_position_embeddings=4096)
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    opts = Options(model="preset:x", devices="cpu", block_size=16, num_kv_blocks=16384, dtype="float32", port=port, host="127.0.0.1",
                   max_concurrent_requests=4 * concurrency, model_id="x", max_seqs_per_batch=max(256, concurrency),
                   enable_prefix_cache=False)
    return opts, LLMEngine(opts, model_args=args, model=model)


def offline(concurrency: int, tokens: int) -> dict:
    from .. import LLM, SamplingParams
    opts, eng = _engine(concurrency)
    llm = LLM(model="preset:x", devices="cpu", engine=eng)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (16,), generator=g).tolist() for _ in range(concurrency)]
    llm.generate(prompts[:8], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    s0, t0 = eng.step_count, time.perf_counter()
    llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=tokens, ignore_eos=True))
    dt, n = time.perf_counter() - t0, eng.step_count - s0
    trace = eng.host_trace_summary(n)
    return {"steps": n, "ms_per_step": dt / n * 1e3, "model_forward_ms_per_step": trace.get("kernel_issue_ms", 0.0),
            "tokens_per_second_bound": concurrency * tokens / dt}


def http_streaming(concurrency: int, tokens: int, clients: int = 4) -> dict:
    import socket
    from ..api.openai_service import APIService
    from ..api.server import HttpServer
    from .master import LLMMaster
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    opts, eng = _engine(concurrency, port)
    master = LLMMaster(opts, eng)
    master.run()
    loop = asyncio.new_event_loop()
    ready = threading.Event()

    def run():
        asyncio.set_event_loop(loop)
        srv = APIService(master, opts).register(HttpServer())
        loop.run_until_complete(srv.start("127.0.0.1", port))
        ready.set()
        loop.run_forever()
    th = threading.Thread(target=run, daemon=True)
    th.start()
    ready.wait(30)
    try:
        # several client processes, so that parsing the event streams is not what bounds the rate
        best = None
        per = max(1, concurrency // clients)
        for _ in range(2):
            t0 = time.perf_counter()
            procs = [subprocess.Popen([sys.executable, "-c", _CLIENT, str(port), str(per), str(tokens)], stdout=subprocess.PIPE,
                                      text=True) for _ in range(clients)]
            rows = [json.loads(pr.communicate(timeout=600)[0].strip().splitlines()[-1]) for pr in procs]
            # the clients do not start together: the rate is over the window from the first start to the last end
            row = {"chunks": sum(r["chunks"] for r in rows), "seconds": max(r["end"] for r in rows) - min(r["start"] for r in rows),
                   "wall_seconds_with_client_start": time.perf_counter() - t0}
            if best is None or row["seconds"] < best["seconds"]:
                best = row
        concurrency = per * clients
    finally:
        loop.call_soon_threadsafe(loop.stop)
        th.join(5)
        master.stop()
    return {"chunks": best["chunks"], "seconds": best["seconds"], "streamed_tokens_per_second": concurrency * tokens / best["seconds"]}


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--concurrency", type=int, default=256)
    p.add_argument("--tokens", type=int, default=64)
    p.add_argument("--no-http", action="store_true")
    p.add_argument("--clients", type=int, default=4, help="client processes that share the streaming requests")
    p.add_argument("--watchdog", type=float, default=900.0, help="seconds after which every thread's stack is printed and the run ends")
    a = p.parse_args()
    import faulthandler
    faulthandler.dump_traceback_later(a.watchdog, exit=True)          # a run that hangs says where
    torch.set_num_threads(min(4, os.cpu_count() or 1))
    row = {"concurrency": a.concurrency, "tokens": a.tokens, "offline_generate": offline(a.concurrency, a.tokens)}
    if not a.no_http:
        row["http_streaming"] = http_streaming(a.concurrency, a.tokens, a.clients)
    print(json.dumps(row))
    return 0


if __name__ == "__main__":
    sys.exit(main())
