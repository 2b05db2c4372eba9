#!/usr/bin/env python
"""Serving benchmark: output tokens/s per box at fixed concurrency (+ p50 TTFT / TPOT).

Workload (the Qwen3-8B configuration of the baseline definition): `--concurrency` requests are always in
flight, each with a `--prompt-len`-token random prompt and `--output-len` generated tokens (EOS ignored), block
size 16, continuous batching with chunked prefill.  The system is first ramped to its steady state: requests arrive at the
fixed rate that keeps `--concurrency` of them in flight (concurrency / output-len per step: one per step for 256 / 256), so
after `output-len` steps every step decodes one token for each running request and prefills the prompts that arrived.
Then W warm-up steps (at least 3) and K timed steps follow.

One "step" is one engine iteration: scheduler (C++) -> packed inputs in pinned memory -> H2D copy -> model forward
(hand-written sm_100a kernels) -> sampler -> D2H of the sampled tokens.  The timed region is bracketed by a
barrier + device synchronisation on every rank; elapsed time is taken with CUDA events on each rank's stream and
reduced with MAX over ranks.

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29501 \
        bench.py --gpus 8 --steps 64 --warmup 8
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

METRIC = "output_tok_per_s_per_box_at_fixed_concurrency"


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=64)
    p.add_argument("--warmup", type=int, default=8)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference", "nccl"])
    p.add_argument("--model", type=str, default="qwen3-8b")
    p.add_argument("--concurrency", type=int, default=256)
    p.add_argument("--prompt-len", type=int, default=1024)
    p.add_argument("--output-len", type=int, default=256)
    p.add_argument("--block-size", type=int, default=16)
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-overlap", action="store_true")
    p.add_argument("--no-graph", action="store_true", help="run every step eagerly (no CUDA graphs)")
    p.add_argument("--parallel", type=str, default="tp", choices=["tp", "ep"],
                   help="tp: tensor parallel over all GPUs; ep: attention data-parallel x expert-parallel over all GPUs (MoE models)")
    p.add_argument("--pd", type=str, default="", help="P+D: prefill / decode disaggregation with P prefill and D decode instances of one "
                   "GPU each (1+1 on two GPUs); the KV blocks travel over NVLink (--pd-mode PUSH or PULL)")
    p.add_argument("--pd-mode", type=str, default="PUSH", choices=["PUSH", "PULL"])
    p.add_argument("--layers", type=int, default=0, help="run only the first N layers of the preset (a model too large for the "
                   "GPUs at hand, e.g. deepseek-v3; the result is then a per-depth figure, not the named model's headline)")
    p.add_argument("--router-zipf", type=float, default=0.0,
                   help="MoE: add log of a Zipf(s) expert popularity to the router logits (skewed expert load); 0: off")
    p.add_argument("--eplb", action="store_true", help="MoE: expert-parallel load balancing with one redundant slot per rank")
    p.add_argument("--tp-mlp-mode", type=str, default="auto", choices=["auto", "tp", "rows"],
                   help="dense MLP under tensor parallelism: sharded weights (tp), replicated weights run by rows, or auto")
    p.add_argument("--seed", type=int, default=0)
    return p.parse_args()


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs (read-only queries)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(power), "samples": len(sm),
                "reasons": sorted(reasons)}


def reference_arm(a):
    if int(os.environ.get("RANK", "0")) != 0:          # launched as N ranks: one line, from rank 0
        return 0
    out = {"impl": "reference", "metric": METRIC, "n_gpus": a.gpus,
           "unavailable": "refused by a safety check: offline pip install of the reference tree was denied (its build code may not "
                          "run here); the reference also needs network-fetched submodules, vcpkg and FlashInfer AOT modules"}
    print(json.dumps(out))
    return 0


def pd_arm(a):
    """Disaggregated serving, one prefill and one decode instance (one GPU each, one process each: ranks 0 and 1 of the
    launch).  The prefill instance takes the requests, computes the prompts and hands every request over after its first
    token; the KV blocks cross NVLink under the forward pass (PUSH) or are fetched by the decode instance (PULL); the decode
    instance streams the tokens back.  Timed: a wave of `concurrency` requests through `LLM.generate` on the prefill
    instance, wall clock, after one untimed wave of the same shape.  One JSON line from rank 0."""
    rank = int(os.environ.get("RANK", "0"))
    port = 27000 + int(os.environ.get("MASTER_PORT", "29517")) % 2000
    json_fd = os.dup(1)
    os.dup2(2, 1)
    import numpy as np
    import torch
    from xllm_wxh_b200 import LLM, SamplingParams
    from xllm_wxh_b200.config import Options
    from xllm_wxh_b200.ops import cuda_ops
    from xllm_wxh_b200.runtime.disagg_pd import DecodeCoordinator, PrefillCoordinator, SocketTransport
    from xllm_wxh_b200.runtime.engine import LLMEngine
    from xllm_wxh_b200.runtime.master import LLMMaster
    torch.cuda.set_device(rank)
    ctx = a.prompt_len + a.output_len
    blocks_per_seq = (ctx + a.block_size - 1) // a.block_size + 1
    role = "PREFILL" if rank == 0 else "DECODE"
    opts = Options(model=f"preset:{a.model}", devices=f"cuda:{rank}", block_size=a.block_size,
                   max_tokens_per_batch=4 * a.prompt_len + a.concurrency, max_seqs_per_batch=a.concurrency + 8,
                   max_tokens_per_chunk_for_prefill=a.prompt_len, enable_chunked_prefill=True, enable_prefix_cache=False,
                   enable_schedule_overlap=not a.no_overlap, max_model_len=ctx + 64,
                   num_kv_blocks=(a.concurrency + 16) * blocks_per_seq + 64, enable_graph=not a.no_graph,
                   enable_prefill_piecewise_graph=not a.no_graph, max_tokens_for_graph_mode=4 * a.prompt_len + a.concurrency,
                   random_seed=a.seed, enable_disagg_pd=True, instance_role=role, kv_cache_transfer_mode=a.pd_mode)
    os.environ["LOCAL_RANK"] = str(rank)
    engine = LLMEngine(opts, rank=0, world_size=1)
    master = LLMMaster(opts, engine)
    stop_file = f"/tmp/xllm_bench_pd_{port}.stop"
    if rank == 1:
        if os.path.exists(stop_file):
            os.remove(stop_file)
        DecodeCoordinator(master).serve(port)
        master.run()
        deadline = time.time() + 1500
        while not os.path.exists(stop_file) and time.time() < deadline:
            time.sleep(0.05)
        sys.stderr.write(f"decode instance: {engine.scheduler.stats()['generated_tokens']} tokens, status {cuda_ops.read_status()}\n")
        os._exit(0)
    llm = LLM(model=opts.model, devices=opts.devices, engine=engine)
    llm.master = master
    PrefillCoordinator(master, SocketTransport.connect("127.0.0.1", port, timeout=600.0))
    llm.generate_timeout_s = 1200.0
    rng = np.random.default_rng(a.seed)
    V = engine.args.vocab_size
    sp = SamplingParams(temperature=0.0, max_tokens=a.output_len, ignore_eos=True)
    try:
        llm.generate([rng.integers(0, V, a.prompt_len).tolist() for _ in range(a.concurrency)], sp)     # untimed wave
        prompts = [rng.integers(0, V, a.prompt_len).tolist() for _ in range(a.concurrency)]
        sampler = ClockSampler(0)
        sampler.start()
        moved0 = getattr(engine.kv_transfer, "bytes_moved", 0) if engine.kv_transfer else 0
        s0 = engine.step_count
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        clocks = sampler.stop()
    finally:
        open(stop_file, "w").close()
    n_tok = sum(len(o.outputs[0].token_ids) for o in outs)
    moved = (getattr(engine.kv_transfer, "bytes_moved", 0) if engine.kv_transfer else 0) - moved0
    out = {"metric": METRIC, "value": n_tok / dt, "unit": "tok/s", "n_gpus": 2, "steps": a.steps, "warmup": a.warmup,
           "ms_per_step": None, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)", "impl": a.impl,
           "config": {"model": a.model, "global_batch": a.concurrency, "seq_len": ctx, "prompt_len": a.prompt_len,
                      "output_len": a.output_len, "block_size": a.block_size, "parallelism": "pd 1+1 (one GPU per instance)",
                      "kv_cache_transfer_mode": a.pd_mode, "what": "one wave of requests through LLM.generate on the prefill "
                      "instance (prefill burst, hand-over, decode on the other GPU), wall clock; one untimed wave before it"},
           "seconds": dt, "output_tokens": n_tok, "prefill_steps": engine.step_count - s0, "kv_bytes_pushed": moved,
           "clocks": clocks, "device_status": cuda_ops.read_status(), "gpu_launches": engine.kernel_launches()}
    os.write(json_fd, (json.dumps(out) + "\n").encode())
    os._exit(0)


def main():
    a = parse()
    if a.impl == "reference":
        return reference_arm(a)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if a.pd:
        if a.pd != "1+1":
            print(json.dumps({"metric": METRIC, "unavailable": "--pd takes 1+1 (one GPU per instance)"}))
            return 0
        a.gpus = 2
    if a.gpus > 1 and world == 1:     # convenience: re-launch under torchrun
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}", "--master-addr",
               "127.0.0.1", "--master-port", "29517", os.path.abspath(__file__)] + sys.argv[1:]
        return subprocess.call(cmd)
    if a.pd:
        return pd_arm(a)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # libraries (NCCL's version banner, ...) must not write to the stream that carries the one JSON line
    json_fd = os.dup(1)
    os.dup2(2, 1)

    import numpy as np
    import torch
    from xllm_wxh_b200 import LLM, SamplingParams
    from xllm_wxh_b200.config import Options
    from xllm_wxh_b200.ops import cuda_ops
    from xllm_wxh_b200.runtime.engine import LLMEngine
    from xllm_wxh_b200 import _core

    torch.cuda.set_device(local_rank)
    ctx = a.prompt_len + a.output_len
    blocks_per_seq = (ctx + a.block_size - 1) // a.block_size + 1
    opts = Options(model=f"preset:{a.model}", devices=",".join(f"cuda:{i}" for i in range(max(1, a.gpus))),
                   block_size=a.block_size, max_tokens_per_batch=4 * a.prompt_len + a.concurrency,
                   max_seqs_per_batch=a.concurrency + 8, max_tokens_per_chunk_for_prefill=a.prompt_len,
                   enable_chunked_prefill=True, enable_prefix_cache=False, enable_schedule_overlap=not a.no_overlap,
                   max_memory_utilization=0.9, max_model_len=ctx + 64,
                   num_kv_blocks=(a.concurrency + 16) * blocks_per_seq + 64,
                   enable_graph=not a.no_graph, enable_prefill_piecewise_graph=not a.no_graph,
                   max_tokens_for_graph_mode=4 * a.prompt_len + a.concurrency,
                   communication_backend="nccl" if a.impl == "nccl" else "fused", random_seed=a.seed,
                   tp_mlp_mode=a.tp_mlp_mode)
    if a.parallel == "ep" and a.gpus > 1:
        # every GPU runs attention on its own requests (data parallel) and holds 1 / N of the experts; the all-to-all is the
        # fused dispatch / combine (--impl ours) or all-gather + all-reduce through NCCL (--impl nccl)
        opts.dp_size = opts.ep_size = a.gpus
        opts.expert_parallel_degree = 0 if a.impl == "nccl" else 2
        opts.max_seqs_per_batch = a.concurrency // a.gpus + 8
        opts.num_kv_blocks = (a.concurrency // a.gpus + 16) * blocks_per_seq + 64
        # One prompt arrives per step and lands whole on one DP rank (chunks of prompt_len / N tokens were tried to even the
        # ranks out: the step shapes then vary from step to step, graphs are captured all the time, and the 4-GPU step
        # went from 24 to 29 ms).
    if a.eplb:
        opts.enable_eplb, opts.redundant_experts_num = True, 1
        opts.eplb_update_interval, opts.eplb_update_threshold = 64, 1.1
    model_args = None
    if a.layers > 0:
        import dataclasses
        from xllm_wxh_b200.models.args import preset
        model_args = dataclasses.replace(preset(a.model), n_layers=a.layers, num_nextn_predict_layers=0)
    engine = LLMEngine(opts, model_args=model_args)
    if a.router_zipf > 0 and engine.args.n_routed_experts > 0:
        E = engine.args.n_routed_experts
        pop = 1.0 / (np.random.default_rng(a.seed + 7).permutation(E) + 1.0) ** a.router_zipf
        engine.worker.model.router_logit_bias = torch.tensor(np.log(pop / pop.sum()), dtype=torch.float32, device=engine.device)
    if rank != 0:
        engine.worker_loop()
        return 0

    rng = np.random.default_rng(a.seed)
    V = engine.args.vocab_size
    sp = _core.SamplingParams()                 # greedy, as in the baseline definition
    sched = engine.scheduler
    t_add, t_first, t_last, n_out = {}, {}, {}, {}
    ttft, tpot = [], []

    def add(max_tokens):
        st = _core.StopCriteria()
        st.max_tokens, st.ignore_eos = int(max_tokens), True
        rid = engine.add_request(rng.integers(0, V, a.prompt_len).tolist(), sp, st)
        t_add[rid] = time.perf_counter()
        n_out[rid] = 0

    def pump(outs):
        """Account the outputs of one engine step.  Returns tokens produced."""
        now = time.perf_counter()
        produced = 0
        for o in outs:
            k = len(o.new_tokens)
            if k:
                produced += k
                rid = o.request_id
                if rid not in t_first:
                    t_first[rid] = now
                    ttft.append((now - t_add[rid]) * 1e3)
                else:
                    tpot.append((now - t_last[rid]) * 1e3 / k)
                t_last[rid] = now
            if o.request_finished:
                for d in (t_add, t_first, t_last, n_out):
                    d.pop(o.request_id, None)
        return produced

    # Requests arrive at the fixed rate that keeps `concurrency` of them in flight: concurrency / output_len new requests
    # per step (one per step for 256 / 256), each living for output_len steps.  Every step of the steady state is then
    # the same: one decode token for each running request plus the prompts that arrived.
    credit = [0.0]

    def arrivals():
        credit[0] += a.concurrency / a.output_len
        k = int(credit[0])
        credit[0] -= k
        for _ in range(k):
            add(a.output_len)

    def one_step():
        arrivals()
        return pump(engine.step())

    # ---- ramp to the steady state (set-up, untimed): after output_len steps the population is complete
    for _ in range(a.output_len + 8):
        one_step()
    a.warmup = max(3, a.warmup)                 # never fewer than three untimed steps in the steady state
    for _ in range(a.warmup):
        one_step()
    ttft.clear(); tpot.clear()

    # ---- timed region
    engine.barrier_sync()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0, h2d0, d2h0 = engine.kernel_launches(), engine.worker.h2d_bytes, engine.worker.d2h_bytes
    kt = cuda_ops.kernel_timing()      # XLLM_KERNEL_TIMING=1: per-entry-point device time (diagnosis only)
    if kt is not None:
        kt.reset()
    engine.mark_timing(0)
    wall0 = time.perf_counter()
    produced = 0
    torch.cuda.nvtx.range_push("xllm_timed")       # lets a profiler restrict itself to the timed steps
    for _ in range(a.steps):
        produced += one_step()
    torch.cuda.nvtx.range_pop()
    engine.mark_timing(1)
    engine.barrier_sync()
    wall = time.perf_counter() - wall0
    elapsed_ms = engine.elapsed_ms_max_over_ranks()
    clocks = sampler.stop()
    launches = engine.kernel_launches() - launches0
    host_ms = engine.host_trace_summary(a.steps)
    if kt is not None:
        rows = sorted(kt.summary().items(), key=lambda kv: -kv[1][1])
        sys.stderr.write("kernel timing (rank 0), ms per step:\n" + "".join(
            f"  {n:36s} {c / a.steps:7.1f} launches {t / a.steps:9.3f} ms\n" for n, (c, t) in rows))
    h2d = (engine.worker.h2d_bytes - h2d0) / a.steps
    d2h = (engine.worker.d2h_bytes - d2h0) / a.steps
    value = produced / (elapsed_ms * 1e-3)
    ttft_p50 = statistics.median(ttft) if ttft else None
    tpot_p50 = statistics.median(tpot) if tpot else None
    status = cuda_ops.read_status()

    # ---- end to end through the public API: LLM.generate on a fresh wave of `concurrency` requests
    e2e = None
    if not a.no_e2e:
        # drain the steady-state population first
        for rid in list(t_add):
            engine.cancel(rid)
        while engine.has_unfinished():
            engine.step()
        llm = LLM(model=opts.model, devices=opts.devices, engine=engine)
        # one untimed wave of the same shape first: the graphs of this workload's step shapes are captured here
        warm = [rng.integers(0, V, a.prompt_len).tolist() for _ in range(a.concurrency)]
        llm.generate(warm, SamplingParams(temperature=0.0, max_tokens=a.output_len, ignore_eos=True))
        prompts = [rng.integers(0, V, a.prompt_len).tolist() for _ in range(a.concurrency)]
        h2d0, d2h0, s0 = engine.worker.h2d_bytes, engine.worker.d2h_bytes, engine.step_count
        engine.barrier_sync()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=a.output_len, ignore_eos=True))
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        n_tok = sum(len(o.outputs[0].token_ids) for o in outs)
        nsteps = max(1, engine.step_count - s0)
        e2e = {"value": n_tok / dt, "unit": "tok/s", "seconds": dt, "output_tokens": n_tok, "steps": nsteps,
               "h2d_bytes_per_step": (engine.worker.h2d_bytes - h2d0) / nsteps,
               "d2h_bytes_per_step": (engine.worker.d2h_bytes - d2h0) / nsteps,
               "what": "LLM.generate() on a fresh wave of requests (prefill burst then decode; one untimed wave before it), wall clock incl. scheduling, "
                       "pinned-host -> device input copies and device -> host token reads every step"}
    engine.shutdown()

    out = {
        "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": elapsed_ms / a.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)",
        "impl": a.impl,
        "config": {"model": a.model if a.layers <= 0 else f"{a.model} (first {a.layers} layers only: not the named model's headline)",
                   "global_batch": a.concurrency, "seq_len": a.prompt_len + a.output_len,
                   "prompt_len": a.prompt_len, "output_len": a.output_len, "block_size": a.block_size,
                   "parallelism": f"tp{a.gpus}" if a.parallel == "tp" else f"dp{a.gpus} x ep{a.gpus}",
                   "prefill_chunk_tokens": opts.max_tokens_per_chunk_for_prefill, "router_zipf": a.router_zipf, "eplb": a.eplb, "schedule_overlap": not a.no_overlap, "cuda_graphs": not a.no_graph,
                   "tp_mlp": ("rows: attention tensor parallel; every rank holds the whole MLP and runs it on its own rows"
                              if engine.comm.cfg.mlp_replicated else "tp: MLP weights sharded"),
                   "tokens_per_step": {"decode": a.concurrency, "prefill": a.prompt_len * a.concurrency / a.output_len},
                   "arrivals_per_step": a.concurrency / a.output_len,
                   "l2": "no flush needed: every step streams the full weights and the KV cache (>> 126 MB L2)"},
        "ttft_p50_ms": ttft_p50, "tpot_p50_ms": tpot_p50, "wall_ms_per_step": wall * 1e3 / a.steps,
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
        "device_status": status, "host_ms_per_step": host_ms,
    }
    os.write(json_fd, (json.dumps(out) + "\n").encode())
    return 0


if __name__ == "__main__":
    sys.exit(main())
