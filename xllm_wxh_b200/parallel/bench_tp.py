"""Microbenchmark of the tensor-parallel row-parallel step  y = all_reduce(x W^T) ; residual' = y + residual ;
h = RMSNorm(residual')  on N ranks of one node, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29533 \
        -m xllm_wxh_b200.parallel.bench_tp [--tokens 1280] [--hidden 4096] [--k-total 4096,12288] [--iters 50]

Implementations timed on every rank with CUDA events (all ranks start from a barrier; one sample is a chain of steps with
distinct weights, larger than L2 together; the median per-step time is reduced with MAX over ranks):
  fused-nvls : GEMM into a multicast-bound buffer + flag; the owner reads its rows with `multimem.ld_reduce` (the NVSwitch
               adds the partials of all ranks), normalises, and writes them to every rank with `multimem.st`
  fused-pull : GEMM into a peer-mapped buffer + flag, owner fetches and reduces its rows, normalises, all-gathers
  fused-push : GEMM epilogue stores rows into the owner's buffer, owner reduces, normalises, all-gathers
  nccl       : GEMM, NCCL all-reduce, add + RMSNorm kernel (what the reference does)
The roofline of the step is the slower of the GEMM at the measured cuBLAS bf16 peak and of the bytes each GPU must
receive over NVLink at the measured per-direction peer bandwidth: reduce-scatter plus all-gather over peer memory bring in
2 (n-1)/n of the activation; with the reduction in the switch one activation (1/n reduced rows + (n-1)/n gathered rows)
enters and one leaves, and the nvls row is held against that tighter bound.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def bench_sampling(a, comm, dev, rank, world):
    """Vocabulary-parallel sampling: rows x (vocab / ranks) logits per rank."""
    import numpy as np
    from .. import ops
    from ..framework.step_input import StepInput, make_layout
    S, V = 256, 151936
    Vs = V // world
    g = torch.Generator(device=dev).manual_seed(3 + rank)
    logits = (torch.randn(S, Vs, device=dev, generator=g) * 2.5).to(torch.bfloat16)
    L = make_layout(S, S, 1, S, 32)
    host = torch.zeros(L.total_words, dtype=torch.int32)
    host[L.temperature:L.temperature + S] = torch.full((S,), 0.8).view(torch.int32)
    host[L.top_p:L.top_p + S] = torch.full((S,), 0.9).view(torch.int32)
    host[L.top_k:L.top_k + S] = 50
    host[L.seed_lo:L.seed_lo + S] = torch.arange(S, dtype=torch.int32)
    hdr = np.zeros(32, dtype=np.int32)
    hdr[0] = hdr[1] = hdr[2] = S
    inp = StepInput(host.to(dev), L, hdr)
    W = 96

    def gathered():
        full = comm.all_gather(logits, dim=-1)
        return ops.sample(full, inp)[0]

    def candidates():
        vals, ids, over = ops.topk_candidates(logits, inp, rank * Vs, W)
        packed = torch.cat([vals, ids.view(torch.float32)], dim=-1).contiguous()
        allc = comm.all_gather(packed, dim=0).view(world, S, 2 * W)
        mv = allc[:, :, :W].permute(1, 0, 2).reshape(S, world * W).contiguous()
        mi = allc[:, :, W:].contiguous().view(torch.int32).view(world, S, W).permute(1, 0, 2).reshape(S, world * W)
        pick = ops.sample(mv, inp)[0]
        return mi.gather(1, pick.long()[:, None])[:, 0]
    same = int((gathered() == candidates()).sum().item())
    res = {}
    for name, fn in (("logits gathered", gathered), ("per-shard candidates", candidates)):
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(a.iters):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(4):
                fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / 4)
        t = torch.tensor(sorted(times)[len(times) // 2], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[name] = float(t.item())
    if rank == 0:
        print(json.dumps({"ranks": world, "rows": S, "vocab": V, "ms": res, "equal_tokens": same,
                          "bytes_exchanged_per_rank": {"logits gathered": S * Vs * 2 * (world - 1), "per-shard candidates": S * W * 8 * (world - 1)}}),
              flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--tokens", type=int, default=1280)
    p.add_argument("--hidden", type=int, default=4096)
    p.add_argument("--k-total", type=str, default="4096,12288", help="K of the unsharded weight(s): o_proj, down_proj")
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--chain", type=int, default=12, help="steps per timed sample (distinct weights)")
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--peak-tflops", type=float, default=0.0, help="bf16 GEMM peak (default: MEASURED_PEAKS.json or 1590)")
    p.add_argument("--link-gbs", type=float, default=770.0, help="NVLink bandwidth per direction per GPU")
    p.add_argument("--modes", type=str, default="nvls,pull", help="fused variants to time (nvls, pull, push)")
    p.add_argument("--sampling", action="store_true",
                   help="instead: time sampling 256 rows over a vocabulary of 151936 sharded over the ranks (top-k 50, top-p 0.9), with "
                        "the logits gathered on every rank against per-shard candidates exchanged")
    a = p.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    from .. import ops
    from ..ops import cuda_ops
    from .comm import Comm, ParallelConfig
    from .fused_tp import FusedTP

    peak = a.peak_tflops
    if peak <= 0:
        peak = 1590.0
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
        if os.path.exists(path):
            with open(path) as f:
                peak = float(json.load(f).get("bf16_tflops", peak))
    comm = Comm(ParallelConfig(world_size=world, rank=rank))
    comm.tp_group = dist.group.WORLD
    if a.sampling:
        return bench_sampling(a, comm, dev, rank, world)
    T, H = a.tokens, a.hidden
    fused = {m: FusedTP(comm, H, T + 16, dev, timeout_s=0.2, mode=m) for m in a.modes.split(",") if m}
    fused = {f.mode: f for f in fused.values()}          # a mode that is unavailable falls back to "pull"
    g = torch.Generator(device=dev).manual_seed(1)
    norm_w = torch.ones(H, dtype=torch.bfloat16, device=dev)
    rows_out = []
    for k_total in (int(v) for v in a.k_total.split(",")):
        K = k_total // world
        x = torch.randn(T, K, device=dev, generator=g).to(torch.bfloat16)
        # a chain of steps with distinct weights (together larger than L2), as consecutive layers of a model
        # present them; one timed sample is the whole chain, so that start-up skew between ranks is amortised
        n_chain = max(a.chain, (160 << 20) // (H * K * 2) + 1)
        ws = [(torch.randn(H, K, device=dev, generator=g) * 0.02).to(torch.bfloat16) for _ in range(n_chain)]
        res_full = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        dist.broadcast(res_full, 0)

        def run_nccl(w):
            y = ops.linear(x, w)
            dist.all_reduce(y)
            return ops.add_rms_norm(y, res_full, norm_w, 1e-6)

        def make_fused(f):
            res_shard = f.init_residual(res_full)
            return lambda w: f.row_linear_add_rms_norm(x, w, res_shard, norm_w, 1e-6)

        impls = {f"fused-{m}": make_fused(f) for m, f in fused.items()}
        impls["nccl"] = run_nccl
        # agreement with the NCCL path (same roundings by construction)
        want, _ = run_nccl(ws[0])
        for name in [n for n in impls if n != "nccl"]:
            got, _ = impls[name](ws[0])
            torch.cuda.synchronize()
            err = (got.float() - want.float()).abs().max().item()
            assert err <= 0.05 * want.float().abs().max().item() + 1e-3, (name, err)
        res = {}
        for name, fn in impls.items():
            for _ in range(a.warmup):
                fn(ws[0])
            torch.cuda.synchronize()
            dist.barrier()
            # the chain is replayed from a CUDA graph, as the serving engine runs its steps: host launch cost is out
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.graph(graph, stream=side):
                for w in ws:
                    fn(w)
            torch.cuda.synchronize()
            dist.barrier()
            times = []
            for _ in range(a.iters):
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                graph.replay()
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1) / len(ws))
            del graph
            t = torch.tensor(sorted(times)[len(times) // 2], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res[name] = float(t.item())
        flops = 2.0 * T * H * K
        t_compute = flops / (peak * 1e12) * 1e3
        # per GPU and direction: the reduce-scatter brings in (n-1)/n of the result from the peers' partials and the
        # all-gather brings in the (n-1)/n of the normalised rows that other ranks own (and sends as much)
        link_bytes = 2 * (world - 1) / world * T * H * 2
        t_link = link_bytes / (a.link_gbs * 1e9) * 1e3
        roof = max(t_compute, t_link)
        t_link_nvls = T * H * 2 / (a.link_gbs * 1e9) * 1e3
        roof_nvls = max(t_compute, t_link_nvls)
        row = {"tokens": T, "hidden": H, "k_per_rank": K, "ranks": world, "ms": res, "roofline_ms": roof,
               "roofline_compute_ms": t_compute, "roofline_link_ms": t_link, "roofline_link_nvls_ms": t_link_nvls,
               "fraction_of_roofline": {k: (roof_nvls if k == "fused-nvls" else roof) / v for k, v in res.items()},
               "status": cuda_ops.read_status()}
        rows_out.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
