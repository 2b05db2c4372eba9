"""Microbenchmark of one expert-parallel MoE layer (attention data-parallel: every rank brings its own tokens) on N ranks
of one node, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29535 \
        -m xllm_wxh_b200.parallel.bench_ep [--tokens 640] [--hidden 2048] [--inter 768] [--experts 128] [--top-k 8] [--fp8]

Timed on every rank with CUDA events around a CUDA-graph replay of a chain of layers (distinct expert weights, larger than
L2 together); the median per-layer time is reduced with MAX over ranks:
  fused      : dispatch kernel (count exchange, expert-major placement, peer stores, arrival wait), the two grouped GEMMs
               on the received rows, return kernel (peer stores into the source's slots), combine (wait + weighted sum)
  fused-fp8  : the same with rows quantised to e4m3 + 1x128 scales on the way out and block-scaled fp8 expert weights
  gather     : all-gather of every rank's tokens and routes (NCCL), local experts on all tokens, all-reduce (NCCL), slice -
               what the reference does without its all-to-all layer (dp_utils.cpp:109-205)
  exchange   : the fused path's dispatch, return and combine with no expert math in between (held against the link time)
Roofline of the layer: the slowest of the expert FLOPs at the measured cuBLAS bf16 peak, of the bytes each GPU must send
(and receive) over NVLink at the measured per-direction peer bandwidth (T k (N-1)/N rows out and as many back), and of
one read of this rank's expert weights from HBM at the measured copy bandwidth (what bounds the layer at these sizes).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import types

import torch
import torch.distributed as dist


def _time_graph(fn, n_chain, iters, warmup, dev):
    for _ in range(warmup):
        fn(0)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.graph(graph, stream=side):
        for i in range(n_chain):
            fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    times = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / n_chain)
    del graph
    t = torch.tensor(sorted(times)[len(times) // 2], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--tokens", type=int, default=640, help="tokens per rank and step")
    p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--inter", type=int, default=768)
    p.add_argument("--experts", type=int, default=128)
    p.add_argument("--top-k", type=int, default=8)
    p.add_argument("--fp8", action="store_true", help="also time the fp8 exchange with block-scaled fp8 experts")
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--chain", type=int, default=0, help="layers per timed sample (0: enough weights to exceed L2)")
    p.add_argument("--peak-tflops", type=float, default=0.0)
    p.add_argument("--link-gbs", type=float, default=770.0)
    p.add_argument("--hbm-gbs", type=float, default=0.0, help="copy bandwidth (default: MEASURED_PEAKS.json or 6650)")
    a = p.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    from .. import ops
    from ..ops import cuda_ops, reference as ref
    from .comm import Comm, ParallelConfig
    from .fused_ep import FusedEP, GatherEP

    peak = a.peak_tflops
    if peak <= 0:
        peak = 1590.0
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
        if os.path.exists(path):
            with open(path) as f:
                peak = float(json.load(f).get("bf16_tflops", peak))
    if a.hbm_gbs <= 0:
        a.hbm_gbs = 6650.0
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
        if os.path.exists(path):
            with open(path) as f:
                a.hbm_gbs = float(json.load(f).get("hbm_gbs", a.hbm_gbs))
    comm = Comm(ParallelConfig(world_size=world, rank=rank, dp_size=world, ep_size=world))
    comm.ep_group = comm.world_group = comm.dp_group = dist.group.WORLD
    T, H, I, E, k = a.tokens, a.hidden, a.inter, a.experts, a.top_k
    El = E // world
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    n_chain = a.chain or max(4, (160 << 20) // (El * 3 * I * H * 2) + 1)
    layers = []
    for _ in range(n_chain):
        m = types.SimpleNamespace(interleaved=False, w13_scale=None, w2_scale=None)
        m.w13 = (torch.randn(El, 2 * I, H, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        m.w2 = (torch.randn(El, H, I, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        layers.append(m)
    h = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, device=dev, generator=g)
    w, ids = ops.moe_router(logits.to(torch.bfloat16), k, "softmax", True)
    ids = ids.contiguous()
    counts = [T] * world

    fused = FusedEP(comm, H, E, k, T + 16, dev, timeout_s=0.5)
    fused.dp_token_counts = counts
    gather = GatherEP(comm, rank * El)
    gather.dp_token_counts = counts
    impls = {"fused": lambda i: fused(h, layers[i], w, ids, i), "gather": lambda i: gather(h, layers[i], w, ids, i)}

    y_dummy = torch.zeros((fused._rows_bound(), H), dtype=torch.bfloat16, device=dev)
    out_dummy = torch.empty((T, H), dtype=torch.bfloat16, device=dev)

    def round_trip_without_experts(i):
        # dispatch + return + combine with no expert math in between: the exchange itself
        import ctypes
        from ..ops.cuda_ops import _check, _ptr, _stream, c_int, lib
        fused.dispatch(h, ids)
        _check(lib().xl_ep_return(ctypes.byref(fused.args), _ptr(y_dummy), c_int(y_dummy.stride(0)), c_int(y_dummy.shape[0]), _stream()),
               "xl_ep_return")
        _check(lib().xl_ep_combine(ctypes.byref(fused.args), _ptr(ids), _ptr(w.contiguous()), _ptr(None), _ptr(out_dummy), c_int(T), c_int(k),
                                   _stream()), "xl_ep_combine")
    impls["exchange only (dispatch + return + combine)"] = round_trip_without_experts

    if a.fp8:
        fused8 = FusedEP(comm, H, E, k, T + 16, dev, timeout_s=0.5, fp8=True)
        fused8.dp_token_counts = counts
        layers8 = []
        for m in layers:
            q = types.SimpleNamespace(interleaved=False)
            w13q, w13s = zip(*(ref.quant_weight_128x128(m.w13[e]) for e in range(El)))
            w2q, w2s = zip(*(ref.quant_weight_128x128(m.w2[e]) for e in range(El)))
            q.w13, q.w13_scale, q.w2, q.w2_scale = torch.stack(w13q), torch.stack(w13s), torch.stack(w2q), torch.stack(w2s)
            layers8.append(q)
        impls["fused-fp8"] = lambda i: fused8(h, layers8[i], w, ids, i)

    # agreement of the fused exchange with the gather path
    want = gather(h, layers[0], w, ids, 0).float()
    got = fused(h, layers[0], w, ids, 0).float()
    torch.cuda.synchronize()
    err = (got - want).abs().max().item()
    assert err <= 0.03 * want.abs().max().item() + 1e-3, ("fused vs gather", err)
    res = {name: _time_graph(fn, n_chain, a.iters, a.warmup, dev) for name, fn in impls.items()}
    flops = 2.0 * (T * k) * 3 * I * H           # rows this rank's experts see on average = T k (uniform routing)
    t_compute = flops / (peak * 1e12) * 1e3
    link_bytes = 2.0 * T * k * (world - 1) / world * H * 2       # out with the dispatch, back with the return
    t_link = link_bytes / (a.link_gbs * 1e9) * 1e3
    weight_ms = El * 3 * I * H * 2 / (a.hbm_gbs * 1e9) * 1e3     # the local expert weights (bf16) read once from HBM
    roof = max(t_compute, t_link, weight_ms)
    roof8 = max(t_compute / 2, t_link * (1 + 4.0 / 128) * 0.75, weight_ms / 2)   # e4m3 rows + scales out, bf16 rows back
    roofs = {n: (roof8 if n == "fused-fp8" else t_link if n.startswith("exchange") else roof) for n in res}
    row = {"ranks": world, "tokens_per_rank": T, "hidden": H, "inter": I, "experts": E, "top_k": k, "layers_per_sample": n_chain,
           "ms": res, "roofline_ms": roofs, "roofline_compute_ms": t_compute, "roofline_link_ms": t_link,
           "weights_read_once_ms": weight_ms, "fraction_of_roofline": {n: roofs[n] / v for n, v in res.items()},
           "status": cuda_ops.read_status()}
    if rank == 0:
        print(json.dumps(row), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
