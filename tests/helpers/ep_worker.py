"""Rank program of the expert-parallel kernel test (launched with torch.distributed.run on 2, 4 or 8 GPUs).

Every rank holds E / R experts of one MoE layer and its own tokens (a different number on every rank, one rank possibly
none).  The fused dispatch -> grouped GEMMs -> return -> combine path must give, for the tokens of each rank, what the
plain PyTorch statement of the layer gives with ALL experts (every rank builds the whole weight set from the same seed).
Checked for bf16 rows and for rows quantised to e4m3 on the way (block-scaled fp8 experts), several layers in a row
(the flags are epoch-valued) and with the calls replayed from a CUDA graph.
    argv: <out.json>
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from xllm_wxh_b200.ops import cuda_ops, moe_cuda  # noqa: E402
from xllm_wxh_b200.ops import reference as ref  # noqa: E402
from xllm_wxh_b200.parallel.comm import Comm, ParallelConfig  # noqa: E402
from xllm_wxh_b200.parallel.fused_ep import FusedEP  # noqa: E402


class _Mlp:
    pass


def main():
    out = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    comm = Comm(ParallelConfig(world_size=world, rank=rank, dp_size=world, ep_size=world))
    H, I, E, k = 512, 256, 4 * world, 4
    El = E // world
    g = torch.Generator(device=dev).manual_seed(7)                      # same weights on every rank
    w13_all = (torch.randn(E, 2 * I, H, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    w2_all = (torch.randn(E, H, I, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    report = {"rank": rank, "cases": []}
    T_cap = 300
    for fp8 in (False, True):
        mlp = _Mlp()
        mlp.interleaved = False
        if fp8:
            qs = [ref.quant_weight_128x128(w13_all[e]) for e in range(E)]
            q2 = [ref.quant_weight_128x128(w2_all[e]) for e in range(E)]
            w13_q, w13_s = torch.stack([q[0] for q in qs]), torch.stack([q[1] for q in qs])
            w2_q, w2_s = torch.stack([q[0] for q in q2]), torch.stack([q[1] for q in q2])
            sl = slice(rank * El, (rank + 1) * El)
            mlp.w13, mlp.w13_scale, mlp.w2, mlp.w2_scale = (w13_q[sl].contiguous(), w13_s[sl].contiguous(), w2_q[sl].contiguous(),
                                                             w2_s[sl].contiguous())
            w13_ref = torch.stack([ref.dequant_weight_128x128(w13_q[e], w13_s[e]) for e in range(E)]).to(torch.bfloat16)
            w2_ref = torch.stack([ref.dequant_weight_128x128(w2_q[e], w2_s[e]) for e in range(E)]).to(torch.bfloat16)
        else:
            sl = slice(rank * El, (rank + 1) * El)
            mlp.w13 = moe_cuda.interleave_w13(w13_all[sl].clone())
            mlp.w2 = w2_all[sl].contiguous()
            mlp.interleaved = True
            mlp.w13_scale = mlp.w2_scale = None
            w13_ref, w2_ref = w13_all, w2_all
        ep = FusedEP(comm, H, E, k, T_cap, dev, timeout_s=1.0, fp8=fp8)
        for layer, T in enumerate([200 - 37 * rank, 0 if rank == 1 else 64, 300]):
            gl = torch.Generator(device=dev).manual_seed(100 * layer + rank)
            h = torch.randn(T, H, device=dev, generator=gl).to(torch.bfloat16)
            logits = torch.randn(T, E, device=dev, generator=gl)
            if layer == 2:
                logits[:, :2] += 4.0                                      # a skewed router: two hot experts
            w, ids = ref.moe_router(logits, k)
            ids = ids.int()
            add = torch.randn(T, H, device=dev, generator=gl).to(torch.bfloat16) if layer == 1 else None
            counts = [0] * world
            tt = torch.tensor([T], device=dev)
            allT = [torch.zeros_like(tt) for _ in range(world)]
            dist.all_gather(allT, tt)
            ep.dp_token_counts = [int(x.item()) for x in allT]
            got = ep(h, mlp, w, ids, layer, add=add)
            torch.cuda.synchronize()
            if fp8:
                want = ref.moe_experts_fp8(h, w13_ref, w2_ref, w, ids, 0)
            else:
                want = ref.moe_experts(h, w13_ref, w2_ref, w, ids, 0)
            if add is not None:
                want = (want.float() + add.float()).to(want.dtype)
            err = float((got.float() - want.float()).abs().max()) if T else 0.0
            scale = float(want.float().abs().max()) if T else 1.0
            report["cases"].append({"fp8": fp8, "layer": layer, "T": T, "err": err, "scale": scale,
                                    "rows": int(ep.table.total_rows.item()), "tiles": int(ep.table.num_m_tiles.item())})
        # the same exchange replayed from a CUDA graph (flags are epoch-valued, nothing is reset by the host)
        T = 128
        gl = torch.Generator(device=dev).manual_seed(999 + rank)
        h = torch.randn(T, H, device=dev, generator=gl).to(torch.bfloat16)
        w, ids = ref.moe_router(torch.randn(T, E, device=dev, generator=gl), k)
        ids = ids.int().contiguous()
        ep.dp_token_counts = [T] * world
        eager = ep(h, mlp, w, ids, 0).clone()
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.graph(graph, stream=side):
            y = ep(h, mlp, w, ids, 0)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        report["cases"].append({"fp8": fp8, "layer": "graph", "T": T, "err": float((y.float() - eager.float()).abs().max()),
                                "scale": float(eager.float().abs().max()), "rows": int(ep.table.total_rows.item()), "tiles": 0})
        dist.barrier()
    report["status"] = cuda_ops.read_status()
    gathered = [None] * world
    dist.all_gather_object(gathered, report)
    if rank == 0:
        with open(out, "w") as f:
            json.dump(gathered, f)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
