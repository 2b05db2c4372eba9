"""Bandwidth of the paged-KV block transfer between two GPUs of one node (prefill / decode disaggregation):

    python -m xllm_wxh_b200.parallel.bench_kv_transfer [--layers 36] [--kv-heads 8] [--head-dim 128] [--block-size 16]
                                                       [--tokens 1024,4096,16384]

One process, source cache on cuda:0, destination cache on cuda:1 (peer access).  For each prompt length the blocks of the
prompt (scattered block ids on both sides) are moved three ways, timed with CUDA events on the launching GPU (median of
`--iters`, after warm-up; every sample moves other blocks, and the caches are far larger than L2):
  push whole  : one launch of the push kernel over all cache tensors, issued by the source GPU (peer stores)
  push layers : one launch per layer (what a prefill step does under its forward pass)
  pull whole  : the same kernel issued by the destination GPU (peer loads), as the PULL mode does
against the measured 770 GB/s per direction of a peer copy."""
from __future__ import annotations

import argparse
import json
import sys

import torch


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--layers", type=int, default=36)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--block-size", type=int, default=16)
    p.add_argument("--tokens", type=str, default="1024,4096,16384")
    p.add_argument("--iters", type=int, default=6)
    p.add_argument("--link-gbs", type=float, default=770.0)
    a = p.parse_args()
    if torch.cuda.device_count() < 2:
        print(json.dumps({"unavailable": "needs two GPUs"}))
        return 0
    from ..ops import cuda_ops
    from .kv_transfer import NvlinkPushTransfer, local_peer_handles
    d0, d1 = torch.device("cuda:0"), torch.device("cuda:1")
    lens = [int(v) for v in a.tokens.split(",")]
    n_blocks = max(lens) // a.block_size * (a.iters + 4) + 8
    shape = (n_blocks, a.block_size, a.kv_heads, a.head_dim)

    def caches(dev):
        return [(torch.randn(shape, device=dev, dtype=torch.bfloat16), torch.randn(shape, device=dev, dtype=torch.bfloat16))
                for _ in range(a.layers)]
    src, dst = caches(d0), caches(d1)
    torch.cuda.synchronize(d0); torch.cuda.synchronize(d1)
    # peer access is switched on by the first copy between the two devices
    src[0][0][:1].copy_(dst[0][0][:1]); dst[0][0][:1].copy_(src[0][0][:1])
    torch.cuda.synchronize(d0); torch.cuda.synchronize(d1)
    torch.cuda.set_device(d0)
    push = NvlinkPushTransfer(src, local_peer_handles(dst), d0)
    torch.cuda.set_device(d1)
    pull = NvlinkPushTransfer(dst, local_peer_handles(src), d1, pull=True)
    block_bytes = 2 * a.layers * a.block_size * a.kv_heads * a.head_dim * 2
    g = torch.Generator().manual_seed(0)
    rows = []
    for T in lens:
        nb = T // a.block_size
        perm_s, perm_d = torch.randperm(n_blocks, generator=g).tolist(), torch.randperm(n_blocks, generator=g).tolist()

        def pairs_of(i):
            return [(perm_s[(i * nb + j) % n_blocks], perm_d[(i * nb + j) % n_blocks]) for j in range(nb)]

        def timed(dev, fn):
            torch.cuda.set_device(dev)
            ts = []
            for i in range(a.iters + 2):
                ps = pairs_of(i)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize(dev)
                e0.record()
                fn(ps)
                e1.record()
                torch.cuda.synchronize(dev)
                if i >= 2:
                    ts.append(e0.elapsed_time(e1))
            return sorted(ts)[len(ts) // 2]

        def push_layers(ps):
            for layer in range(a.layers):
                push.push(ps, layer)
        ms = {"push whole": timed(d0, lambda ps: push.push(ps)), "push layers": timed(d0, push_layers),
              "pull whole": timed(d1, lambda ps: pull.push(ps))}
        byts = nb * block_bytes
        # one block moved both ways must arrive intact
        ps = pairs_of(0)
        torch.cuda.set_device(d0)
        push.push(ps)
        torch.cuda.synchronize(d0)
        ok = bool(torch.equal(src[3][1][ps[0][0]].cpu(), dst[3][1][ps[0][1]].cpu()))
        row = {"tokens": T, "blocks": nb, "bytes": byts, "ms": ms, "gbs": {k: byts / v / 1e6 for k, v in ms.items()},
               "fraction_of_link": {k: byts / v / 1e6 / a.link_gbs for k, v in ms.items()}, "copied_block_matches": ok,
               "status": cuda_ops.read_status()}
        rows.append(row)
        print(json.dumps(row), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
