"""Kernel micro-benchmarks (CUDA-event timed, L2 flushed between iterations) for the shapes of the serving
configurations.  The counterpart of the reference's `xllm/core/kernels/cuda/benchmarks` tool.

    python -m xllm_wxh_b200.ops.bench_kernels gemm [--bn 0] [--json out.json]
    python -m xllm_wxh_b200.ops.bench_kernels attn
    python -m xllm_wxh_b200.ops.bench_kernels gemm-layer | prefill-split | decode-split     (kernel time by CUDA-graph replay)
"""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np
import torch

from . import cuda_ops as c
from . import reference as ref


def _flush_buf():
    return torch.empty(256 << 20, dtype=torch.uint8, device="cuda")


def time_op(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    return float(np.median(ts)), float(min(ts))


GEMM_SHAPES = [  # (M, N, K, what)
    (1280, 3072, 4096, "qkv, TP2 shard"), (1280, 4096, 2048, "o_proj, TP2 shard"), (1280, 12288, 4096, "gate_up, TP2 shard"),
    (1280, 4096, 6144, "down, TP2 shard"), (1280, 768, 4096, "qkv, TP8 shard"), (1280, 4096, 512, "o_proj, TP8 shard"),
    (1280, 3072, 4096, "gate_up, TP8 shard"), (1280, 4096, 1536, "down, TP8 shard"),
    (1280, 6144, 4096, "qwen3-8b qkv, mixed step"), (1280, 4096, 4096, "qwen3-8b o_proj"),
    (1280, 24576, 4096, "qwen3-8b gate_up"), (1280, 4096, 12288, "qwen3-8b down"),
    (256, 6144, 4096, "qwen3-8b qkv, decode"), (256, 4096, 4096, "o_proj decode"), (256, 24576, 4096, "gate_up decode"),
    (256, 4096, 12288, "down decode"), (256, 151936, 4096, "lm_head"), (4096, 4096, 4096, "square 4k"),
    (8192, 8192, 8192, "square 8k"), (10240, 24576, 4096, "gate_up, full prefill batch"),
]


def bench_gemm(bn=0, shapes=None):
    flush = _flush_buf()
    rows = []
    for M, N, K, what in shapes or GEMM_SHAPES:
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        c.gemm_force_bn(bn)
        c.gemm_set_mode(1)
        single, _ = time_op(lambda: c.linear(x, w, out=out), flush=flush)
        c.gemm_set_mode(2)
        pair, _ = time_op(lambda: c.linear(x, w, out=out), flush=flush)
        c.gemm_set_mode(0)
        ours, ours_min = time_op(lambda: c.linear(x, w, out=out), flush=flush)
        c.gemm_force_bn(0)
        lib, lib_min = time_op(lambda: torch.matmul(x, w.t(), out=out), flush=flush)
        fl = 2.0 * M * N * K
        rows.append(dict(M=M, N=N, K=K, what=what, ours_ms=ours, ours_tflops=fl / ours / 1e9, cublas_ms=lib,
                         cublas_tflops=fl / lib / 1e9, ratio=lib / ours))
        print(f"{what:32s} M={M:6d} N={N:6d} K={K:6d}  ours {ours:8.3f} ms {fl / ours / 1e9:7.1f} TF (1-CTA {single:.3f}, "
              f"pair {pair:.3f}) | cuBLAS {lib:8.3f} ms {fl / lib / 1e9:7.1f} TF | x{lib / ours:.2f}", flush=True)
    return rows


def bench_attn(decode_only=False, prefill_only=False):
    from ..framework.step_input import StepInput, make_layout
    flush = _flush_buf()
    rows = []
    cases = [(256, 1152, 32, 8)] if decode_only else [(256, 1152, 32, 8), (256, 4096, 32, 8), (64, 8192, 32, 8),
                                                       (8, 32768, 32, 8), (256, 1152, 64, 8)]
    if prefill_only:
        cases = []
    for B, kv, nq, nkv in cases:
        D, bs = 128, 16
        nb = (kv + bs - 1) // bs
        L = make_layout(B, B, nb, B, 32)
        host = torch.zeros(L.total_words, dtype=torch.int32)
        host[L.q_cu:L.q_cu + B + 1] = torch.arange(B + 1, dtype=torch.int32)
        host[L.kv_lens:L.kv_lens + B] = kv
        bt = (torch.randperm(B * nb) + 1).int().view(B, nb)
        host[L.block_tables:L.block_tables + B * L.MB_cap] = torch.nn.functional.pad(bt, (0, L.MB_cap - nb)).reshape(-1)
        hdr = np.zeros(32, dtype=np.int32)
        hdr[0], hdr[1], hdr[3], hdr[5], hdr[6], hdr[17] = B, B, B, 1, kv, bs
        inp = StepInput(host.cuda(), L, hdr)
        q = torch.randn(B, nq, D, device="cuda").to(torch.bfloat16)
        kc = torch.randn(B * nb + 1, bs, nkv, D, device="cuda").to(torch.bfloat16)
        vc = torch.randn(B * nb + 1, bs, nkv, D, device="cuda").to(torch.bfloat16)
        ms, _ = time_op(lambda: c.paged_attention(q, kc, vc, inp, D ** -0.5), flush=flush)
        byts = 2.0 * B * kv * nkv * D * 2
        rows.append(dict(B=B, kv=kv, nq=nq, nkv=nkv, ms=ms, gbs=byts / ms / 1e6))
        print(f"decode attn B={B:4d} kv={kv:6d} Hq={nq} Hkv={nkv}: {ms:8.3f} ms  {byts / ms / 1e6:8.1f} GB/s", flush=True)
    # prefill
    for T, nq, nkv in ([] if decode_only else [(1024, 32, 8), (1024, 32, 4), (1024, 16, 4), (1024, 8, 2), (1024, 4, 1), (256, 32, 8),
                                               (4096, 32, 8), (4096, 4, 1), (8192, 32, 8)]):
        D, bs = 128, 16
        nb = (T + bs - 1) // bs
        L = make_layout(T, 1, nb, 1, 32)
        host = torch.zeros(L.total_words, dtype=torch.int32)
        host[L.q_cu + 1] = T
        host[L.kv_lens] = T
        host[L.block_tables:L.block_tables + nb] = torch.arange(1, nb + 1, dtype=torch.int32)
        hdr = np.zeros(32, dtype=np.int32)
        hdr[0], hdr[1], hdr[4], hdr[5], hdr[6], hdr[17], hdr[21] = T, 1, 1, T, T, bs, T
        inp = StepInput(host.cuda(), L, hdr)
        q = torch.randn(T, nq, D, device="cuda").to(torch.bfloat16)
        kc = torch.randn(nb + 1, bs, nkv, D, device="cuda").to(torch.bfloat16)
        vc = torch.randn(nb + 1, bs, nkv, D, device="cuda").to(torch.bfloat16)
        fl = 4.0 * T * T / 2 * nq * D
        for name, tc in (("tcgen05", True), ("tc-nosplit", True), ("mma.sync", False)):
            c.prefill_use_tc(tc)
            c.prefill_kv_split(0 if name == "tc-nosplit" else 1)       # automatic key-range split against none
            ms, _ = time_op(lambda: c.paged_attention(q, kc, vc, inp, D ** -0.5), flush=flush)
            rows.append(dict(T=T, nq=nq, kernel=name, ms=ms, tflops=fl / ms / 1e9))
            print(f"prefill attn T={T:6d} Hq={nq} Hkv={nkv} [{name:10s}]: {ms:8.3f} ms  {fl / ms / 1e9:7.1f} TFLOP/s (causal)", flush=True)
        c.prefill_use_tc(True)
        c.prefill_kv_split(1)
    return rows


# ----------------------------------------------------------------------------- kernel time by graph replay
def time_graph(fns, reps=5):
    """Microseconds per call of `fns` (a list of closures, one launch sequence each) when they are replayed from one CUDA
    graph: kernel time without the host's launch overhead, which for 10-40 us kernels is as large as the kernel."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        fns[0]()
        with torch.cuda.graph(g, stream=s):
            for f in fns:
                f()
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) / len(fns))
    return best * 1e3


def bench_gemm_layer(M=1279, sustained_tflops=1383.0):
    """The four GEMMs of a Qwen3-8B layer for the whole model and its TP shards, against cuBLAS, weights rotated through
    more memory than L2 holds."""
    H, I, QKV, O = 4096, 12288, 6144, 4096
    rows = []
    for tp in (8, 4, 2, 1):
        shapes = [("qkv", QKV // tp, H, False), ("o_proj", H, O // tp, False), ("gate_up", 2 * I // tp, H, True), ("down", H, I // tp, False)]
        tot = [0.0, 0.0, 0.0]
        line = []
        for name, N, K, swiglu in shapes:
            nw = min(24, max(2, int(200e6 // (N * K * 2)) + 1))
            ws = [torch.randn(N, K, device="cuda").to(torch.bfloat16) * 0.02 for _ in range(nw)]
            x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
            if swiglu:
                wi = [c.interleave_gate_up(w) for w in ws]
                ours = time_graph([(lambda w=w: c.linear_swiglu(x, w)) for w in wi])
            else:
                ours = time_graph([(lambda w=w: c.linear(x, w)) for w in ws])
            cub = time_graph([(lambda w=w: torch.matmul(x, w.t())) for w in ws])
            ideal = 2.0 * M * N * K / (sustained_tflops * 1e12) * 1e6
            tot[0] += ours
            tot[1] += cub
            tot[2] += ideal
            rows.append(dict(tp=tp, name=name, N=N, K=K, ours_us=ours, cublas_us=cub, at_sustained_peak_us=ideal))
            line.append(f"{name} [{N}x{K}] ours {ours:.1f} cuBLAS {cub:.1f} (at sustained peak {ideal:.1f})")
        print(f"TP{tp}: " + "; ".join(line) + f" | layer: ours {tot[0]:.1f} us, cuBLAS {tot[1]:.1f}, at sustained peak {tot[2]:.1f}", flush=True)
    return rows


def _one_seq_input(T, kv, bs=16):
    from ..framework.step_input import StepInput, make_layout
    nb = (kv + bs - 1) // bs
    L = make_layout(T, 1, nb, 1, 32)
    host = torch.zeros(L.total_words, dtype=torch.int32)
    host[L.q_cu + 1] = T
    host[L.kv_lens] = kv
    host[L.block_tables:L.block_tables + nb] = torch.arange(1, nb + 1, dtype=torch.int32)
    hdr = np.zeros(32, dtype=np.int32)
    hdr[0], hdr[1], hdr[4], hdr[5], hdr[6], hdr[17], hdr[21] = T, 1, 1, T, kv, bs, T
    return StepInput(host.cuda(), L, hdr), nb


def bench_prefill_split():
    """tcgen05 prefill attention with and without the split of the key range."""
    rows = []
    for T, nq, nkv, kv in [(1024, 32, 8, 1024), (1024, 4, 1, 1024), (256, 4, 1, 256), (1024, 4, 1, 8192), (4096, 4, 1, 4096),
                           (128, 32, 8, 4096)]:
        inp, nb = _one_seq_input(T, kv)
        q = torch.randn(T, nq, 128, device="cuda").to(torch.bfloat16)
        kc = torch.randn(nb + 1, 16, nkv, 128, device="cuda").to(torch.bfloat16)
        vc = torch.randn(nb + 1, 16, nkv, 128, device="cuda").to(torch.bfloat16)
        us = []
        for mode in (0, 1, 2, 4, 8):
            c.prefill_kv_split(mode)
            us.append(time_graph([lambda: c.paged_attention(q, kc, vc, inp, 128 ** -0.5)] * 20))
        c.prefill_kv_split(1)
        rows.append(dict(T=T, kv=kv, nq=nq, nkv=nkv, us=us))
        print(f"prefill T={T} kv={kv} Hq={nq} Hkv={nkv}: no split {us[0]:.1f} us, auto {us[1]:.1f}, x2 {us[2]:.1f}, x4 {us[3]:.1f}, "
              f"x8 {us[4]:.1f}", flush=True)
    return rows


def bench_decode_split():
    """TMA decode attention for TP-shard head counts and forced numbers of key splits."""
    from ..framework.step_input import StepInput, make_layout
    rows = []
    orig = c.decode_splits
    for B, kv, nq, nkv in [(255, 1150, 4, 1), (255, 1150, 8, 2), (255, 1150, 32, 8), (64, 4000, 4, 1), (16, 8000, 4, 1)]:
        bs = 16
        nbs = (kv + bs - 1) // bs
        L = make_layout(B, B, nbs, B, 32)
        host = torch.zeros(L.total_words, dtype=torch.int32)
        host[L.q_cu:L.q_cu + B + 1] = torch.arange(B + 1, dtype=torch.int32)
        lens = torch.full((B,), kv, dtype=torch.int32) - torch.randint(0, 64, (B,), dtype=torch.int32)
        host[L.kv_lens:L.kv_lens + B] = lens
        bt = torch.zeros(B, L.MB_cap, dtype=torch.int32)
        bt[:, :nbs] = (torch.randperm(B * nbs, dtype=torch.int32) + 1).view(B, nbs)
        host[L.block_tables:L.block_tables + B * L.MB_cap] = bt.reshape(-1)
        hdr = np.zeros(32, dtype=np.int32)
        hdr[0], hdr[1], hdr[3], hdr[5], hdr[6], hdr[17] = B, B, B, 1, kv, bs
        inp = StepInput(host.cuda(), L, hdr)
        q = torch.randn(B, nq, 128, device="cuda").to(torch.bfloat16)
        kc = torch.randn(B * nbs + 1, bs, nkv, 128, device="cuda").to(torch.bfloat16)
        vc = torch.randn(B * nbs + 1, bs, nkv, 128, device="cuda").to(torch.bfloat16)
        byts = float(lens.sum()) * 2 * nkv * 128 * 2
        res = []
        for sp in (None, 1, 2, 4, 8):
            c.decode_splits = orig if sp is None else (lambda a, b, m, sp=sp: sp)
            us = time_graph([lambda: c.paged_attention(q, kc, vc, inp, 128 ** -0.5)] * 10)
            res.append((sp, us))
        c.decode_splits = orig
        rows.append(dict(B=B, kv=kv, nq=nq, nkv=nkv, us=res))
        print(f"decode B={B} kv={kv} Hq={nq} Hkv={nkv}: " + ", ".join(
            f"{'auto(' + str(orig(B, nkv, kv)) + ')' if sp is None else 'x' + str(sp)} {us:.1f} us ({byts / us / 1e6:.2f} TB/s)"
            for sp, us in res), flush=True)
    return rows


def _mla_batch(seqs, Hh, bs=64):
    """StepInput + head-major queries + latent cache for (q_len, kv_len) pairs."""
    from ..framework.step_input import StepInput, make_layout
    B = len(seqs)
    T = sum(q for q, _ in seqs)
    nbs = [(kv + bs - 1) // bs for _, kv in seqs]
    L = make_layout(T, B, max(nbs), B, 32)
    host = torch.zeros(L.total_words, dtype=torch.int32)
    q_cu = [0]
    for q, _ in seqs:
        q_cu.append(q_cu[-1] + q)
    host[L.q_cu:L.q_cu + B + 1] = torch.tensor(q_cu, dtype=torch.int32)
    host[L.kv_lens:L.kv_lens + B] = torch.tensor([kv for _, kv in seqs], dtype=torch.int32)
    bt = torch.zeros(B, L.MB_cap, dtype=torch.int32)
    perm = torch.randperm(sum(nbs), dtype=torch.int32) + 1
    at = 0
    for i, nb in enumerate(nbs):
        bt[i, :nb] = perm[at:at + nb]
        at += nb
    host[L.block_tables:L.block_tables + B * L.MB_cap] = bt.reshape(-1)
    hdr = np.zeros(32, dtype=np.int32)
    hdr[0], hdr[1], hdr[17] = T, B, bs
    inp = StepInput(host.cuda(), L, hdr)
    q_lat = (torch.randn(Hh, T, 512, device="cuda") * 0.3).to(torch.bfloat16)
    q_pe = (torch.randn(Hh, T, 64, device="cuda") * 0.3).to(torch.bfloat16)
    cache = (torch.randn(sum(nbs) + 1, bs, 576, device="cuda") * 0.3).to(torch.bfloat16)
    return inp, q_lat, q_pe, cache


def bench_mla(cases=None, reps=10):
    """Absorbed MLA attention: the tcgen05 kernel against the mma.sync kernel.  Bytes = latent cache rows read once per
    sequence; FLOPs = 2 * rows * keys * (576 + 512)."""
    import os
    rows = []
    cases = cases or [("decode B=256 kv=1152 Hh=128", [(1, 1152)] * 256, 128), ("decode B=64 kv=4096 Hh=128", [(1, 4096)] * 64, 128),
                      ("decode B=8 kv=8192 Hh=128", [(1, 8192)] * 8, 128), ("decode B=256 kv=1152 Hh=16 (TP 8)", [(1, 1152)] * 256, 16),
                      ("verify B=128 q=2 kv=1152 Hh=128", [(2, 1152)] * 128, 128), ("prefill 1 x 1024 Hh=128", [(1024, 1024)], 128)]
    for name, seqs, Hh in cases:
        inp, q_lat, q_pe, cache = _mla_batch(seqs, Hh)
        byts = sum(kv for _, kv in seqs) * 576 * 2.0
        flops = sum(q * (kv - (q - 1) / 2.0) for q, kv in seqs) * Hh * 2.0 * (576 + 512)
        us = {}
        for kern in ("tcgen05", "tcgen05_single", "mma_sync"):
            os.environ["XLLM_MLA_TC"] = "0" if kern == "mma_sync" else "1"
            c.lib().xl_mla_pair_mode(0 if kern == "tcgen05_single" else 1)
            us[kern] = time_graph([lambda: c.mla_attention(q_lat, q_pe, cache, inp, 192 ** -0.5, 512)] * reps)
        os.environ["XLLM_MLA_TC"] = "1"
        c.lib().xl_mla_pair_mode(0)
        rows.append(dict(case=name, us=us, bytes=byts, flops=flops))
        print(f"mla {name}: tcgen05 pair {us['tcgen05']:.1f} us ({byts / us['tcgen05'] / 1e6:.2f} TB/s of cache, "
              f"{flops / us['tcgen05'] / 1e6:.0f} TFLOP/s), independent CTAs {us['tcgen05_single']:.1f} us, "
              f"mma.sync {us['mma_sync']:.1f} us  ({us['mma_sync'] / us['tcgen05']:.2f}x)", flush=True)
    return rows


def bench_sparse_mla(reps=4):
    """DeepSeek-V3.2 decode step of one layer: the lightning indexer's ranking (64 heads x 128, top 2048 of the causal keys)
    and the MLA attention over the kept slots, beside the dense MLA attention over the whole context."""
    import types
    from ..models.indexer import LightningIndexer
    rows = []
    ix_args = types.SimpleNamespace(index_n_heads=64, index_head_dim=128, qk_rope_head_dim=64, index_topk=2048,
                                    index_rope_interleave=False)
    ix = LightningIndexer(ix_args, "cuda", torch.bfloat16)
    for name, B, kv, Hh in (("decode B=64 kv=8192 Hh=128", 64, 8192, 128), ("decode B=16 kv=32768 Hh=128", 16, 32768, 128),
                            ("decode B=64 kv=8192 Hh=16 (TP 8)", 64, 8192, 16)):
        inp, q_lat, q_pe, cache = _mla_batch([(1, kv)] * B, Hh)
        inp.positions = torch.full((B,), kv - 1, dtype=torch.int32, device="cuda")
        inp.token_seq = torch.arange(B, dtype=torch.int32, device="cuda")
        inp.max_kv = kv
        idx_cache = (torch.randn(cache.shape[0], cache.shape[1], 128, device="cuda") * 0.3).to(torch.bfloat16)
        q = (torch.randn(B, 64, 128, device="cuda") * 0.3).to(torch.bfloat16)
        w = (torch.randn(B, 64, device="cuda") * 0.3).to(torch.bfloat16)
        sel, sel_len = ix.select(q, w, idx_cache, inp)
        us = dict(select=time_graph([lambda: ix.select(q, w, idx_cache, inp)] * reps),
                  sparse=time_graph([lambda: c.mla_attention_sparse(q_lat, q_pe, cache, sel, sel_len, 192 ** -0.5, 512)] * reps),
                  dense=time_graph([lambda: c.mla_attention(q_lat, q_pe, cache, inp, 192 ** -0.5, 512)] * reps))
        rows.append(dict(case=name, us=us, kept=int(sel.shape[1])))
        print(f"sparse mla {name}: ranking {us['select']:.1f} us, attention over {sel.shape[1]} kept slots {us['sparse']:.1f} us, "
              f"dense attention over all keys {us['dense']:.1f} us", flush=True)
    return rows


def bench_moe(T=1279, H=2048, I=768, E=128, k=8):
    """One MoE layer of the Qwen3-30B-A3B shape on one GPU (all experts local): sort, gather, the two grouped GEMMs,
    combine, each timed alone (L2 flushed), with the weight bytes per second of the GEMMs."""
    from . import moe_cuda as m
    flush = _flush_buf()
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device="cuda", generator=g)[:k] for _ in range(T)]).int()
    wts = torch.full((T, k), 1.0 / k, device="cuda")
    r = m.moe_sort(ids, 0, E)
    xs = m.gather_rows(x, r, k)
    h = m.grouped_gemm(xs, w13, r, swiglu=True)
    y = m.grouped_gemm(h, w2, r)
    rows = []
    for name, fn, byts, fl in (
            ("moe_sort", lambda: m.moe_sort(ids, 0, E), 0, 0),
            ("gather_rows", lambda: m.gather_rows(x, r, k), 2.0 * T * k * H * 2, 0),
            ("grouped_gemm w13 + SwiGLU", lambda: m.grouped_gemm(xs, w13, r, swiglu=True), w13.numel() * 2.0, 2.0 * T * k * 2 * I * H),
            ("grouped_gemm w2", lambda: m.grouped_gemm(h, w2, r), w2.numel() * 2.0, 2.0 * T * k * H * I),
            ("combine", lambda: m.combine(y, r, wts, T), T * k * H * 2.0, 0),
            ("whole layer (moe_experts)", lambda: m.moe_experts(x, w13, w2, wts, ids, 0, True), (w13.numel() + w2.numel()) * 2.0,
             2.0 * T * k * 3 * I * H)):
        ms, _ = time_op(fn, flush=flush)
        rows.append(dict(op=name, ms=ms, gbs=byts / ms / 1e6 if byts else None, tflops=fl / ms / 1e9 if fl else None))
        print(f"{name:28s} {ms * 1e3:8.1f} us" + (f"  {byts / ms / 1e6:8.1f} GB/s (weights or rows)" if byts else "") +
              (f"  {fl / ms / 1e9:7.1f} TFLOP/s" if fl else ""), flush=True)
    return rows

# ----------------------------------------------------------------------------- small cases of the memory-bound kernels
def bench_small(which: str):
    """One kernel on a case larger than L2 (126 MB) and far below a GB-scale footprint: sized for a single profiler
    capture.  Prints the CUDA-event time (L2 flushed between launches) and the algorithmic bytes / FLOPs it moved."""
    import types
    flush = _flush_buf()
    out = {}
    dev = "cuda"
    if which == "rope":
        T, nq, nkv, D, bs = 16384, 32, 8, 128, 16
        qkv = torch.randn(T, (nq + 2 * nkv) * D, device=dev).to(torch.bfloat16)
        pos = torch.arange(T, device=dev, dtype=torch.int32) % 4096
        slots = torch.randperm(T, device=dev).int()
        from . import reference as ref
        from ..models.args import ModelArgs
        cos_sin = ref.build_cos_sin_cache(D, 4096, 1e6, dtype=torch.float32, device=dev)
        qw, kw = torch.ones(D, device=dev, dtype=torch.bfloat16), torch.ones(D, device=dev, dtype=torch.bfloat16)
        kc = torch.zeros(T // bs, bs, nkv, D, device=dev, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        ms, _ = time_op(lambda: c.rope_qknorm_kvwrite(qkv, pos, slots, cos_sin, qw, kw, 1e-6, kc, vc, nq, nkv, D), flush=flush)
        byts = T * ((nq + 2 * nkv) * D * 2 + (nq + nkv) * D * 2 + 2 * nkv * D * 2)    # qkv read, q and k rewritten, K and V cache rows
        out = dict(kernel="rope_qknorm_kvwrite", T=T, ms=ms, gbs=byts / ms / 1e6)
    elif which == "sample":
        S, V = 512, 151936
        logits = torch.randn(S, V, device=dev).to(torch.bfloat16)
        inp = types.SimpleNamespace(any_penalty=False, any_logprobs=True, max_top_logprobs=0,
                                    temperature=torch.full((S,), 0.8, device=dev), top_k=torch.full((S,), 50, device=dev, dtype=torch.int32),
                                    top_p=torch.full((S,), 0.9, device=dev), seed_lo=torch.arange(S, device=dev, dtype=torch.int32),
                                    seed_hi=torch.zeros(S, device=dev, dtype=torch.int32))
        ms, _ = time_op(lambda: c.sample(logits, inp), flush=flush)
        out = dict(kernel="sample (temperature, top-k 50, top-p 0.9, logprob)", S=S, V=V, ms=ms, gbs=S * V * 2 / ms / 1e6)
    elif which == "router":
        T, E, k = 524288, 128, 8
        logits = torch.randn(T, E, device=dev).to(torch.bfloat16)
        ms, _ = time_op(lambda: c.moe_router(logits, k, "softmax", True), flush=flush)
        byts = T * (E * 2 + k * 8)
        out = dict(kernel="moe_router softmax top-8 of 128", T=T, ms=ms, gbs=byts / ms / 1e6)
        T2, E2 = 262144, 256
        lg2 = torch.randn(T2, E2, device=dev).to(torch.bfloat16)
        bias = torch.randn(E2, device=dev)
        ms2, _ = time_op(lambda: c.moe_router(lg2, 8, "sigmoid", True, bias, 8, 4, 2.5), flush=flush)
        print(f"moe_router sigmoid group-limited top-8 of 256: T={T2} {ms2 * 1e3:8.1f} us {T2 * (E2 * 2 + 64) / ms2 / 1e6:8.1f} GB/s", flush=True)
    elif which == "fp8":
        rows = []
        for M, N, K in [(4096, 7168, 2048), (4096, 4096, 7168), (1279, 6144, 4096), (1279, 4096, 4096), (1279, 24576, 4096),
                        (1279, 4096, 12288), (256, 24576, 4096)]:
            x = torch.randn(M, K, device=dev).to(torch.bfloat16)
            wq = (torch.randn(N, K, device=dev) * 0.5).to(torch.float8_e4m3fn)
            ws = torch.rand((N + 127) // 128, (K + 127) // 128, device=dev) * 0.02 + 0.01
            xq, xs = c.quant_act_1x128(x)
            o = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            def run():
                c._check(c.lib().xl_gemm_fp8_block(c._ptr(xq), c._ptr(wq), c._ptr(o), c._ptr(xs), c._ptr(ws), M, N, K, N, c._stream()),
                         "xl_gemm_fp8_block")
            ms, _ = time_op(run, flush=flush)
            # torch._scaled_mm: per-tensor scales (the reference's sm100 kernel computes the same contraction)
            sa, sb = torch.tensor(1.0, device=dev), torch.tensor(1.0, device=dev)
            ms_lib, _ = time_op(lambda: torch._scaled_mm(xq, wq.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16), flush=flush)
            fl = 2.0 * M * N * K
            # the per-token / per-channel kernel (whole K accumulated in TMEM) against the library with the same scaling
            xq2, xs2 = c.quant_rows_fp8(x)
            cs = torch.rand(N, device=dev) * 0.02 + 0.01
            ms_sc, _ = time_op(lambda: c.linear_fp8_scaled(xq2, xs2, wq, cs), flush=flush)
            ms_row, _ = time_op(lambda: torch._scaled_mm(xq2, wq.t(), scale_a=xs2.view(-1, 1), scale_b=cs.view(1, -1),
                                                         out_dtype=torch.bfloat16), flush=flush)
            rows.append(dict(M=M, N=N, K=K, block_ms=ms, block_tflops=fl / ms / 1e9, scaled_ms=ms_sc, scaled_tflops=fl / ms_sc / 1e9,
                             scaled_mm_tensor_ms=ms_lib, scaled_mm_rowwise_ms=ms_row))
            print(f"fp8 {M}x{N}x{K}: block-scaled {ms * 1e3:7.1f} us {fl / ms / 1e9:6.0f} TF | per-token x per-channel "
                  f"{ms_sc * 1e3:7.1f} us {fl / ms_sc / 1e9:6.0f} TF | torch._scaled_mm per-tensor {ms_lib * 1e3:7.1f} us "
                  f"{fl / ms_lib / 1e9:6.0f} TF, row-wise {ms_row * 1e3:7.1f} us {fl / ms_row / 1e9:6.0f} TF", flush=True)
        out = dict(kernel="gemm_fp8_block", rows=rows)
    if "ms" in out:
        print(f"{out['kernel']}: {out['ms'] * 1e3:8.1f} us  {out['gbs']:8.1f} GB/s (algorithmic bytes)", flush=True)
    return out


def main():
    p = argparse.ArgumentParser()
    p.add_argument("what", choices=["gemm", "attn", "decode", "prefill", "moe", "all", "gemm-layer", "prefill-split", "decode-split",
                                   "small-rope", "small-sample", "small-router", "small-fp8", "mla", "small-mla", "sparse-mla"])
    p.add_argument("--bn", type=int, default=0)
    p.add_argument("--json", type=str, default="")
    p.add_argument("--only", type=str, default="", help="gemm: a single M,N,K shape (small profiling runs)")
    a = p.parse_args()
    out = {}
    if a.what in ("gemm", "all"):
        shapes = None
        if a.only:
            M, N, K = (int(v) for v in a.only.split(","))
            shapes = [(M, N, K, "selected")]
        out["gemm"] = bench_gemm(a.bn, shapes)
    if a.what in ("attn", "all"):
        out["attn"] = bench_attn()
    if a.what == "decode":
        out["attn"] = bench_attn(decode_only=True)
    if a.what == "prefill":
        out["attn"] = bench_attn(prefill_only=True)
    if a.what == "moe":
        out["moe"] = bench_moe()
    if a.what == "gemm-layer":
        out["gemm_layer"] = bench_gemm_layer()
    if a.what == "prefill-split":
        out["prefill_split"] = bench_prefill_split()
    if a.what == "decode-split":
        out["decode_split"] = bench_decode_split()
    if a.what == "mla":
        out["mla"] = bench_mla()
    if a.what == "sparse-mla":
        out["sparse_mla"] = bench_sparse_mla()
    if a.what == "small-mla":         # one launch worth profiling: 148 sequences x 2304 keys (390 MB of cache, above L2)
        out["mla"] = bench_mla([("decode B=148 kv=2304 Hh=128", [(1, 2304)] * 148, 128)], reps=2)
    elif a.what.startswith("small-"):
        out[a.what] = bench_small(a.what[6:])
    out["status"] = c.read_status()
    if a.json:
        with open(a.json, "w") as f:
            json.dump(out, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
