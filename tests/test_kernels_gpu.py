"""Each sm_100a kernel against the plain-PyTorch fp32 statement of the same op."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from xllm_wxh_b200.framework.step_input import StepInput, make_layout
from xllm_wxh_b200.ops import reference as ref


def cuda_ops():
    from xllm_wxh_b200.ops import cuda_ops as c
    return c


def _close(a, b, rtol, atol, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = (err > tol).sum().item()
    assert bad == 0, f"{what}: {bad}/{a.numel()} beyond tolerance, max abs err {err.max().item():.4g}, ref max {b.abs().max().item():.4g}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1, 128, 128), (77, 4096, 4096), (1280, 6144, 4096), (256, 4096, 12288),
                                   (300, 1000 // 8 * 8, 520), (1024, 24576, 512)])
@pytest.mark.parametrize("bias", [False, True])
def test_gemm_bf16(M, N, K, bias):
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16)
    b = torch.randn(N, device="cuda", generator=g).to(torch.bfloat16) if bias else None
    y = c.linear(x, w, b)
    want = x.float() @ w.float().t() + (b.float() if bias else 0)
    assert c.read_status() == 0
    _close(y, want, 2e-2, 2e-2, f"gemm {M}x{N}x{K}")


@pytest.mark.parametrize("bn", [32, 48, 64, 96, 128, 144, 192, 256])
def test_gemm_tile_widths(bn):
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(bn)
    M, N, K = 333, 1536, 1024
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16)
    c.gemm_force_bn(bn)
    try:
        y = c.linear(x, w)
        assert c.read_status() == 0
    finally:
        c.gemm_force_bn(0)
    _close(y, x.float() @ w.float().t(), 2e-2, 2e-2, f"gemm bn={bn}")


@pytest.mark.parametrize("M,N,K,bn", [(256, 512, 256, 0), (1279, 3072, 1024, 0), (300, 1000, 520, 0), (129, 96, 64, 0),
                                      (512, 2048, 2048, 64), (512, 2048, 512, 160), (700, 1536, 1024, 256)])
def test_gemm_cta_pairs(M, N, K, bn):
    """The 2-CTA (`cta_group::2`) kernel forced on: plain, bias and SwiGLU epilogues, ragged edges, several tile widths."""
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16)
    b = torch.randn(N, device="cuda", generator=g).to(torch.bfloat16)
    c.gemm_set_mode(2)
    c.lib().xl_gemm_pair_force_bn(bn)
    try:
        y = c.linear(x, w)
        yb = c.linear(x, w, b)
        fused = c.linear_swiglu(x, c.interleave_gate_up(w)) if (N // 2) % 16 == 0 else None
        assert c.read_status() == 0
    finally:
        c.gemm_set_mode(0)
        c.lib().xl_gemm_pair_force_bn(0)
    want = x.float() @ w.float().t()
    _close(y, want, 2e-2, 2e-2, f"pair gemm {M}x{N}x{K}")
    _close(yb, want + b.float(), 2e-2, 2e-2, "pair gemm + bias")
    if fused is not None:
        _close(fused, ref.silu_and_mul(want), 3e-2, 3e-2, "pair gemm + swiglu")


@pytest.mark.parametrize("M,N,K", [(256, 4096, 4096), (256, 1024, 8192), (100, 512, 2048), (300, 768, 4096), (17, 1536, 2048),
                                   (64, 4096, 1024), (256, 1000, 3000)])
def test_gemm_split_k(M, N, K):
    """Few output tiles and a long K: the pair kernel cuts the K loop over several CTA pairs and sums the fp32 partials in
    a fixed order.  Plain, bias and SwiGLU epilogues; the result is bit-identical from run to run and matches the kernel
    without the split to bf16 rounding."""
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(M * 3 + N + K)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16)
    b = torch.randn(N, device="cuda", generator=g).to(torch.bfloat16)
    want = x.float() @ w.float().t()
    y1 = c.linear(x, w)
    y2 = c.linear(x, w)
    yb = c.linear(x, w, b)
    fused = c.linear_swiglu(x, c.interleave_gate_up(w)) if (N // 2) % 16 == 0 else None
    assert c.read_status() == 0
    assert torch.equal(y1, y2), "split-K result depends on timing"
    _close(y1, want, 2e-2, 2e-2, f"split-K gemm {M}x{N}x{K}")
    _close(yb, want + b.float(), 2e-2, 2e-2, "split-K gemm + bias")
    if fused is not None:
        _close(fused, ref.silu_and_mul(want), 3e-2, 3e-2, "split-K gemm + swiglu")
    c.lib().xl_gemm_pair_splitk(0)
    try:
        y0 = c.linear(x, w)
    finally:
        c.lib().xl_gemm_pair_splitk(1)
    _close(y1, y0.float(), 1e-2, 1e-2, "split-K vs unsplit")


@pytest.mark.parametrize("M,N,K", [(1279, 4096, 4096), (1279, 4096, 12288), (1279, 4096, 1536), (1279, 24576, 4096), (2048, 4352, 2048),
                                   (300, 10240, 1024)])
def test_gemm_split_tail_wave(M, N, K):
    """Large outputs whose last wave holds few tiles (80 tiles on 74 SM pairs): whole tiles first, the remaining tiles cut
    along K over all pairs.  Same requirements as the full split: bit-stable, equal to the unsplit kernel to bf16 rounding,
    every epilogue."""
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16)
    b = torch.randn(N, device="cuda", generator=g).to(torch.bfloat16)
    want = x.float() @ w.float().t()
    ys = [c.linear(x, w) for _ in range(3)]
    yb = c.linear(x, w, b)
    fused = c.linear_swiglu(x, c.interleave_gate_up(w))
    assert c.read_status() == 0
    assert torch.equal(ys[0], ys[1]) and torch.equal(ys[0], ys[2]), "result depends on timing"
    _close(ys[0], want, 2e-2, 2e-2, f"gemm with split tail {M}x{N}x{K}")
    _close(yb, want + b.float(), 2e-2, 2e-2, "gemm with split tail + bias")
    _close(fused, ref.silu_and_mul(want), 3e-2, 3e-2, "gemm with split tail + swiglu")
    c.lib().xl_gemm_pair_splitk(0)
    try:
        y0 = c.linear(x, w)
    finally:
        c.lib().xl_gemm_pair_splitk(1)
    _close(ys[0], y0.float(), 1e-2, 1e-2, "split tail vs unsplit")


def test_gemm_strided_input_and_swiglu():
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(5)
    M, K, I = 200, 512, 768
    big = torch.randn(M, K + 64, device="cuda", generator=g).to(torch.bfloat16)
    x = big[:, :K]                                    # row pitch K + 64
    w = (torch.randn(2 * I, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16)
    y = c.linear(x, w)
    _close(y, x.float() @ w.float().t(), 2e-2, 2e-2, "strided A")
    fused = c.linear_swiglu(x.contiguous(), c.interleave_gate_up(w))
    want = ref.silu_and_mul((x.float() @ w.float().t()))
    assert c.read_status() == 0
    _close(fused, want, 3e-2, 3e-2, "swiglu epilogue")


@pytest.mark.parametrize("T,H", [(1, 256), (37, 4096), (300, 8192), (5, 2048)])
def test_rms_norm_and_add(T, H):
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(T + H)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    r = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    _close(c.rms_norm(x, w, 1e-6), ref.rms_norm(x, w, 1e-6), 1e-2, 1e-2, "rms_norm")
    y, r2 = c.add_rms_norm(x, r, w, 1e-6)
    yw, rw = ref.add_rms_norm(x, r, w, 1e-6)
    _close(r2, rw, 0, 1e-6, "residual out")
    _close(y, yw, 1e-2, 1e-2, "add_rms_norm")


def test_silu_mul_and_embedding():
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(333, 2 * 1536, device="cuda", generator=g).to(torch.bfloat16)
    _close(c.silu_and_mul(x), ref.silu_and_mul(x), 1e-2, 1e-2, "silu_mul")
    table = torch.randn(1000, 512, device="cuda", generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 1000, (77,), device="cuda", generator=g, dtype=torch.int32)
    assert torch.equal(c.embedding(ids, table), ref.embedding(ids, table))


@pytest.mark.parametrize("D,norm", [(128, True), (128, False), (64, True)])
def test_rope_qknorm_kvwrite(D, norm):
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(D)
    T, nq, nkv, blocks, bs = 50, 8, 2, 16, 16
    qkv = torch.randn(T, (nq + 2 * nkv) * D, device="cuda", generator=g).to(torch.bfloat16)
    pos = torch.randint(0, 500, (T,), device="cuda", generator=g, dtype=torch.int32)
    slots = torch.randperm(blocks * bs, device="cuda", generator=g)[:T].int()
    cs = ref.build_cos_sin_cache(D, 512, 1e6, device="cuda")
    qw = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(torch.bfloat16) if norm else None
    kw = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(torch.bfloat16) if norm else None
    kc = torch.zeros(blocks, bs, nkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kc2, vc2 = kc.clone(), vc.clone()
    want_q = ref.rope_qknorm_kvwrite(qkv.clone(), pos, slots, cs, qw, kw, 1e-6, kc2, vc2, nq, nkv, D)
    got_q = c.rope_qknorm_kvwrite(qkv, pos, slots, cs, qw, kw, 1e-6, kc, vc, nq, nkv, D)
    _close(got_q, want_q, 2e-2, 2e-2, "q")
    _close(kc, kc2, 2e-2, 2e-2, "k cache")
    assert torch.equal(vc, vc2)


def _attn_case(seqs, nq, nkv, D, bs, n_decode, seed=0):
    """seqs: list of (q_len, kv_len).  Builds paged caches with random block tables and a StepInput."""
    g = torch.Generator().manual_seed(seed)
    B = len(seqs)
    T = sum(q for q, _ in seqs)
    mb = max((kv + bs - 1) // bs for _, kv in seqs)
    n_blocks = sum((kv + bs - 1) // bs for _, kv in seqs) + 1
    perm = (torch.randperm(n_blocks - 1, generator=g) + 1).tolist()
    L = make_layout(T, B, mb, B, 32)
    host = torch.zeros(L.total_words, dtype=torch.int32)
    hdr = np.zeros(32, dtype=np.int32)
    q_cu, kv_lens = [0], []
    bt = torch.zeros(B, L.MB_cap, dtype=torch.int32)
    at = 0
    for i, (ql, kv) in enumerate(seqs):
        q_cu.append(q_cu[-1] + ql)
        kv_lens.append(kv)
        nb = (kv + bs - 1) // bs
        bt[i, :nb] = torch.tensor(perm[at:at + nb], dtype=torch.int32)
        at += nb
    host[L.q_cu:L.q_cu + B + 1] = torch.tensor(q_cu, dtype=torch.int32)
    host[L.kv_lens:L.kv_lens + B] = torch.tensor(kv_lens, dtype=torch.int32)
    host[L.block_tables:L.block_tables + B * L.MB_cap] = bt.reshape(-1)
    hdr[0], hdr[1], hdr[3], hdr[4] = T, B, n_decode, B - n_decode
    hdr[5], hdr[6], hdr[17] = max(q for q, _ in seqs), max(kv for _, kv in seqs), bs
    hdr[21] = sum(q for q, _ in seqs[n_decode:])
    inp = StepInput(host.cuda(), L, hdr)
    gq = torch.Generator(device="cuda").manual_seed(seed + 1)
    q = torch.randn(T, nq, D, device="cuda", generator=gq).to(torch.bfloat16)
    kc = torch.randn(n_blocks, bs, nkv, D, device="cuda", generator=gq).to(torch.bfloat16)
    vc = torch.randn(n_blocks, bs, nkv, D, device="cuda", generator=gq).to(torch.bfloat16)
    return q, kc, vc, inp


@pytest.mark.parametrize("nq,nkv,D,bs", [(8, 2, 128, 16), (4, 4, 128, 16), (16, 2, 128, 128), (8, 2, 64, 16)])
def test_prefill_attention(nq, nkv, D, bs):
    c = cuda_ops()
    seqs = [(64, 64), (1, 1), (100, 100), (37, 165), (200, 777), (5, 5)]
    q, kc, vc, inp = _attn_case(seqs, nq, nkv, D, bs, n_decode=0, seed=nq)
    scale = D ** -0.5
    got = c.paged_attention(q, kc, vc, inp, scale)
    want = ref.paged_attention(q, kc, vc, inp.q_cu, inp.kv_lens, inp.block_tables, inp.n_seqs, scale)
    _close(got, want, 2e-2, 2e-2, "prefill attention")


@pytest.mark.parametrize("bs", [16, 32, 64, 128])
@pytest.mark.parametrize("window", [-1, 200])
def test_prefill_attention_tcgen05_long_and_chunked(bs, window):
    """The tcgen05 prefill kernel on prompts that span many KV tiles, chunked prefill (kv_len > q_len), tile-boundary
    lengths, every supported block size and a sliding window; the mma.sync kernel must agree as well."""
    c = cuda_ops()
    seqs = [(1024, 1024), (300, 1500), (128, 128), (129, 400), (64, 64), (1, 1), (127, 255), (65, 4000)]
    q, kc, vc, inp = _attn_case(seqs, 8, 2, 128, bs, n_decode=0, seed=bs)
    scale = 128 ** -0.5
    want = ref.paged_attention(q, kc, vc, inp.q_cu, inp.kv_lens, inp.block_tables, inp.n_seqs, scale, window)
    try:
        for tc in (True, False):
            c.prefill_use_tc(tc)
            got = c.paged_attention(q, kc, vc, inp, scale, window)
            assert c.read_status() == 0
            _close(got, want, 2e-2, 2e-2, f"prefill attention (tcgen05={tc}, block {bs}, window {window})")
    finally:
        c.prefill_use_tc(True)


@pytest.mark.parametrize("nq,nkv", [(4, 1), (2, 2), (8, 2)])
@pytest.mark.parametrize("splits", [0, 1, 3, 8])
def test_prefill_attention_tcgen05_kv_split(nq, nkv, splits):
    """Key-range split of the tcgen05 prefill kernel (few heads per GPU: tensor-parallel shards, short prompts): fp32
    partials merged by the last split to arrive; tiles with fewer key tiles than splits, chunked prefill, a sliding window,
    and a second launch on the same counters."""
    c = cuda_ops()
    seqs = [(1024, 1024), (200, 3000), (1, 1), (64, 64), (129, 129), (300, 301)]
    q, kc, vc, inp = _attn_case(seqs, nq, nkv, 128, 16, n_decode=0, seed=splits + nq)
    scale = 128 ** -0.5
    try:
        c.prefill_kv_split(splits)
        for window in (-1, 150):
            want = ref.paged_attention(q, kc, vc, inp.q_cu, inp.kv_lens, inp.block_tables, inp.n_seqs, scale, window)
            for rep in range(2):
                got = c.paged_attention(q, kc, vc, inp, scale, window)
                assert c.read_status() == 0
                _close(got, want, 2e-2, 2e-2, f"prefill attention, {splits} key splits, window {window}, launch {rep}")
    finally:
        c.prefill_kv_split(1)


def test_prefill_attention_tcgen05_strided_q():
    """q as a column slice of the fused qkv buffer (row pitch larger than Hq * D), as the models pass it."""
    c = cuda_ops()
    seqs = [(200, 200), (70, 333)]
    q, kc, vc, inp = _attn_case(seqs, 8, 2, 128, 16, n_decode=0, seed=3)
    T = q.shape[0]
    qkv = torch.randn(T, (8 + 4) * 128, device="cuda").to(torch.bfloat16)
    qkv[:, :8 * 128] = q.reshape(T, -1)
    qv = qkv[:, :8 * 128].view(T, 8, 128)
    got = c.paged_attention(qv, kc, vc, inp, 128 ** -0.5)
    assert c.read_status() == 0
    want = ref.paged_attention(q, kc, vc, inp.q_cu, inp.kv_lens, inp.block_tables, inp.n_seqs, 128 ** -0.5)
    _close(got, want, 2e-2, 2e-2, "prefill attention, strided q")


@pytest.mark.parametrize("kernel", ["tma", "cp_async"])
@pytest.mark.parametrize("nq,nkv,D,bs", [(8, 2, 128, 16), (32, 8, 128, 16), (8, 1, 128, 128), (4, 4, 64, 16), (16, 2, 128, 32),
                                         (8, 2, 64, 64)])
def test_decode_attention(nq, nkv, D, bs, kernel):
    c = cuda_ops()
    seqs = [(1, 1), (1, 17), (1, 64), (1, 1000), (1, 3333), (1, 129), (1, 65), (1, 4096)]
    q, kc, vc, inp = _attn_case(seqs, nq, nkv, D, bs, n_decode=len(seqs), seed=nkv)
    scale = D ** -0.5
    c.decode_kernel = kernel
    try:
        got = c.paged_attention(q, kc, vc, inp, scale)
        assert c.read_status() == 0
    finally:
        c.decode_kernel = "tma"
    want = ref.paged_attention(q, kc, vc, inp.q_cu, inp.kv_lens, inp.block_tables, inp.n_seqs, scale)
    _close(got, want, 2e-2, 2e-2, f"decode attention ({kernel})")


def test_mixed_and_speculative_rows():
    """Decode rows with q_len 2 (one draft token) followed by prefill chunks, in one call."""
    c = cuda_ops()
    seqs = [(2, 40), (2, 513), (1, 90), (70, 300), (128, 128)]
    q, kc, vc, inp = _attn_case(seqs, 8, 2, 128, 16, n_decode=3, seed=9)
    got = c.paged_attention(q, kc, vc, inp, 128 ** -0.5)
    want = ref.paged_attention(q, kc, vc, inp.q_cu, inp.kv_lens, inp.block_tables, inp.n_seqs, 128 ** -0.5)
    _close(got, want, 2e-2, 2e-2, "mixed attention")


def test_mixed_attention_padded_reads_ranges_on_device():
    """A padded step (graph capture / replay): launches are sized for the layout capacities and the kernels take the
    decode / prefill split from the device-side header, so one launch configuration serves different splits."""
    c = cuda_ops()
    from xllm_wxh_b200.framework.step_input import FWD_MIXED, H_FWD_TYPE
    for seqs, n_dec in (([(1, 40), (1, 513), (1, 90), (70, 300), (128, 128)], 3), ([(1, 700), (200, 200), (3, 64), (9, 9)], 1)):
        q, kc, vc, inp0 = _attn_case(seqs, 8, 2, 128, 16, n_decode=n_dec, seed=11)
        T, B = inp0.n_tokens, inp0.n_seqs
        Lp = make_layout(256, 8, 64, 8, 32)               # capacities beyond the real sizes
        host = torch.zeros(Lp.total_words, dtype=torch.int32)
        hdr = inp0.header.copy()
        hdr[H_FWD_TYPE] = FWD_MIXED
        host[Lp.header:Lp.header + 32] = torch.from_numpy(hdr)
        q_cu = inp0.q_cu.cpu()
        host[Lp.q_cu:Lp.q_cu + B + 1] = q_cu
        host[Lp.q_cu + B + 1:Lp.q_cu + Lp.B_cap + 1] = int(q_cu[-1])          # padding sequences are empty
        host[Lp.kv_lens:Lp.kv_lens + B] = inp0.kv_lens.cpu()
        bt = torch.zeros(Lp.B_cap, Lp.MB_cap, dtype=torch.int32)
        bt[:B, :inp0.block_tables.shape[1]] = inp0.block_tables.cpu()
        host[Lp.block_tables:Lp.block_tables + Lp.B_cap * Lp.MB_cap] = bt.reshape(-1)
        inp = StepInput(host.cuda(), Lp, hdr, padded=True)
        qp = torch.zeros(Lp.T_cap, 8, 128, device="cuda", dtype=torch.bfloat16)
        qp[:T] = q
        got = c.paged_attention(qp, kc, vc, inp, 128 ** -0.5)
        assert c.read_status() == 0
        want = ref.paged_attention(q, kc, vc, inp0.q_cu, inp0.kv_lens, inp0.block_tables, B, 128 ** -0.5)
        _close(got[:T], want, 2e-2, 2e-2, "padded mixed attention")
        assert torch.count_nonzero(got[T:]).item() == 0


def _sample_inp(S, temps, top_k, top_p, seeds, logprobs=0):
    L = make_layout(S, S, 1, S, 32)
    host = torch.zeros(L.total_words, dtype=torch.int32)
    host[L.temperature:L.temperature + S] = torch.tensor(temps, dtype=torch.float32).view(torch.int32)
    host[L.top_p:L.top_p + S] = torch.tensor(top_p, dtype=torch.float32).view(torch.int32)
    host[L.top_k:L.top_k + S] = torch.tensor(top_k, dtype=torch.int32)
    host[L.seed_lo:L.seed_lo + S] = torch.tensor(seeds, dtype=torch.int32)
    host[L.rep_pen:L.rep_pen + S] = torch.ones(S).view(torch.int32)
    hdr = np.zeros(32, dtype=np.int32)
    hdr[0] = hdr[1] = hdr[2] = S
    hdr[15] = int(all(t == 0 for t in temps))
    hdr[16] = int(logprobs > 0)
    hdr[20] = max(0, logprobs - 1)
    return StepInput(host.cuda(), L, hdr)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sampling_greedy_and_logprobs(dtype):
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(3)
    S, V = 9, 151936
    logits = (torch.randn(S, V, device="cuda", generator=g) * 3).to(dtype)
    inp = _sample_inp(S, [0.0] * S, [-1] * S, [1.0] * S, list(range(S)), logprobs=6)
    tok, lp, tv, ti = c.sample(logits, inp)
    want_tok, want_lp, want_tv, want_ti = ref.sample(logits, inp.temperature, inp.top_k, inp.top_p, inp.seed_lo, inp.seed_hi, True, 5)
    assert torch.equal(tok.cpu(), want_tok.cpu())
    _close(lp, want_lp, 1e-3, 1e-3, "logprob")
    _close(tv, want_tv, 1e-3, 1e-3, "top logprobs")
    # equal logits may be listed in either order: compare the logits the ids point at
    _close(logits.float().gather(1, ti.long()), logits.float().gather(1, want_ti.long()), 0, 0, "top ids")


def test_sampling_topk_topp_distribution():
    """Tokens drawn by the kernel must lie in the reference's top-k/top-p set and follow its probabilities."""
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(11)
    V, S = 4096, 2048
    base = torch.randn(V, device="cuda", generator=g) * 2.5
    logits = base[None, :].repeat(S, 1).contiguous()
    temp, k, p = 0.8, 50, 0.9
    inp = _sample_inp(S, [temp] * S, [k] * S, [p] * S, [1000 + i for i in range(S)])
    tok, _, _, _ = c.sample(logits, inp)
    filt = ref.top_k_top_p_filter((base / temp)[None, :], torch.tensor([k], device="cuda"), torch.tensor([p], device="cuda"))[0]
    probs = torch.softmax(filt, -1)
    allowed = probs > 0
    assert bool(allowed[tok.long()].all()), "sampled a token outside the nucleus"
    freq = torch.bincount(tok.long(), minlength=V).float() / S
    tvd = 0.5 * (freq - probs).abs().sum().item()
    assert tvd < 0.12, f"total variation distance {tvd}"


@pytest.mark.parametrize("dtype,V", [(torch.bfloat16, 151936), (torch.float32, 32000), (torch.bfloat16, 5000)])
def test_sampling_candidate_way_equals_general_way(dtype, V):
    """Rows with a small top-k decide among the candidates above a lower bound of their k-th largest logit; the tokens
    must be those of the general radix selection over the whole row (same seeds), for top-k alone and with top-p, with
    ties in the logits (bf16), and the log-probabilities must agree."""
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(V)
    S = 96
    logits = (torch.randn(S, V, device="cuda", generator=g) * 2.5).to(dtype)
    ks = [1, 2, 7, 50, 64, 200, 256, 20] * (S // 8)
    ps = [1.0, 0.9, 0.5, 0.95] * (S // 4)
    temps = [0.7, 1.0, 1.3] * (S // 3)
    inp = _sample_inp(S, temps, ks, ps, [77 + i for i in range(S)], logprobs=1)
    try:
        c.lib().xl_sample_short_way(0)
        want_tok, want_lp, _, _ = c.sample(logits, inp)
        c.lib().xl_sample_short_way(1)
        tok, lp, _, _ = c.sample(logits, inp)
    finally:
        c.lib().xl_sample_short_way(1)
    torch.cuda.synchronize()
    same = (tok == want_tok).sum().item()
    assert same >= S - 2, (same, S)            # a draw that lands on a rounding boundary may fall to the neighbour
    ok = tok == want_tok
    _close(lp[ok], want_lp[ok], 1e-3, 1e-3, "logprob of the drawn token")
    # every drawn token is among the k largest of its row
    kth = torch.topk(logits.float(), 256, dim=-1).values
    for r in range(S):
        assert logits[r, tok[r].long()].float() >= kth[r, ks[r] - 1]


@pytest.mark.parametrize("dtype,V", [(torch.bfloat16, 18992), (torch.float32, 4096), (torch.bfloat16, 600)])
def test_topk_candidates_of_a_vocabulary_slice(dtype, V):
    """Per-shard candidates of vocabulary-parallel sampling against the PyTorch statement: the k largest logits with the
    ties at the k-th, in index order, global ids; the arg-max for greedy rows; a row that asks for more than fits raises
    the overflow flag."""
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(V)
    S, W = 24, 96
    logits = (torch.randn(S, V, device="cuda", generator=g) * 2.5).to(dtype)
    ks = [1, 2, 7, 50, 64, 20] * (S // 6)
    temps = [0.0, 0.8, 1.0, 0.7] * (S // 4)
    inp = _sample_inp(S, temps, ks, [1.0] * S, list(range(S)))
    vals, ids, over = c.topk_candidates(logits, inp, 1000, W)
    want_v, want_i, want_o = ref.topk_candidates(logits, inp.temperature, inp.top_k, 1000, W)
    torch.cuda.synchronize()
    assert int(over.item()) == 0 and int(want_o.item()) == 0
    assert torch.equal(ids.cpu(), want_i.cpu())
    assert torch.equal(vals.cpu(), want_v.cpu())
    inp2 = _sample_inp(S, [0.9] * S, [200] * S, [1.0] * S, list(range(S)))
    _, _, over2 = c.topk_candidates(logits, inp2, 0, W)
    assert int(over2.item()) == 1


def test_penalties():
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(2)
    S, V = 3, 1000
    logits = torch.randn(S, V, device="cuda", generator=g)
    L = make_layout(S, S, 1, S, 64)
    host = torch.zeros(L.total_words, dtype=torch.int32)
    host[L.pen_cu:L.pen_cu + S + 1] = torch.tensor([0, 3, 3, 8], dtype=torch.int32)
    host[L.pen_ids:L.pen_ids + 8] = torch.tensor([5, 9, 700, 1, 2, 3, 4, 999], dtype=torch.int32)
    # low half: occurrences in the whole sequence; high half: occurrences among the generated tokens (what the frequency
    # and presence penalties count)
    total, generated = [1, 2, 3, 1, 1, 4, 1, 2], [0, 1, 3, 1, 0, 2, 1, 0]
    host[L.pen_counts:L.pen_counts + 8] = torch.tensor([t | (g << 16) for t, g in zip(total, generated)], dtype=torch.int32)
    host[L.rep_pen:L.rep_pen + S] = torch.tensor([1.3, 1.0, 1.1]).view(torch.int32)
    host[L.freq_pen:L.freq_pen + S] = torch.tensor([0.5, 0.0, 0.2]).view(torch.int32)
    host[L.pres_pen:L.pres_pen + S] = torch.tensor([0.1, 0.0, 0.3]).view(torch.int32)
    host[L.top_p:L.top_p + S] = torch.ones(S).view(torch.int32)
    hdr = np.zeros(32, dtype=np.int32)
    hdr[0] = hdr[1] = hdr[2] = S
    hdr[14] = 1
    hdr[15] = 1
    inp = StepInput(host.cuda(), L, hdr)
    want = ref.apply_penalties(logits.clone(), inp.pen_cu, inp.pen_ids, inp.pen_counts, inp.rep_pen, inp.freq_pen, inp.pres_pen)
    tok, _, _, _ = c.sample(logits, inp)          # applies the penalties in place first
    _close(logits, want, 1e-5, 1e-5, "penalised logits")
    assert torch.equal(tok.cpu().long(), want.argmax(-1).cpu())


@pytest.mark.parametrize("E,k,scoring,groups", [(128, 8, "softmax", (1, 1)), (256, 8, "sigmoid", (8, 4)), (64, 6, "sigmoid", (1, 1)),
                                                (8, 2, "softmax", (1, 1)), (256, 8, "softmax", (8, 4))])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_moe_router(E, k, scoring, groups, dtype):
    from xllm_wxh_b200.ops import moe_cuda
    g = torch.Generator(device="cuda").manual_seed(E + k)
    T = 333
    logits = (torch.randn(T, E, device="cuda", generator=g) * 2).to(dtype)
    bias = (torch.randn(E, device="cuda", generator=g) * 0.1) if scoring == "sigmoid" else None
    hist = torch.zeros(E, dtype=torch.int64, device="cuda")
    w, ids = moe_cuda.moe_router(logits, k, scoring, True, bias, groups[0], groups[1], 2.5, load_hist=hist)
    ww, wi = ref.moe_router(logits, k, scoring, True, bias, groups[0], groups[1], 2.5)
    # same expert sets (order inside the top-k is by score in both) and same weights
    assert torch.equal(ids.sort(-1).values.cpu(), wi.sort(-1).values.cpu())
    order_g, order_w = ids.argsort(-1), wi.argsort(-1)
    _close(w.gather(-1, order_g), ww.gather(-1, order_w), 1e-3, 1e-5, "router weights")
    assert int(hist.sum()) == T * k
    assert torch.equal(hist.cpu(), torch.bincount(ids.reshape(-1).long().cpu(), minlength=E))


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("T,E,k,H,I,e0,El", [(200, 16, 4, 512, 256, 0, 16), (77, 32, 8, 256, 128, 8, 8), (1, 8, 2, 256, 64, 0, 8),
                                              (700, 128, 8, 2048, 768, 0, 128)])
def test_moe_experts_grouped_gemm(T, E, k, H, I, e0, El, interleaved):
    from xllm_wxh_b200.ops import moe_cuda
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(T + E)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    w13 = (torch.randn(El, 2 * I, H, device="cuda", generator=g) / math.sqrt(H)).to(torch.bfloat16)
    w2 = (torch.randn(El, H, I, device="cuda", generator=g) / math.sqrt(I)).to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda", generator=g)
    w, ids = ref.moe_router(logits, k)
    want = ref.moe_experts(x, w13, w2, w, ids, e0)
    w13_dev = moe_cuda.interleave_w13(w13.clone()) if interleaved else w13
    got = moe_cuda.moe_experts(x, w13_dev, w2, w, ids, e0, interleaved)
    assert c.read_status() == 0
    _close(got, want, 3e-2, 3e-2, "moe experts")


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 1536, 7168), (1280, 4096, 512), (77, 576, 1024), (1024, 2048, 2048)])
def test_gemm_fp8_block_scaled(M, N, K):
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16)
    wq, ws = ref.quant_weight_128x128(w)
    got = c.linear_fp8_block(x, wq, ws)
    want = ref.linear_fp8_block(x, wq, ws)
    assert c.read_status() == 0
    _close(got, want, 2e-2, 2e-2, "fp8 block-scaled gemm")
    # and the quantiser itself
    q, s = c.quant_act_1x128(x)
    qw, sw = ref.quant_act_1x128(x)
    _close(s, sw, 1e-6, 1e-9, "activation scales")
    _close(q.float() * s.repeat_interleave(128, 1), qw.float() * sw.repeat_interleave(128, 1), 0.07, 1e-3, "quantised activations")


def test_moe_experts_fp8_grouped():
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(4)
    T, E, k, H, I = 300, 16, 4, 512, 256
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, device="cuda", generator=g) / math.sqrt(H)).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, device="cuda", generator=g) / math.sqrt(I)).to(torch.bfloat16)
    q13 = [ref.quant_weight_128x128(w13[e]) for e in range(E)]
    q2 = [ref.quant_weight_128x128(w2[e]) for e in range(E)]
    w13q, s13 = torch.stack([a for a, _ in q13]), torch.stack([b for _, b in q13])
    w2q, s2 = torch.stack([a for a, _ in q2]), torch.stack([b for _, b in q2])
    w, ids = ref.moe_router(torch.randn(T, E, device="cuda", generator=g), k)
    got = c.moe_experts_fp8(x, w13q, s13, w2q, s2, w, ids, 0)
    d13 = torch.stack([ref.dequant_weight_128x128(w13q[e], s13[e]) for e in range(E)]).to(torch.bfloat16)
    d2 = torch.stack([ref.dequant_weight_128x128(w2q[e], s2[e]) for e in range(E)]).to(torch.bfloat16)
    want = ref.moe_experts_fp8(x, d13, d2, w, ids, 0)
    assert c.read_status() == 0
    _close(got, want, 5e-2, 5e-2, "fp8 moe experts")


def _mla_case(seqs, Hh, bs, seed=0):
    g = torch.Generator().manual_seed(seed)
    C, R = 512, 64
    B = len(seqs)
    T = sum(q for q, _ in seqs)
    mb = max((kv + bs - 1) // bs for _, kv in seqs)
    n_blocks = sum((kv + bs - 1) // bs for _, kv in seqs) + 1
    perm = (torch.randperm(n_blocks - 1, generator=g) + 1).tolist()
    L = make_layout(T, B, mb, B, 32)
    host = torch.zeros(L.total_words, dtype=torch.int32)
    q_cu, at = [0], 0
    bt = torch.zeros(B, L.MB_cap, dtype=torch.int32)
    for i, (ql, kv) in enumerate(seqs):
        q_cu.append(q_cu[-1] + ql)
        nb = (kv + bs - 1) // bs
        bt[i, :nb] = torch.tensor(perm[at:at + nb], dtype=torch.int32)
        at += nb
    host[L.q_cu:L.q_cu + B + 1] = torch.tensor(q_cu, dtype=torch.int32)
    host[L.kv_lens:L.kv_lens + B] = torch.tensor([kv for _, kv in seqs], dtype=torch.int32)
    host[L.block_tables:L.block_tables + B * L.MB_cap] = bt.reshape(-1)
    hdr = np.zeros(32, dtype=np.int32)
    hdr[0], hdr[1], hdr[17] = T, B, bs
    inp = StepInput(host.cuda(), L, hdr)
    gq = torch.Generator(device="cuda").manual_seed(seed + 1)
    q_lat = (torch.randn(T, Hh, C, device="cuda", generator=gq) * 0.5).to(torch.bfloat16)
    q_pe = (torch.randn(T, Hh, R, device="cuda", generator=gq) * 0.5).to(torch.bfloat16)
    cache = (torch.randn(n_blocks, bs, C + R, device="cuda", generator=gq) * 0.5).to(torch.bfloat16)
    return q_lat, q_pe, cache, inp


@pytest.mark.parametrize("Hh,bs,seqs", [(16, 16, [(1, 1), (1, 200), (2, 77), (1, 1000)]), (32, 64, [(40, 40), (100, 300), (3, 500)]),
                                        (128, 16, [(1, 600), (17, 17)]), (128, 32, [(1, 64), (1, 65), (1, 4000), (2, 129)]),
                                        (64, 128, [(5, 700), (1, 1)]), (16, 16, [(5, 5), (70, 70), (33, 33), (130, 130)]),
                                        (16, 16, [(1, 6), (1, 71), (1, 34), (1, 131)]), (16, 32, [(20, 300), (9, 9)])])
@pytest.mark.parametrize("kernel", ["tcgen05", "tcgen05_split", "tcgen05_single", "tcgen05_single_split", "mma_sync"])
def test_mla_attention(Hh, bs, seqs, kernel, monkeypatch):
    """`tcgen05`: the tensor-memory kernel, two CTAs of a tile as a cluster that shares the Q K^T work (automatic key
    splits); `..._split`: every key range cut into up to 5 splits and merged; `tcgen05_single`: the two CTAs of a tile
    working independently; `mma_sync`: the older kernel; all against the fp32 statement of the op."""
    c = cuda_ops()
    monkeypatch.setenv("XLLM_MLA_TC", "0" if kernel == "mma_sync" else "1")
    c.lib().xl_mla_pair_mode(0 if "single" in kernel else 1)
    q_lat, q_pe, cache, inp = _mla_case(seqs, Hh, bs, seed=Hh)
    scale = 192 ** -0.5
    want = ref.mla_attention(q_lat, q_pe, cache, inp.q_cu, inp.kv_lens, inp.block_tables, inp.n_seqs, scale, 512)
    c.lib().xl_mla_kv_split(5 if kernel.endswith("_split") else 1)
    try:
        before = c.launch_count
        got_hm = c.mla_attention(q_lat.transpose(0, 1).contiguous(), q_pe.transpose(0, 1).contiguous(), cache, inp, scale, 512)
        torch.cuda.synchronize()
    finally:
        c.lib().xl_mla_kv_split(1)
        c.lib().xl_mla_pair_mode(0)
    assert c.launch_count == before + 1 and c.read_status() == 0
    _close(got_hm.transpose(0, 1), want, 2e-2, 2e-2, "mla attention")


@pytest.mark.parametrize("Hh,T,k,n_blocks,bs", [(16, 70, 12, 9, 16), (128, 3, 200, 20, 64), (32, 130, 64, 40, 16), (16, 1, 1, 2, 16)])
def test_mla_attention_sparse(Hh, T, k, n_blocks, bs):
    """Attention over per-token lists of cache slots (what a lightning indexer keeps): the paged MLA kernel reads every
    row of `sel` as a block table of one-slot blocks; against the fp32 statement of the op."""
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(Hh + T)
    C, R = 512, 64
    q_lat = (torch.randn(T, Hh, C, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    q_pe = (torch.randn(T, Hh, R, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    cache = (torch.randn(n_blocks, bs, C + R, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    slots = n_blocks * bs
    sel = torch.stack([torch.randperm(slots, device="cuda", generator=g)[:k] for _ in range(T)]).int()
    sel_len = torch.randint(1, k + 1, (T,), device="cuda", generator=g, dtype=torch.int32)
    sel_len[0] = k
    scale = 192 ** -0.5
    want = ref.mla_attention_sparse(q_lat, q_pe, cache, sel, sel_len, scale, 512)
    before = c.launch_count
    got_hm = c.mla_attention_sparse(q_lat.transpose(0, 1).contiguous(), q_pe.transpose(0, 1).contiguous(), cache, sel, sel_len, scale, 512)
    torch.cuda.synchronize()
    assert c.launch_count == before + 1 and c.read_status() == 0
    _close(got_hm.transpose(0, 1), want, 2e-2, 2e-2, "sparse mla attention")


@pytest.mark.parametrize("NH,bs,lens,q_lens", [(64, 16, [200, 77, 1000], [1, 1, 1]), (16, 64, [300, 40], [300, 40]),
                                             (32, 16, [130, 65, 64, 1], [3, 2, 1, 1]), (64, 128, [5000], [70])])
def test_index_scores(NH, bs, lens, q_lens):
    """Lightning-indexer scores sum_h w_h relu(q_h . k) over the causal keys of each token's sequence, read through the
    block tables; -inf at later keys; against the fp32 statement."""
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(NH + bs)
    B = len(lens)
    nbs = [(L + bs - 1) // bs for L in lens]
    n_blocks = sum(nbs) + 1
    mb = max(nbs) + 1
    perm = (torch.randperm(n_blocks - 1) + 1).int()
    bt = torch.zeros(B, mb, dtype=torch.int32)
    at = 0
    for i, nb in enumerate(nbs):
        bt[i, :nb] = perm[at:at + nb]
        at += nb
    pos, seq = [], []
    for i, (L, n) in enumerate(zip(lens, q_lens)):
        pos += list(range(L - n, L))
        seq += [i] * n
    pos, seq = pos + [0], seq + [-1]                       # one padded row
    T = len(pos)
    S = max(nbs) * bs
    keys = (torch.randn(n_blocks, bs, 128, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    q = (torch.randn(T, NH, 128, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w = torch.randn(T, NH, device="cuda", generator=g)
    bt_d = bt.cuda()
    pos_d, seq_d = torch.tensor(pos, dtype=torch.int32, device="cuda"), torch.tensor(seq, dtype=torch.int32, device="cuda")
    before = c.launch_count
    got = c.index_scores(q, w, keys, bt_d, seq_d, pos_d, S)
    torch.cuda.synchronize()
    assert got is not None and got.shape == (T, S) and c.launch_count == before + 1 and c.read_status() == 0
    flat = keys.view(-1, 128).float()
    for t in range(T):
        i = max(seq[t], 0)
        slots = (bt_d[i, :S // bs].long()[:, None] * bs + torch.arange(bs, device="cuda")[None, :]).reshape(S)
        logit = q[t].float() @ flat[slots].t()                                       # [NH, S]
        want = (torch.relu(logit) * w[t][:, None]).sum(0)
        n = pos[t] + 1
        assert torch.isinf(got[t, n:]).all() and (got[t, n:] < 0).all(), t
        _close(got[t, :n], want[:n], 2e-2, 2e-2 * float(want[:n].abs().max()), f"index scores of token {t}")


def test_mla_prepare_and_v_up():
    import xllm_wxh_b200.ops as ops
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(8)
    T, Hh, nope, rope, C, bs, blocks = 70, 16, 128, 64, 512, 16, 8
    q = torch.randn(T, Hh, nope + rope, device="cuda", generator=g).to(torch.bfloat16)
    kv_a = torch.randn(T, C + rope, device="cuda", generator=g).to(torch.bfloat16)
    pos = torch.randint(0, 300, (T,), device="cuda", generator=g, dtype=torch.int32)
    slots = torch.randperm(blocks * bs, device="cuda", generator=g)[:T].int()
    cs = ref.build_cos_sin_cache(rope, 512, 1e4, device="cuda")
    nw = (1 + 0.1 * torch.randn(C, device="cuda", generator=g)).to(torch.bfloat16)
    w_kc = (torch.randn(Hh, nope, C, device="cuda", generator=g) / math.sqrt(nope)).to(torch.bfloat16)
    w_vc = (torch.randn(Hh, 128, C, device="cuda", generator=g) / math.sqrt(C)).to(torch.bfloat16)
    cache_ref = torch.zeros(blocks, bs, C + rope, device="cuda", dtype=torch.bfloat16)
    cache = cache_ref.clone()
    # reference (token-major) through the CPU formulation evaluated on GPU tensors
    cs_t = cs.index_select(0, pos.long())
    lat = ref.rms_norm(kv_a[:, :C], nw, 1e-6)
    k_pe = ref.apply_rope_interleaved(kv_a[:, None, C:], cs_t[:, :rope // 2], cs_t[:, rope // 2:])[:, 0]
    cache_ref.view(-1, C + rope).index_copy_(0, slots.long(), torch.cat([lat, k_pe], -1))
    want_pe = ref.apply_rope_interleaved(q[..., nope:], cs_t[:, :rope // 2], cs_t[:, rope // 2:])
    want_lat = torch.einsum("thn,hnc->thc", q[..., :nope].float(), w_kc.float())
    got_lat, got_pe = c.mla_prepare(q, kv_a, pos, slots, cs, nw, 1e-6, cache, w_kc, nope, rope, C)
    _close(cache, cache_ref, 2e-2, 2e-2, "latent cache")
    _close(got_pe.transpose(0, 1), want_pe, 2e-2, 2e-2, "q_pe")
    _close(got_lat.transpose(0, 1), want_lat, 2e-2, 3e-2, "q_lat")
    o_lat = torch.randn(Hh, T, C, device="cuda", generator=g).to(torch.bfloat16)
    want_o = torch.einsum("htc,hvc->thv", o_lat.float(), w_vc.float()).reshape(T, -1)
    _close(c.mla_v_up(o_lat, w_vc), want_o, 2e-2, 3e-2, "v up-projection")
    assert c.read_status() == 0


def test_mla_absorb_weights_are_not_shared_between_models_at_one_address():
    """The absorb GEMM reads a transposed copy of W_kc; a second model whose W_kc lands at the address the first one freed
    must get its own copy."""
    c = cuda_ops()
    Hh, nope, C = 16, 128, 512
    w1 = torch.randn(Hh, nope, C, device="cuda").to(torch.bfloat16)
    t1 = c._w_kc_t(w1)
    addr = w1.data_ptr()
    assert torch.equal(t1, w1.transpose(1, 2))
    del w1, t1
    w2 = torch.randn(Hh, nope, C, device="cuda").to(torch.bfloat16)
    if w2.data_ptr() != addr:
        pytest.skip("the allocator did not reuse the address")
    assert torch.equal(c._w_kc_t(w2), w2.transpose(1, 2))
    w2.mul_(2)                                            # rewritten in place: the copy follows
    assert torch.equal(c._w_kc_t(w2), w2.transpose(1, 2))


# ----------------------------------------------------------------------------- fp8 with per-token / per-channel scales
@pytest.mark.parametrize("T,H", [(1, 128), (77, 1024), (300, 4096), (129, 12288)])
def test_quant_rows_fp8_and_fused_norm(T, H):
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(T + H)
    x = (torch.randn(T, H, device="cuda", generator=g) * 3).to(torch.bfloat16)
    res = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    q, s = c.quant_rows_fp8(x)
    qr, sr = ref.quant_rows_fp8(x)
    _close(s, sr, 1e-6, 1e-9, "row scales")
    _close(q.float() * s[:, None], x.float(), 0.07, 1e-3, "quantised rows")          # e4m3: 3 mantissa bits
    q1, s1 = c.rms_norm_quant_fp8(x, w, 1e-6)
    h = ref.rms_norm(x, w, 1e-6)
    _close(s1, ref.quant_rows_fp8(h)[1], 1e-2, 1e-6, "row scales after the norm")
    _close(q1.float() * s1[:, None], h.float(), 0.07, 2e-2, "norm + quant")
    q2, s2, r2 = c.add_rms_norm_quant_fp8(x, res, w, 1e-6)
    h2, want_res = ref.add_rms_norm(x, res, w, 1e-6)
    assert torch.equal(r2, want_res)
    _close(q2.float() * s2[:, None], h2.float(), 0.07, 2e-2, "add + norm + quant")
    assert c.read_status() == 0


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 1536, 4096), (1279, 4096, 512), (77, 576, 1024), (1279, 6144, 4096),
                                   (256, 4096, 12288)])
@pytest.mark.parametrize("mode", ["tensor", "channel", "bias"])
def test_gemm_fp8_scaled(M, N, K, mode):
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)
    if mode == "tensor":
        cs, ts = None, float(w.abs().max() / 448.0)
        wq = (w / ts).to(torch.float8_e4m3fn)
    else:
        cs, ts = (w.abs().amax(1).clamp_min(1e-8) / 448.0).float(), 1.0
        wq = (w / cs[:, None]).to(torch.float8_e4m3fn)
    bias = torch.randn(N, device="cuda", generator=g).to(torch.bfloat16) if mode == "bias" else None
    xq, xs = c.quant_rows_fp8(x)
    got = c.linear_fp8_scaled(xq, xs, wq, cs, ts, bias)
    want = ref.linear_fp8_scaled(xq, xs, wq, cs, ts, bias, out_dtype=torch.float32)
    assert c.read_status() == 0
    _close(got, want, 1e-2, 1e-2, "fp8 scaled gemm")                     # same quantised operands: only bf16 output rounding
    _close(got, x.float() @ w.t() + (bias.float() if bias is not None else 0), 0.1, 0.3, "fp8 scaled gemm vs unquantised")


def test_gemm_fp8_scaled_swiglu():
    c = cuda_ops()
    g = torch.Generator(device="cuda").manual_seed(9)
    M, I, K = 333, 1536, 1024
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn(2 * I, K, device="cuda", generator=g) / math.sqrt(K)
    cs = (w.abs().amax(1).clamp_min(1e-8) / 448.0).float()
    wq = (w / cs[:, None]).to(torch.float8_e4m3fn)
    xq, xs = c.quant_rows_fp8(x)
    wq_i = c.interleave_gate_up(wq.view(torch.uint8)).view(torch.float8_e4m3fn)
    cs_i = c.interleave_gate_up(cs.view(-1, 1)).view(-1).contiguous()
    got = c.linear_fp8_scaled(xq, xs, wq_i, cs_i, 1.0, None, swiglu=True)
    y = ref.linear_fp8_scaled(xq, xs, wq, cs, 1.0, None, out_dtype=torch.float32)
    want = torch.nn.functional.silu(y[:, :I]) * y[:, I:]
    assert c.read_status() == 0
    _close(got, want, 2e-2, 2e-2, "fp8 gate_up with SwiGLU epilogue")
