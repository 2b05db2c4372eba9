"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the kernel library may not allocate device memory where they call it (they run under another
framework's memory plan, or next to a CUDA-graph capture that forbids allocator traffic).  For them the library
exports `xl_decode_attention_noalloc`, which keeps its split-KV workspace in a device array compiled into the library.
This test checks, on two calls in a row (the second one reuses whatever the first left in the workspace), that it
returns bit for bit what the regular entry point returns (the same kernels run) and what a plain fp32 attention gives
within the kernel tests' tolerance, that its own status word (read through `xl_decode_attention_noalloc_status`) stays
0, that an oversized request is refused with a message, and that a sequence the workspace has no room for is skipped and
reported instead of written out of bounds.
The file name keeps it last in collection order, so a failure here cannot hide another test's result under `-x`."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, n_seqs, kv_max, nq=32, nkv=8, D=128, bs=16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    kv = torch.randint(1, kv_max, (n_seqs,), generator=g, device="cuda").int()
    kv[0] = kv_max
    nb = [(int(k) + bs - 1) // bs for k in kv.tolist()]
    mb = max(nb)
    total = sum(nb) + 1
    perm = (torch.randperm(total - 1, device="cuda", generator=g) + 1).int()
    bt = torch.zeros(n_seqs, mb, dtype=torch.int32, device="cuda")
    at = 0
    for i, n in enumerate(nb):
        bt[i, :n] = perm[at:at + n]
        at += n
    q = torch.randn(n_seqs, nq * D, device="cuda", generator=g).to(torch.bfloat16)
    kc = torch.randn(total, bs, nkv, D, device="cuda", generator=g).to(torch.bfloat16)
    vc = torch.randn(total, bs, nkv, D, device="cuda", generator=g).to(torch.bfloat16)
    q_cu = torch.arange(n_seqs + 1, dtype=torch.int32, device="cuda")
    return q, kc, vc, q_cu, kv, bt, mb, total


def _call_both(lib, case, splits, nq=32, nkv=8, D=128, bs=16):
    q, kc, vc, q_cu, kv, bt, mb, total = case
    n = q.shape[0]
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    scale = ctypes.c_float(D ** -0.5)
    # regular entry point: caller-provided workspace
    want = torch.empty(n, nq * D, dtype=torch.bfloat16, device="cuda")
    po = torch.empty(n, nq, splits, D, dtype=torch.float32, device="cuda")
    pl = torch.empty(n, nq, splits, dtype=torch.float32, device="cuda")
    rc = lib.xl_decode_attention_tma(p(q), p(kc), p(vc), p(want), p(q_cu), p(kv), p(bt), 0, n, mb, bs, total, nq, nkv, D, nq * D,
                                     scale, -1, splits, p(po), p(pl), st)
    assert rc == 0
    if splits > 1:
        assert lib.xl_decode_split_merge(p(po), p(pl), p(want), p(q_cu), 0, n, nq, D, splits, ctypes.c_long(n), st) == 0
    # allocation-free entry point
    got = torch.empty_like(want)
    err = ctypes.create_string_buffer(256)
    rc = lib.xl_decode_attention_noalloc(p(q), p(kc), p(vc), p(got), p(q_cu), p(kv), p(bt), n, n, mb, bs, total, nq, nkv, D, nq * D,
                                         scale, splits, st, err, 256)
    assert rc == 0, err.value.decode()
    torch.cuda.synchronize()
    return got, want


def _fp32_reference(case, nq=32, nkv=8, D=128, bs=16):
    q, kc, vc, q_cu, kv, bt, mb, total = case
    out = torch.empty(q.shape[0], nq * D, dtype=torch.float32, device="cuda")
    group = nq // nkv
    for i in range(q.shape[0]):
        n = int(kv[i])
        blocks = bt[i, :(n + bs - 1) // bs].long()
        k = kc[blocks].reshape(-1, nkv, D)[:n].float()               # [n, nkv, D]
        v = vc[blocks].reshape(-1, nkv, D)[:n].float()
        qi = q[i].view(nkv, group, D).float()
        s = torch.einsum("hgd,nhd->hgn", qi, k) * D ** -0.5
        out[i] = torch.einsum("hgn,nhd->hgd", torch.softmax(s, -1), v).reshape(-1)
    return out


def test_noalloc_entry_point_matches_regular_one():
    from xllm_wxh_b200.ops import cuda_ops
    lib = cuda_ops.lib()
    lib.xl_decode_attention_noalloc_status.restype = ctypes.c_int
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for seed, n_seqs, kv_max, splits in [(1, 24, 3000, 4), (2, 7, 900, 2)]:       # two calls in a row share the workspace
        case = _case(seed, n_seqs, kv_max)
        got, want = _call_both(lib, case, splits)
        assert torch.equal(got, want), "the allocation-free entry point runs the same kernels: its output must be identical"
        ref = _fp32_reference(case)
        err = (got.float() - ref).abs()
        assert float(err.max()) <= 2e-2 + 2e-2 * float(ref.abs().max()), float(err.max())
        assert lib.xl_decode_attention_noalloc_status(st) == 0, "a kernel of the allocation-free path reported an error"
    assert cuda_ops.read_status() == 0


def test_noalloc_entry_point_skips_sequences_beyond_the_declared_rows():
    """`max_rows` is the caller's promise about q_cu; the device checks it: with a q_cu that goes further, the sequence
    beyond the limit is left untouched and the status word says so (and is cleared by the read)."""
    from xllm_wxh_b200.ops import cuda_ops
    lib = cuda_ops.lib()
    lib.xl_decode_attention_noalloc_status.restype = ctypes.c_int
    case = _case(5, 6, 400)
    q, kc, vc, q_cu, kv, bt, mb, total = case
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _, want = _call_both(lib, case, 2)
    assert lib.xl_decode_attention_noalloc_status(st) == 0
    # the last sequence now owns two query rows, one more than the six rows that the call declares
    q2 = torch.cat([q, q[-1:]], 0).contiguous()
    q_cu2 = torch.tensor([0, 1, 2, 3, 4, 5, 7], dtype=torch.int32, device="cuda")
    out = torch.full((7, want.shape[1]), 7.0, dtype=want.dtype, device="cuda")
    err = ctypes.create_string_buffer(256)
    rc = lib.xl_decode_attention_noalloc(p(q2), p(kc), p(vc), p(out), p(q_cu2), p(kv), p(bt), 6, 6, mb, 16, total, 32, 8, 128,
                                         32 * 128, ctypes.c_float(128 ** -0.5), 2, st, err, 256)
    assert rc == 0, err.value.decode()
    assert lib.xl_decode_attention_noalloc_status(st) == 6          # XL_ERR_BOUNDS
    assert lib.xl_decode_attention_noalloc_status(st) == 0          # cleared by the read
    assert torch.equal(out[:5], want[:5]) and bool((out[5:] == 7.0).all())


def test_noalloc_entry_point_rejects_oversized_requests():
    from xllm_wxh_b200.ops import cuda_ops
    lib = cuda_ops.lib()
    q, kc, vc, q_cu, kv, bt, mb, total = _case(3, 4, 200)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    err = ctypes.create_string_buffer(256)
    out = torch.empty_like(q)
    rc = lib.xl_decode_attention_noalloc(p(q), p(kc), p(vc), p(out), p(q_cu), p(kv), p(bt), 4, 4096, mb, 16, total, 32, 8, 128,
                                         32 * 128, ctypes.c_float(0.088), 16, ctypes.c_void_p(0), err, 256)
    assert rc == -5 and b"16 MiB" in err.value
