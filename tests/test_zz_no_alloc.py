"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the kernel library may not allocate device memory where they call it (they run under another
framework's memory plan, or next to a CUDA-graph capture that forbids allocator traffic).  For them the library
exports `xl_decode_attention_noalloc`, which keeps its split-KV workspace in a device array compiled into the library.
This test checks, on two calls in a row (the second one reuses whatever the first left in the workspace), that it
returns what the regular entry point returns, and that an oversized request is refused with a message.
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


def test_noalloc_entry_point_matches_regular_one():
    from xllm_wxh_b200.ops import cuda_ops
    lib = cuda_ops.lib()
    for seed, n_seqs, kv_max, splits in [(1, 24, 3000, 4), (2, 7, 900, 2)]:       # two calls in a row share the workspace
        got, want = _call_both(lib, _case(seed, n_seqs, kv_max), splits)
        err = (got.float() - want.float()).abs()
        assert float(err.max()) <= 2e-2 + 2e-2 * float(want.float().abs().max()), float(err.max())
    assert cuda_ops.read_status() == 0


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
