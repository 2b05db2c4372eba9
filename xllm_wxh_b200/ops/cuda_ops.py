"""ctypes bindings of `libxllm_kernels.so` (hand-written sm_100a kernels; sources in `csrc/cuda`).

Kernels are launched on PyTorch's current stream, so they are captured by `torch.cuda.graph` like any other
work.  A missing or failing library raises: there is no silent fallback to PyTorch on a CUDA device.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(os.path.dirname(_HERE), "libxllm_kernels.so")
_lib = None
launch_count = 0          # kernels launched through this module (reported by bench.py as `gpu_launches`)

c_void_p, c_int, c_long, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float


class _TimedLib:
    """Opt-in profiling aid (`XLLM_KERNEL_TIMING=1`): brackets every kernel entry point with a pair of CUDA events on
    the current stream and accumulates device time per entry point.  Off by default; the events add a few
    microseconds of host time per launch, so numbers taken with it on are for shares, not for reporting."""
    _PLAIN = ("xl_dev_malloc", "xl_dev_free", "xl_ipc_get_handle", "xl_ipc_open_handle", "xl_ipc_close_handle",
              "xl_read_status", "xl_sm_count", "xl_gemm_force_bn", "xl_reset_status", "xl_prefill_use_tc", "xl_gemm_set_mode", "xl_gemm_pair_force_bn", "xl_gemm_pair_splitk", "xl_prefill_kv_split")

    def __init__(self, real):
        self._real = real
        self._wrapped = {}
        self.records = []        # (name, start_event, stop_event)
        self.enabled = True

    def __getattr__(self, name):
        f = getattr(self._real, name)
        if name in self._PLAIN or not name.startswith("xl_"):
            return f
        w = self._wrapped.get(name)
        if w is None:
            def w(*a, _f=f, _n=name):
                if not self.enabled or torch.cuda.is_current_stream_capturing():
                    return _f(*a)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                rc = _f(*a)
                e1.record()
                self.records.append((_n, e0, e1))
                return rc
            self._wrapped[name] = w
        return w

    def reset(self):
        self.records = []

    def summary(self):
        """{entry point: (launches, total device ms)} since the last reset (synchronises the device)."""
        torch.cuda.synchronize()
        out = {}
        for n, e0, e1 in self.records:
            c, t = out.get(n, (0, 0.0))
            out[n] = (c + 1, t + e0.elapsed_time(e1))
        return out


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(f"{_LIB_PATH} is missing: run `python -m xllm_wxh_b200.build_ext` (needs nvcc)")
        real = ctypes.CDLL(_LIB_PATH)
        real.xl_read_status.restype = c_int
        real.xl_sm_count.restype = c_int
        _lib = _TimedLib(real) if os.environ.get("XLLM_KERNEL_TIMING") == "1" else real
    return _lib


def kernel_timing():
    """The `_TimedLib` when kernel timing is on, else None."""
    L = lib()
    return L if isinstance(L, _TimedLib) else None


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc: int, name: str):
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc} (-2: unsupported shape/alignment, -1: launch error)")


def read_status() -> int:
    """Device status word: non-zero when a bounded wait inside a kernel gave up (synchronises the device)."""
    return int(lib().xl_read_status())


def sm_count() -> int:
    return int(lib().xl_sm_count())


# ----------------------------------------------------------------------------- GEMM
def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    global launch_count
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "GEMM kernel is bf16"
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    M, K = x2.shape
    N = w.shape[0]
    assert w.shape[1] == K and w.stride(-1) == 1
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    if M > 0:
        rc = lib().xl_gemm_bf16(_ptr(x2), _ptr(w), _ptr(out), _ptr(bias), c_int(M), c_int(N), c_int(K), c_int(x2.stride(0)),
                                c_int(w.stride(0)), c_int(out.stride(0)), _stream())
        _check(rc, "xl_gemm_bf16")
        launch_count += 1
    return out.reshape(x.shape[:-1] + (N,))


def linear_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor) -> torch.Tensor:
    """gate_up GEMM with the SwiGLU epilogue; `w_interleaved` from `interleave_gate_up`."""
    global launch_count
    if x.stride(-1) != 1:
        x = x.contiguous()
    M, K = x.shape
    N = w_interleaved.shape[0]
    out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    if M > 0:
        rc = lib().xl_gemm_bf16_swiglu(_ptr(x), _ptr(w_interleaved), _ptr(out), c_int(M), c_int(N), c_int(K), c_int(x.stride(0)),
                                       c_int(w_interleaved.stride(0)), c_int(out.stride(0)), _stream())
        _check(rc, "xl_gemm_bf16_swiglu")
        launch_count += 1
    return out


def interleave_gate_up(w: torch.Tensor) -> torch.Tensor:
    """[2I, K] (gate rows then up rows) -> rows interleaved in groups of 16 (16 gate, 16 up, ...)."""
    I = w.shape[0] // 2
    assert I % 16 == 0
    g, u = w[:I].reshape(I // 16, 16, -1), w[I:].reshape(I // 16, 16, -1)
    return torch.stack([g, u], dim=1).reshape(2 * I, -1).contiguous()


def gemm_force_bn(bn: int):
    lib().xl_gemm_force_bn(c_int(bn))


def gemm_set_mode(mode: int):
    """0: choose per problem; 1: single-CTA tiles only; 2: CTA-pair (`cta_group::2`) tiles whenever M > 128."""
    lib().xl_gemm_set_mode(c_int(mode))


# ----------------------------------------------------------------------------- elementwise
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    global launch_count
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    out = torch.empty((x2.shape[0], shp[-1]), dtype=x.dtype, device=x.device)
    _check(lib().xl_rms_norm(_ptr(x2), _ptr(w), _ptr(out), c_int(x2.shape[0]), c_int(shp[-1]), c_int(x2.stride(0)), c_float(eps),
                             _stream()), "xl_rms_norm")
    launch_count += 1
    return out.reshape(shp)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    global launch_count
    T, H = x.shape
    assert residual.is_contiguous()
    if x.stride(-1) != 1:
        x = x.contiguous()
    out = torch.empty((T, H), dtype=x.dtype, device=x.device)
    res_out = torch.empty((T, H), dtype=x.dtype, device=x.device)
    _check(lib().xl_add_rms_norm(_ptr(x), _ptr(residual), _ptr(w), _ptr(out), _ptr(res_out), c_int(T), c_int(H),
                                 c_int(x.stride(0)), c_float(eps), _stream()), "xl_add_rms_norm")
    launch_count += 1
    return out, res_out


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    global launch_count
    T, I2 = x.shape
    out = torch.empty((T, I2 // 2), dtype=x.dtype, device=x.device)
    _check(lib().xl_silu_mul(_ptr(x), _ptr(out), c_int(T), c_int(I2 // 2), c_int(x.stride(0)), _stream()), "xl_silu_mul")
    launch_count += 1
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    global launch_count
    T = ids.numel()
    V, H = table.shape
    out = torch.empty((T, H), dtype=table.dtype, device=table.device)
    _check(lib().xl_embedding(_ptr(ids), _ptr(table), _ptr(out), c_int(T), c_int(H), c_int(V), _stream()), "xl_embedding")
    launch_count += 1
    return out


def rope_qknorm_kvwrite(qkv, positions, slots, cos_sin, q_w, k_w, eps, k_cache, v_cache, n_q, n_kv, head_dim):
    global launch_count
    T = qkv.shape[0]
    assert qkv.is_contiguous() and cos_sin.dtype == torch.float32 and cos_sin.shape[-1] == head_dim
    cache_slots = k_cache.shape[0] * k_cache.shape[1]
    _check(lib().xl_rope_qknorm_kvwrite(_ptr(qkv), _ptr(positions), _ptr(slots), _ptr(cos_sin), _ptr(q_w), _ptr(k_w),
                                        _ptr(k_cache), _ptr(v_cache), c_int(T), c_int(n_q), c_int(n_kv), c_int(head_dim),
                                        c_float(eps), c_long(cache_slots), _stream()), "xl_rope_qknorm_kvwrite")
    launch_count += 1
    return qkv[:, :n_q * head_dim]


# ----------------------------------------------------------------------------- attention
decode_kernel = "tma"     # "tma" | "cp_async" (the fallback kernel; selectable for tests and comparisons)


def prefill_use_tc(on: bool):
    """Prefill attention kernel choice: tcgen05 (default) or the mma.sync kernel (comparisons, tests)."""
    lib().xl_prefill_use_tc(c_int(int(on)))


def prefill_kv_split(mode: int):
    """Key-range split of the tcgen05 prefill kernel: 0 = never, 1 = automatic (default: when query tiles x heads leave
    SMs idle), 2..8 = that many splits (tests, measurements)."""
    lib().xl_prefill_kv_split(c_int(int(mode)))


def decode_splits(n_seqs: int, n_kv: int, max_kv: int) -> int:
    """Key-range splits of the decode kernel: fill the two CTAs each SM holds, but never spill into a second, partly
    filled wave (measured at 255 sequences x 1 KV head: one split 28 us, two 35 us)."""
    ctas = max(1, n_seqs * n_kv)
    want = (2 * sm_count()) // ctas
    by_len = max(1, max_kv // 512)
    return max(1, min(want, by_len, 16))


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, inp, scale: float, window: int = -1) -> torch.Tensor:
    """q [T, Hq, D] (may be a strided view of the qkv buffer).  Decode sequences (the leading `inp.n_decode` ones) go to the
    split-KV kernel, the rest to the prefill kernel.  In a padded step (CUDA-graph capture / replay) the launches are sized
    for the capacities of the layout and the kernels read the real decode / prefill split from the device-side header."""
    global launch_count
    from ..framework.step_input import H_NUM_DECODE, H_NUM_SEQS
    T, Hq, D = q.shape
    n_kv = k_cache.shape[2]
    block_size = k_cache.shape[1]
    L = inp.layout
    padded = inp.padded
    # padded rows belong to no sequence and are written by no kernel: keep them finite
    out = (torch.zeros if padded else torch.empty)((T, Hq * D), dtype=q.dtype, device=q.device)
    n_dec = inp.B if padded else inp.n_decode
    n_all = inp.B if padded else inp.n_seqs
    has_prefill = inp.has_prefill if padded else n_all > n_dec
    hdr = getattr(inp, "header_dev", None)       # only padded steps read it (rows built on the device carry none)
    dyn_dec = c_void_p(hdr.data_ptr() + 4 * H_NUM_DECODE) if padded else c_void_p(0)
    dyn_all = c_void_p(hdr.data_ptr() + 4 * H_NUM_SEQS) if padded else c_void_p(0)
    q_stride = q.stride(0)
    common = (_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(inp.q_cu), _ptr(inp.kv_lens), _ptr(inp.block_tables))
    if n_dec > 0:
        max_kv = (L.MB_cap * block_size) if padded else inp.max_kv
        splits = decode_splits(n_dec, n_kv, max_kv)
        po = pl = None
        if splits > 1:
            rows = n_dec * max(1, 16 // (Hq // n_kv)) if padded else T
            rows = max(rows, T)
            po = torch.empty((rows, Hq, splits, D), dtype=torch.float32, device=q.device)
            pl = torch.empty((rows, Hq, splits), dtype=torch.float32, device=q.device)
        rc = -3
        if decode_kernel != "cp_async":
            rc = lib().xl_decode_attention_tma_dyn(*common, c_int(0), c_int(n_dec), c_int(L.MB_cap), c_int(block_size),
                                                   c_int(k_cache.shape[0]), c_int(Hq), c_int(n_kv), c_int(D), c_int(q_stride),
                                                   c_float(scale), c_int(window), c_int(splits), _ptr(po), _ptr(pl), dyn_dec,
                                                   _stream())
            if rc == 0 and splits > 1:
                _check(lib().xl_decode_split_merge_dyn(_ptr(po), _ptr(pl), _ptr(out), _ptr(inp.q_cu), c_int(0), c_int(n_dec),
                                                       c_int(Hq), c_int(D), c_int(splits), c_long(po.shape[0]), dyn_dec,
                                                       _stream()), "xl_decode_split_merge")
        if rc == -3:        # shape not covered by the TMA kernel: per-lane cp.async kernel
            rc = lib().xl_paged_attention_dyn(*common, c_int(0), c_int(n_dec), c_int(L.MB_cap), c_int(block_size),
                                              c_int(k_cache.shape[0]), c_int(Hq), c_int(n_kv), c_int(D), c_int(q_stride),
                                              c_float(scale), c_int(window), c_int(1), c_int(0), c_int(splits), _ptr(po),
                                              _ptr(pl), c_void_p(0), dyn_dec, c_int(T), _stream())
        _check(rc, "decode attention")
        launch_count += 1 + (1 if splits > 1 else 0)
    if has_prefill:
        # q tiles of 64 rows: every sequence adds at most one partly filled tile
        tiles = (T + 63) // 64 + n_all if padded else (inp.n_prefill_tokens + 63) // 64 + (n_all - n_dec)
        lo = 0 if padded else n_dec
        _check(lib().xl_paged_attention_dyn(*common, c_int(lo), c_int(n_all), c_int(L.MB_cap), c_int(block_size),
                                            c_int(k_cache.shape[0]), c_int(Hq), c_int(n_kv), c_int(D), c_int(q_stride),
                                            c_float(scale), c_int(window), c_int(0), c_int(tiles), c_int(1), c_void_p(0),
                                            c_void_p(0), dyn_dec, dyn_all, c_int(T), _stream()), "xl_paged_attention(prefill)")
        launch_count += 1
    return out


# ----------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, inp):
    global launch_count
    S, V = logits.shape
    dt = 0 if logits.dtype == torch.float32 else 1
    assert logits.dtype in (torch.float32, torch.bfloat16) and logits.stride(-1) == 1
    if inp.any_penalty:
        _check(lib().xl_apply_penalties(_ptr(logits), c_int(dt), c_int(S), c_int(V), c_long(logits.stride(0)), _ptr(inp.pen_cu),
                                        _ptr(inp.pen_ids), _ptr(inp.pen_counts), _ptr(inp.rep_pen), _ptr(inp.freq_pen),
                                        _ptr(inp.pres_pen), _stream()), "xl_apply_penalties")
        launch_count += 1
    tokens = torch.empty(S, dtype=torch.int32, device=logits.device)
    lp = tv = ti = None
    n_top = 0
    if inp.any_logprobs:
        lp = torch.empty(S, dtype=torch.float32, device=logits.device)
        n_top = inp.max_top_logprobs
        if n_top > 0:
            tv = torch.empty((S, n_top), dtype=torch.float32, device=logits.device)
            ti = torch.empty((S, n_top), dtype=torch.int32, device=logits.device)
    _check(lib().xl_sample(_ptr(logits), c_int(dt), c_int(S), c_int(V), c_long(logits.stride(0)), _ptr(inp.temperature),
                           _ptr(inp.top_k), _ptr(inp.top_p), _ptr(inp.seed_lo), _ptr(inp.seed_hi), _ptr(tokens), _ptr(lp),
                           c_int(n_top), _ptr(tv), _ptr(ti), _stream()), "xl_sample")
    launch_count += 1
    return tokens, lp, tv, ti


def topk_candidates(logits: torch.Tensor, inp, id_offset: int, width: int):
    """Per-shard candidates of vocabulary-parallel sampling: the top_k largest logits of every row of this vocabulary
    slice (ties at the k-th included; the arg-max for greedy rows) as (values fp32 [S, width], global ids int32 [S, width],
    overflow flag int32 [1]); unused places hold -inf / -1."""
    global launch_count
    S, V = logits.shape
    dt = 0 if logits.dtype == torch.float32 else 1
    assert logits.dtype in (torch.float32, torch.bfloat16) and logits.stride(-1) == 1
    vals = torch.empty((S, width), dtype=torch.float32, device=logits.device)
    ids = torch.empty((S, width), dtype=torch.int32, device=logits.device)
    over = torch.zeros(1, dtype=torch.int32, device=logits.device)
    _check(lib().xl_topk_candidates(_ptr(logits), c_int(dt), c_int(S), c_int(V), c_long(logits.stride(0)), _ptr(inp.temperature),
                                    _ptr(inp.top_k), c_int(id_offset), c_int(width), _ptr(vals), _ptr(ids), _ptr(over), _stream()),
           "xl_topk_candidates")
    launch_count += 1
    return vals, ids, over


# ----------------------------------------------------------------------------- MoE
def moe_router(logits, top_k, scoring="softmax", renorm=True, bias=None, n_group=1, topk_group=1, route_scale=1.0):
    from . import moe_cuda
    return moe_cuda.moe_router(logits, top_k, scoring, renorm, bias, n_group, topk_group, route_scale)


def moe_experts(x, w13, w2, weights, ids, expert_offset=0, interleaved=False):
    from . import moe_cuda
    return moe_cuda.moe_experts(x, w13, w2, weights, ids, expert_offset, interleaved)


# ----------------------------------------------------------------------------- MLA
class _HeadTiles:
    """Tile table that treats the heads of a head-major [Hh, T, K] tensor as the groups of a grouped GEMM."""
    _cache = {}

    def __init__(self, Hh: int, T: int, device):
        per = (T + 127) // 128
        h = torch.arange(Hh, device=device, dtype=torch.int32).repeat_interleave(per)
        i = torch.arange(per, device=device, dtype=torch.int32).repeat(Hh)
        self.tile_expert = h.contiguous()
        self.tile_row0 = (h * T + i * 128).contiguous()
        self.tile_row_end = ((h + 1) * T).contiguous()
        self.max_tiles = Hh * per
        self.num_m_tiles = torch.tensor([self.max_tiles], dtype=torch.int32, device=device)

    @classmethod
    def get(cls, Hh, T, device):
        key = (Hh, T, str(device))
        t = cls._cache.get(key)
        if t is None:
            if len(cls._cache) > 256:
                cls._cache.clear()
            t = cls._cache[key] = cls(Hh, T, device)
        return t


def _w_kc_t(w_kc: torch.Tensor) -> torch.Tensor:
    """[Hh, nope, c] -> [Hh, c, nope] (the [N, K] weight layout of the absorb GEMM).  The transposed copy lives on the weight
    tensor itself, so it goes away with it: a table keyed by the data pointer would hand a later model, whose weights the
    allocator put at the same address, the previous model's copy."""
    try:
        version = w_kc._version          # changes when the weights are rewritten in place (wake-up from sleep)
    except RuntimeError:                 # a tensor made under inference mode keeps no version
        version = 0
    t = getattr(w_kc, "_xl_kc_t", None)
    if t is None or t.shape != (w_kc.shape[0], w_kc.shape[2], w_kc.shape[1]) or getattr(w_kc, "_xl_kc_version", -1) != version:
        t = w_kc.transpose(1, 2).contiguous()
        w_kc._xl_kc_t = t
        w_kc._xl_kc_version = version
    return t


def mla_prepare(q, kv_a, positions, slots, cos_sin, kv_norm_w, eps, cache, w_kc, nope, rope, kv_lora):
    """Returns head-major tensors (q_lat [Hh, T, kv_lora], q_pe [Hh, T, rope]) for `mla_attention`."""
    global launch_count
    from . import moe_cuda
    T, Hh, _ = q.shape
    q = q.contiguous()
    kv_a = kv_a.contiguous()
    q_nope = torch.empty((Hh, T, nope), dtype=q.dtype, device=q.device)
    q_pe = torch.empty((Hh, T, rope), dtype=q.dtype, device=q.device)
    slots_total = cache.shape[0] * cache.shape[1]
    _check(lib().xl_mla_prepare(_ptr(q), _ptr(kv_a), _ptr(positions), _ptr(slots), _ptr(cos_sin), _ptr(kv_norm_w), _ptr(cache),
                                _ptr(q_nope), _ptr(q_pe), c_int(T), c_int(Hh), c_int(nope), c_int(rope), c_int(kv_lora),
                                c_float(eps), c_long(slots_total), _stream()), "xl_mla_prepare")
    launch_count += 1
    tiles = _HeadTiles.get(Hh, T, q.device)
    q_lat = moe_cuda.grouped_gemm(q_nope.view(Hh * T, nope), _w_kc_t(w_kc), tiles)
    return q_lat.view(Hh, T, kv_lora), q_pe


def mla_attention(q_lat_hm, q_pe_hm, cache, inp, scale, kv_lora):
    """Head-major in and out.  The tcgen05 kernel serves head counts that divide 128 (XLLM_MLA_TC=0: the mma.sync kernel)."""
    global launch_count
    Hh, T, C = q_lat_hm.shape
    rope = q_pe_hm.shape[-1]
    out = torch.empty_like(q_lat_hm)
    L = inp.layout
    n_all = inp.B if inp.padded else inp.n_seqs
    common = (_ptr(inp.q_cu), _ptr(inp.kv_lens), _ptr(inp.block_tables), c_int(0), c_int(n_all), c_int(L.MB_cap),
              c_int(cache.shape[1]), c_long(cache.shape[0] * cache.shape[1]), c_int(Hh), c_int(T), c_int(C), c_int(rope), c_float(scale))
    if Hh <= 128 and 128 % Hh == 0 and os.environ.get("XLLM_MLA_TC", "1") != "0":
        tpt = 128 // Hh
        max_tiles = (T + n_all * (tpt - 1)) // tpt + 1
        rc = lib().xl_mla_attention_tc(_ptr(q_lat_hm), _ptr(q_pe_hm), _ptr(cache), _ptr(out), *common, c_int(max_tiles), _stream())
        if rc == 0:
            launch_count += 1
            return out
        if rc != -3:
            _check(rc, "xl_mla_attention_tc")
    max_tiles = T * (Hh // 16) + n_all * Hh
    _check(lib().xl_mla_attention(_ptr(q_lat_hm), _ptr(q_pe_hm), _ptr(cache), _ptr(out), *common, c_int(max_tiles), _stream()),
           "xl_mla_attention")
    launch_count += 1
    return out


def index_scores(q, w, keys, block_tables, token_seq, positions, S: int):
    """Lightning-indexer scores [T, S] (fp32; -inf at keys after the query): q [T, n_heads, 128] bf16, w [T, n_heads] fp32
    (softmax scale folded in), keys [blocks, block, 128] bf16 read through `block_tables` [B, max_blocks] of the
    sequence `token_seq[t]`, causal by `positions[t]`.  None where the kernel does not serve the shape."""
    global launch_count
    T, NH, D = q.shape
    if D != 128 or NH not in (16, 32, 64) or T > 65535 or keys.dtype != torch.bfloat16 or q.dtype != torch.bfloat16:
        return None
    q, w, block_tables = q.contiguous(), w.contiguous(), block_tables.contiguous()
    token_seq, positions = token_seq.contiguous(), positions.contiguous()
    assert w.dtype == torch.float32 and block_tables.dtype == torch.int32 and token_seq.dtype == torch.int32
    assert positions.dtype == torch.int32 and keys.is_contiguous() and token_seq.shape[0] >= T and positions.shape[0] >= T
    out = torch.empty((T, S), dtype=torch.float32, device=q.device)
    rc = lib().xl_index_scores(_ptr(q), _ptr(w), _ptr(keys), _ptr(block_tables), _ptr(token_seq), _ptr(positions), _ptr(out),
                               c_int(T), c_int(S), c_int(block_tables.shape[0]), c_int(block_tables.shape[1]),
                               c_int(keys.shape[1]), c_long(keys.shape[0] * keys.shape[1]), c_int(NH), c_int(D), _stream())
    if rc == -3:
        return None
    _check(rc, "xl_index_scores")
    launch_count += 1
    return out


_ARANGE: Dict[Tuple[int, str], torch.Tensor] = {}


def mla_attention_sparse(q_lat_hm, q_pe_hm, cache, sel, sel_len, scale, kv_lora):
    """Head-major in and out.  Every query token is its own one-row sequence whose block table is its row of `sel`
    (blocks of one slot) and whose length is `sel_len[t]`: the paged MLA kernel then gathers exactly the kept rows."""
    global launch_count
    Hh, T, C = q_lat_hm.shape
    rope = q_pe_hm.shape[-1]
    if Hh % 16:
        raise RuntimeError(f"sparse MLA attention needs a multiple of 16 heads per rank (got {Hh})")
    key = (T + 1, str(q_lat_hm.device))
    q_cu = _ARANGE.get(key)
    if q_cu is None:
        q_cu = torch.arange(T + 1, dtype=torch.int32, device=q_lat_hm.device)
        if not torch.cuda.is_current_stream_capturing():      # a tensor made inside a capture lives in the graph's pool
            _ARANGE[key] = q_cu
    sel = sel.contiguous()
    sel_len = sel_len.contiguous()
    assert sel.dtype == torch.int32 and sel_len.dtype == torch.int32 and sel.shape[0] == T and sel_len.shape[0] == T
    out = torch.empty_like(q_lat_hm)
    rc = lib().xl_mla_attention(_ptr(q_lat_hm), _ptr(q_pe_hm), _ptr(cache), _ptr(out), _ptr(q_cu), _ptr(sel_len), _ptr(sel), c_int(0),
                                c_int(T), c_int(sel.shape[1]), c_int(1), c_long(cache.shape[0] * cache.shape[1]), c_int(Hh), c_int(T),
                                c_int(C), c_int(rope), c_float(scale), c_int(T * (Hh // 16)), _stream())
    _check(rc, "xl_mla_attention (sparse)")
    launch_count += 1
    return out


def mla_v_up(o_lat_hm, w_vc):
    """o_lat head-major [Hh, T, c] x W_vc [Hh, v, c] -> [T, Hh * v]."""
    from . import moe_cuda
    Hh, T, C = o_lat_hm.shape
    v = w_vc.shape[1]
    out = torch.empty((T, Hh * v), dtype=o_lat_hm.dtype, device=o_lat_hm.device)
    tiles = _HeadTiles.get(Hh, T, o_lat_hm.device)
    moe_cuda.grouped_gemm(o_lat_hm.view(Hh * T, C), w_vc, tiles, out=out, c_rows_per_expert=T, c_col_stride=v)
    return out


# ----------------------------------------------------------------------------- fp8 block-scaled
def quant_act_1x128(x: torch.Tensor, gated: bool = False, rows_dev: Optional[torch.Tensor] = None):
    """bf16 [T, K] -> (e4m3 [T, K], fp32 scales [T, K/128]).  gated: x is [T, 2K] = [gate | up], quantises silu(gate) * up."""
    global launch_count
    T = x.shape[0]
    K = x.shape[1] // (2 if gated else 1)
    if x.stride(-1) != 1:
        x = x.contiguous()
    q = torch.empty((T, K), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((T, K // 128), dtype=torch.float32, device=x.device)
    _check(lib().xl_quant_act_1x128(_ptr(x), _ptr(q), _ptr(s), c_int(T), c_int(K), c_int(x.stride(0)), c_int(int(gated)),
                                    _ptr(rows_dev), _stream()), "xl_quant_act_1x128")
    launch_count += 1
    return q, s


def linear_fp8_block(x: torch.Tensor, wq: torch.Tensor, wscale: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
    global launch_count
    x2 = x.reshape(-1, x.shape[-1])
    M, K = x2.shape
    N = wq.shape[0]
    xq, xs = quant_act_1x128(x2)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    _check(lib().xl_gemm_fp8_block(_ptr(xq), _ptr(wq), _ptr(out), _ptr(xs), _ptr(wscale), c_int(M), c_int(N), c_int(K),
                                   c_int(out.stride(0)), _stream()), "xl_gemm_fp8_block")
    launch_count += 1
    return out.reshape(x.shape[:-1] + (N,))


def moe_experts_fp8(x, w13, w13_scale, w2, w2_scale, weights, ids, expert_offset=0):
    """Routed experts with fp8 block-scaled weights: sort -> gather -> quant -> grouped fp8 GEMM -> SwiGLU+quant ->
    grouped fp8 GEMM -> combine."""
    global launch_count
    from . import moe_cuda
    T, H = x.shape
    k = ids.shape[1]
    E, I2, _ = w13.shape
    r = moe_cuda.moe_sort(ids, expert_offset, E)
    xs = moe_cuda.gather_rows(x, r, k)
    R = xs.shape[0]
    xq, xsc = quant_act_1x128(xs, rows_dev=r.total_rows)
    h = torch.empty((R, I2), dtype=torch.bfloat16, device=x.device)
    L = lib()
    _check(L.xl_grouped_gemm_fp8_block(_ptr(xq), _ptr(w13), _ptr(h), _ptr(xsc), _ptr(w13_scale), c_int(R), c_int(I2), c_int(H),
                                       c_int(h.stride(0)), c_int(E), _ptr(r.tile_expert), _ptr(r.tile_row0), _ptr(r.tile_row_end),
                                       _ptr(r.num_m_tiles), c_int(r.max_tiles), _stream()), "xl_grouped_gemm_fp8_block(w13)")
    hq, hsc = quant_act_1x128(h, gated=True, rows_dev=r.total_rows)
    y = torch.empty((R, H), dtype=torch.bfloat16, device=x.device)
    _check(L.xl_grouped_gemm_fp8_block(_ptr(hq), _ptr(w2), _ptr(y), _ptr(hsc), _ptr(w2_scale), c_int(R), c_int(H), c_int(I2 // 2),
                                       c_int(y.stride(0)), c_int(E), _ptr(r.tile_expert), _ptr(r.tile_row0), _ptr(r.tile_row_end),
                                       _ptr(r.num_m_tiles), c_int(r.max_tiles), _stream()), "xl_grouped_gemm_fp8_block(w2)")
    launch_count += 2
    return moe_cuda.combine(y, r, weights, T)


# ----------------------------------------------------------------------------- fp8 with per-row / per-channel scales
def _fp8_rows_out(T: int, H: int, device):
    return (torch.empty((T, H), dtype=torch.float8_e4m3fn, device=device), torch.empty((T,), dtype=torch.float32, device=device))


def quant_rows_fp8(x: torch.Tensor):
    """bf16 [T, H] -> (e4m3 [T, H], fp32 [T]): one dynamic scale per row (token)."""
    global launch_count
    if x.stride(-1) != 1:
        x = x.contiguous()
    T, H = x.shape
    q, s = _fp8_rows_out(T, H, x.device)
    _check(lib().xl_quant_rows_fp8(_ptr(x), _ptr(q), _ptr(s), c_int(T), c_int(H), c_int(x.stride(0)), _stream()), "xl_quant_rows_fp8")
    launch_count += 1
    return q, s


def rms_norm_quant_fp8(x: torch.Tensor, w: torch.Tensor, eps: float):
    global launch_count
    if x.stride(-1) != 1:
        x = x.contiguous()
    T, H = x.shape
    q, s = _fp8_rows_out(T, H, x.device)
    _check(lib().xl_rms_norm_quant_fp8(_ptr(x), _ptr(w), _ptr(q), _ptr(s), c_int(T), c_int(H), c_int(x.stride(0)), c_float(eps),
                                       _stream()), "xl_rms_norm_quant_fp8")
    launch_count += 1
    return q, s


def add_rms_norm_quant_fp8(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float):
    """residual' = x + residual; returns (e4m3 RMSNorm(residual') * w, row scales, residual')."""
    global launch_count
    x, residual = x.contiguous(), residual.contiguous()
    T, H = x.shape
    q, s = _fp8_rows_out(T, H, x.device)
    res_out = torch.empty_like(residual)
    _check(lib().xl_add_rms_norm_quant_fp8(_ptr(x), _ptr(residual), _ptr(w), _ptr(q), _ptr(s), _ptr(res_out), c_int(T), c_int(H),
                                           c_float(eps), _stream()), "xl_add_rms_norm_quant_fp8")
    launch_count += 1
    return q, s, res_out


def linear_fp8_scaled(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, col_scale: Optional[torch.Tensor] = None,
                      tensor_scale: float = 1.0, bias: Optional[torch.Tensor] = None, swiglu: bool = False) -> torch.Tensor:
    """bf16 [M, N] = (xq wq^T) * xs[m] * tensor_scale * col_scale[n] (+ bias); `swiglu`: wq holds interleaved gate / up rows
    (as `interleave_gate_up` lays them out, `col_scale` in the same order) and the result is silu(gate) * up [M, N / 2]."""
    global launch_count
    M, K = xq.shape
    N = wq.shape[0]
    assert xq.dtype == torch.float8_e4m3fn and wq.dtype == torch.float8_e4m3fn and wq.shape[1] == K and xq.stride(-1) == 1
    out = torch.empty((M, N // 2 if swiglu else N), dtype=torch.bfloat16, device=xq.device)
    if M > 0:
        epi = 2 if swiglu else (1 if bias is not None else 0)
        assert not (swiglu and bias is not None)
        _check(lib().xl_gemm_fp8_scaled(c_int(epi), _ptr(xq), _ptr(wq), _ptr(out), _ptr(bias), _ptr(xs), _ptr(col_scale),
                                        c_float(tensor_scale), c_int(M), c_int(N), c_int(K), c_int(xq.stride(0)), c_int(wq.stride(0)),
                                        c_int(out.stride(0)), _stream()), "xl_gemm_fp8_scaled")
        launch_count += 1
    return out
