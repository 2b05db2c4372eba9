"""Per-step model inputs: typed views into the single packed int32 buffer produced by the C++
batch builder (`_core.Batch.build`).  The same object serves eager execution (views sliced to the
real sizes) and CUDA-graph replay (views sliced to the bucket capacities, contents refreshed by one
host->device copy).

Counterpart of the reference's `ModelInputParams` / `ForwardInput`
(xllm/core/framework/model/model_input_params.h:326-620, runtime/forward_params.h).
"""
from __future__ import annotations

import numpy as np
import torch

from .. import _core

H_NUM_TOKENS, H_NUM_SEQS, H_NUM_SAMPLE, H_NUM_DECODE, H_NUM_PREFILL, H_MAX_Q, H_MAX_KV, H_FWD_TYPE, H_NUM_SPEC = range(9)
H_T_CAP, H_B_CAP, H_MB_CAP, H_BATCH_LO, H_BATCH_HI, H_ANY_PENALTY, H_ALL_GREEDY, H_ANY_LOGPROBS, H_BLOCK_SIZE = range(9, 18)
H_PEN_TOTAL, H_S_CAP, H_MAX_TOP_LOGPROBS, H_NUM_PREFILL_TOKENS, H_MAX_TOP_K = range(18, 23)

FWD_PREFILL, FWD_CHUNKED_PREFILL, FWD_DECODE, FWD_MIXED, FWD_EMPTY = range(5)


class StepInput:
    """Views over `buf` (int32, on the compute device) laid out by `layout`."""

    def __init__(self, buf: torch.Tensor, layout: "_core.BatchLayout", header: np.ndarray, padded: bool = False):
        L = layout
        self.buf, self.layout, self.header = buf, L, header
        self.n_tokens = int(header[H_NUM_TOKENS])
        self.n_seqs = int(header[H_NUM_SEQS])
        self.n_sample = int(header[H_NUM_SAMPLE])
        self.n_decode = int(header[H_NUM_DECODE])
        self.n_prefill = int(header[H_NUM_PREFILL])
        self.max_q = int(header[H_MAX_Q])
        self.max_kv = int(header[H_MAX_KV])
        self.fwd_type = int(header[H_FWD_TYPE])
        self.n_spec = int(header[H_NUM_SPEC])
        self.block_size = int(header[H_BLOCK_SIZE])
        self.any_penalty = bool(header[H_ANY_PENALTY])
        self.all_greedy = bool(header[H_ALL_GREEDY])
        self.any_logprobs = bool(header[H_ANY_LOGPROBS])
        self.max_top_logprobs = int(header[H_MAX_TOP_LOGPROBS])
        self.n_prefill_tokens = int(header[H_NUM_PREFILL_TOKENS])
        self.max_top_k = int(header[H_MAX_TOP_K])        # over the rows that sample; 2^30 when one of them has no top-k
        self.padded = padded
        self.has_prefill = self.fwd_type != FWD_DECODE
        # rows the kernels run over
        self.T = L.T_cap if padded else self.n_tokens
        self.B = L.B_cap if padded else self.n_seqs
        self.S = L.S_cap if padded else self.n_sample
        T, B, S = self.T, self.B, self.S
        self.tokens = buf[L.tokens:L.tokens + T]
        self.positions = buf[L.positions:L.positions + T]
        self.slots = buf[L.slots:L.slots + T]
        self.token_seq = buf[L.token_seq:L.token_seq + T]
        self.next_tokens = buf[L.next_tokens:L.next_tokens + T]
        self.q_cu = buf[L.q_cu:L.q_cu + B + 1]
        self.kv_lens = buf[L.kv_lens:L.kv_lens + B]
        self.block_tables = buf[L.block_tables:L.block_tables + L.B_cap * L.MB_cap].view(L.B_cap, L.MB_cap)[:B]
        self.sample_idx = buf[L.sample_idx:L.sample_idx + S]
        f = lambda off: buf[off:off + S].view(torch.float32)
        self.temperature, self.top_p = f(L.temperature), f(L.top_p)
        self.top_k = buf[L.top_k:L.top_k + S]
        self.rep_pen, self.freq_pen, self.pres_pen = f(L.rep_pen), f(L.freq_pen), f(L.pres_pen)
        self.seed_lo = buf[L.seed_lo:L.seed_lo + S]
        self.seed_hi = buf[L.seed_hi:L.seed_hi + S]
        self.want_logprobs = buf[L.want_logprobs:L.want_logprobs + S]
        self.pen_cu = buf[L.pen_cu:L.pen_cu + S + 1]
        self.pen_ids = buf[L.pen_ids:L.pen_ids + L.P_cap]
        self.pen_counts = buf[L.pen_counts:L.pen_counts + L.P_cap]
        self.header_dev = buf[L.header:L.header + 32]

    @property
    def is_decode_only(self) -> bool:
        return self.fwd_type == FWD_DECODE


def make_layout(T_cap: int, B_cap: int, MB_cap: int, S_cap: int, P_cap: int = 0) -> "_core.BatchLayout":
    return _core.BatchLayout(max(T_cap, 1), max(B_cap, 1), max(MB_cap, 1), max(S_cap, 1), max(P_cap, 32))
