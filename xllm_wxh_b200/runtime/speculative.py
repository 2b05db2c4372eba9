"""Speculative decoding: MTP draft module or EAGLE-3 draft model (k >= 1: the draft is applied k times in a chain), or
suffix-pattern drafts (k >= 1, no draft model).

Flow follows the reference's speculative workers (xllm/core/runtime/speculative_worker_impl.cpp:85-96,
mtp_worker_impl.cpp:301-445,473-506,638-660,706-790, suffix_worker_impl.cpp; SpeculativeEngine shares the block
manager between target and draft, speculative_engine.cpp):

  prefill step : target forward -> first token; MTP forward on the same positions with the tokens shifted by one and the
                 target's hidden states -> first draft token of every sequence that finished its prompt.
  decode step  : every sequence contributes 1 + k rows [last token, draft_1..draft_k]; one target forward validates
                 them; the target's own samples at those rows decide acceptance (`xl_rejection_sample`); the scheduler
                 receives `[accepted drafts..., correction-or-bonus, -1...]` per sequence; for MTP the draft module then
                 re-runs on the same rows (tokens = what was emitted, hidden = target's) to repair its KV and to
                 propose the next draft ("draft extend").  With k > 1 the module then runs k - 1 more times on one row
                 per sequence (the token it just proposed, the hidden state it just produced, the next position), as the
                 reference's multi-step draft loop does (mtp_worker_impl.cpp:401-445); those rows write the draft's KV at
                 positions past the rows of the step, whose slots come from the sequence's block table (the scheduler
                 reserves `spec_extra_slots` for them).

Every rank of a TP/EP group runs the same device work; only rank 0 keeps the drafts (host dictionary by sequence id)
and writes them into the packed step buffer before it is published.  The acceptance-rate override of the reference
(env XLLM_FIX_SPECULATIVE_ACCEPTANCE_RATE) is honoured.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import numpy as np
import torch

from .. import _core, ops
from ..config import Options
from ..framework.step_input import StepInput
from .engine import CTRL_WORDS, LLMEngine
from .worker import StepResult


def _fixed_rate() -> float:
    v = os.environ.get("XLLM_FIX_SPECULATIVE_ACCEPTANCE_RATE", "")
    try:
        r = float(v)
        return r if 0.0 <= r <= 1.0 else -1.0
    except ValueError:
        return -1.0


def rejection_sample(target: torch.Tensor, draft: torch.Tensor, fixed_rate: float, seed: int):
    """target [B, k+1] int32, draft [B, k] int32 -> (out [B, k+1] with -1 padding, num_accepted [B]).

    `target` holds the target model's own token at every validated row (arg-max, or a sample for requests that sample);
    a draft is accepted where it equals that token, and the first row that differs emits the target's token instead.
    Every proposal here is a single token (the draft's arg-max), i.e. a draft distribution that is a point mass.  For
    such drafts this is the reference's rule (rejection_sampler.cpp:244-300): it accepts draft d with probability
    min(1, p_target(d) / p_draft(d)) = p_target(d) and otherwise draws from the target distribution with d removed;
    drawing x from p_target and accepting where x == d does exactly that, so the emitted tokens follow the target's
    distribution.  `fixed_rate` >= 0 replaces the comparison by a seeded coin (the reference's fixed acceptance rate for
    measurements, :56-84)."""
    B, k1 = target.shape
    k = k1 - 1
    if target.is_cuda:
        from ..ops import cuda_ops
        out = torch.empty_like(target)
        acc = torch.empty(B, dtype=torch.int32, device=target.device)
        cuda_ops._check(cuda_ops.lib().xl_rejection_sample(cuda_ops._ptr(target), cuda_ops._ptr(draft), cuda_ops._ptr(out),
                                                           cuda_ops._ptr(acc), B, k, cuda_ops.c_float(fixed_rate),
                                                           seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF, cuda_ops._stream()),
                        "xl_rejection_sample")
        cuda_ops.launch_count += 1
        return out, acc
    out = torch.full_like(target, -1)
    acc = torch.zeros(B, dtype=torch.int32)
    rng = np.random.default_rng(seed)
    for b in range(B):
        a = 0
        while a < k:
            ok = (rng.random() < fixed_rate) if fixed_rate >= 0 else (int(target[b, a]) == int(draft[b, a]))
            if not ok:
                break
            out[b, a] = draft[b, a]
            a += 1
        out[b, a] = target[b, a]
        acc[b] = a
    return out, acc


class SpeculativeEngine(LLMEngine):
    def __init__(self, options: Options, model_args=None, model=None, draft_model=None, **kw):
        super().__init__(options, model_args=model_args, model=model, **kw)
        self.k = options.num_speculative_tokens
        self.algo = options.speculative_algorithm.upper()
        assert self.k >= 1
        self.draft = None
        self.draft_kv = None
        if self.algo == "MTP":
            self.draft = draft_model if draft_model is not None else self._build_mtp()
            shapes = self.draft.kv_cache_shapes(self.num_blocks, self.block_size)
            self.draft_kv = [tuple(torch.zeros(s, dtype=self.draft.dtype, device=self.device) for s in layer) for layer in shapes]
            if self.host_tier is not None:
                # the draft module keeps its own KV under the same block ids: a block that leaves for the host tier (or
                # the shared store) and comes back under another id must bring the draft's part along
                from .host_kv_tier import HostKvTier
                old = self.host_tier
                old._put_q.put(None)                       # ends the store thread of the tier that is replaced
                self.host_tier = HostKvTier(list(self.worker.kv_caches) + list(self.draft_kv), old.num_host_blocks, self.device)
                if self.kv_store is not None:
                    from ..service.kv_store import model_namespace
                    name = (self.opt.model_id or os.path.basename(os.path.normpath(str(self.opt.model)))) + "+mtp"
                    self._store_ns = model_namespace(name, self.args, self.block_size, self.host_tier.stride,
                                                     getattr(self, "_store_fp", ""), self.opt.kv_cache_dtype)
                    self.host_tier.attach_store(self.kv_store, self.rank, self.world_size, self._store_ns)
        elif self.algo == "EAGLE3":
            # one-layer draft that reads the target's hidden states of three layers (eagle3_worker_impl.cpp:44-102)
            from ..models.eagle3 import default_capture_layers
            self.draft = draft_model if draft_model is not None else self._build_eagle3()
            target = self.worker.model
            if not hasattr(target, "capture_layers"):
                raise ValueError("the EAGLE-3 draft needs a target model that exposes its layer inputs (Qwen / Llama family)")
            target.capture_layers = getattr(self.draft, "capture_layers", None) or default_capture_layers(self.args.n_layers)
            shapes = self.draft.kv_cache_shapes(self.num_blocks, self.block_size)
            self.draft_kv = [tuple(torch.zeros(s, dtype=self.draft.dtype, device=self.device) for s in layer) for layer in shapes]
        elif self.algo == "SUFFIX":
            keep = options.speculative_suffix_max_cached_requests
            self.suffix = _core.SuffixCache(max(2, options.speculative_suffix_cache_max_depth), keep if keep > 0 else 8192)
            self._suffix_fed: Dict[int, int] = {}
        else:
            raise ValueError(f"speculative_algorithm {options.speculative_algorithm} is not supported (MTP | Eagle3 | Suffix)")
        self.drafts: Dict[int, List[int]] = {}          # sequence id -> k draft tokens (rank 0)
        self.fixed_rate = _fixed_rate()
        self.stat_draft_tokens = 0
        self.stat_accepted_tokens = 0

    def transfer_caches(self):
        """Prefill / decode hand-over: the draft module's KV of a block travels with the target's (same block ids), so the
        decode instance's drafts attend to the whole prompt from its first step."""
        return list(self.worker.kv_caches) + (list(self.draft_kv) if self.draft_kv is not None else [])

    def sleep(self, level: int = 1) -> bool:
        """The draft module's weights and KV are not part of the sleep bookkeeping: an engine with one stays awake."""
        if self.draft is not None:
            return False
        return super().sleep(level)

    def _build_mtp(self):
        from ..models.deepseek_impl import DeepseekMTP
        target = self.worker.model
        m = DeepseekMTP(self.args, self.comm, self.device, target.dtype, target=target)
        if self.opt.draft_model and os.path.isdir(self.opt.draft_model):
            from ..utils.safetensors_io import CheckpointReader
            m.load_weights(CheckpointReader(self.opt.draft_model))
        elif self.model_dir is not None:
            from ..utils.safetensors_io import CheckpointReader
            m.load_weights(CheckpointReader(self.model_dir))       # MTP layers live in the same checkpoint at layer n_layers
        else:
            m.init_random(self.opt.random_seed + 1)
        return m

    def _build_eagle3(self):
        from ..models.eagle3 import Eagle3Draft
        target = self.worker.model
        d = self.opt.draft_model
        if d and os.path.isdir(d):
            import json
            from ..models.args import load_model_args
            from ..utils.safetensors_io import CheckpointReader
            dargs = load_model_args(d)
            with open(os.path.join(d, "config.json")) as f:
                cfg = json.load(f)
            m = Eagle3Draft(dargs, self.comm, self.device, target.dtype, target=target,
                            draft_vocab_size=int(cfg.get("draft_vocab_size") or dargs.vocab_size))
            m.load_weights(CheckpointReader(d))
            ids = (cfg.get("eagle_config") or {}).get("eagle_aux_hidden_state_layer_ids")
            if ids:
                m.capture_layers = [int(i) for i in ids]
            return m
        return Eagle3Draft(self.args, self.comm, self.device, target.dtype, target=target).init_random(self.opt.random_seed + 1)

    def _propose(self, hidden: torch.Tensor, sample_idx) -> torch.Tensor:
        """Greedy proposal of the draft at the given rows, in target token ids."""
        if hasattr(self.draft, "propose"):
            return self.draft.propose(hidden, sample_idx)
        return self.draft.logits(hidden, sample_idx).argmax(-1).int()

    def _draft_state(self, hidden: torch.Tensor) -> torch.Tensor:
        """What the draft reads of the target's forward pass: the final hidden states (MTP) or the captured layer inputs."""
        return self.worker.model.aux_hidden if self.algo == "EAGLE3" else hidden

    # ------------------------------------------------------------------ rank-local execution
    @torch.inference_mode()
    def _run_local(self, msg: torch.Tensor, patch: bool, want_emb: int) -> Optional[StepResult]:
        ctrl = msg[:CTRL_WORDS].numpy()
        base = 4 + self.comm.dp_rank * 7
        off = int(ctrl[base])
        if off < 0 or want_emb:
            return super()._run_local(msg, patch, want_emb)
        self._host_tier_step(msg)                       # host-tier copies of the step run ahead of its forward
        w = self.worker
        impl = getattr(w.model, "moe_impl", None)
        if impl is not None:                            # rows every DP rank runs this step (expert-parallel exchange sizes)
            impl.dp_token_counts = [int(v) for v in ctrl[64:64 + max(1, self.opt.dp_size)]]
        T, B, MB, S, P, padded = (int(v) for v in ctrl[base + 1:base + 7])
        L = w.layout_for(T, B, MB, S, P)
        w._ensure_staging(L.total_words)
        host = msg[CTRL_WORDS + off:CTRL_WORDS + off + L.total_words]
        w.set_host(host)
        header = host[L.header:L.header + 32].numpy().copy()
        if w.is_cuda:
            w._dev[:L.total_words].copy_(host, non_blocking=True)
            w.h2d_bytes += L.total_words * 4
        inp = StepInput(w._dev, L, header, padded=False)
        batch_id = int(np.uint32(header[12])) | (int(np.uint32(header[13])) << 32)
        model = w.model
        hidden = model.forward(inp, w.kv_caches)
        logits = model.logits(hidden, inp.sample_idx)
        tokens, lp, _, _ = ops.sample(logits, inp)                  # target's own sample at every validated row
        k = inp.n_spec
        n_rows = inp.n_sample
        extra = None
        if k == 0:
            # ---- prefill: first draft from the MTP module
            out_tokens = tokens
            if self.draft is not None:
                # every chunk runs through the draft module (its KV cache must cover the whole prompt)
                nxt = inp.next_tokens.clone()
                if n_rows > 0:
                    nxt.index_copy_(0, inp.sample_idx.long(), tokens)    # the token sampled now follows the last prompt position
                nxt.clamp_(min=0)
                dh = self.draft.forward_mtp(_with_tokens(inp, nxt), self.draft_kv, self._draft_state(hidden))
                if n_rows > 0:
                    rows0 = inp.sample_idx.long()
                    extra = self._propose(dh, inp.sample_idx)
                    # the first draft sits two positions after the last prompt row
                    extra = self._chain_drafts(inp, rows0, extra, dh.index_select(0, rows0),
                                               inp.positions.index_select(0, rows0) + 1)
        else:
            # ---- decode: validate the drafts that rank 0 wrote into the token buffer
            Bn = n_rows // (k + 1)
            rows = inp.sample_idx.long().view(Bn, k + 1)
            draft = inp.tokens.index_select(0, rows[:, 1:].reshape(-1)).view(Bn, k).contiguous()
            out2, acc = rejection_sample(tokens.view(Bn, k + 1).contiguous(), draft, self.fixed_rate, batch_id)
            out_tokens = out2.reshape(-1)
            if self.draft is not None:
                nxt = torch.zeros_like(inp.tokens)
                nxt.index_copy_(0, inp.sample_idx.long(), out_tokens.clamp(min=0))
                dinp = _with_tokens(inp, nxt)
                dh = self.draft.forward_mtp(dinp, self.draft_kv, self._draft_state(hidden))
                cand = self._propose(dh, inp.sample_idx).view(Bn, k + 1)
                extra = cand.gather(1, acc.long().view(Bn, 1)).reshape(-1)      # proposal after the last emitted token
                last = rows.gather(1, acc.long().view(Bn, 1)).reshape(-1)       # row of the last emitted token
                extra = self._chain_drafts(inp, rows[:, 0], extra, dh.index_select(0, last),
                                           inp.positions.index_select(0, last) + 1)
        w._last_tokens = out_tokens
        slot = w._result_slot(max(n_rows, 1) * 2, 1, 0)
        slot["tokens"][:n_rows].copy_(out_tokens[:n_rows], non_blocking=True)
        n_extra = 0
        if extra is not None:
            n_extra = extra.numel()
            slot["tokens"][n_rows:n_rows + n_extra].copy_(extra, non_blocking=True)
        out_lp = None
        if lp is not None:
            slot["logprobs"][:n_rows].copy_(lp[:n_rows], non_blocking=True)
            out_lp = slot["logprobs"][:n_rows]
        w.d2h_bytes += (n_rows + n_extra) * 4
        ev = None
        if w.is_cuda:
            ev = torch.cuda.Event()
            ev.record()
        res = StepResult(batch_id, n_rows, 1, slot["tokens"][:n_rows + n_extra], out_lp, None, None, ev)
        res.n_extra = n_extra
        self._push_kv_pairs(msg)
        return res

    def _chain_drafts(self, inp: StepInput, seq_rows: torch.Tensor, first: torch.Tensor, hidden: torch.Tensor,
                      pos: torch.Tensor) -> torch.Tensor:
        """Drafts 2..k of every sampling sequence.  `first` [B] is draft 1, `hidden` [B, H] the draft module's state that
        produced it, `pos` [B] the position draft 1 will occupy, `seq_rows` [B] any row of each sequence in this step (it
        names the sequence).  Returns the k drafts of every sequence, flattened [B * k]."""
        k = self.k
        if k == 1:
            return first
        B = first.shape[0]
        seq = inp.token_seq.index_select(0, seq_rows).long()                 # index of each sequence in the step's tables
        bt = inp.block_tables.index_select(0, seq)
        bs = inp.block_size
        out = [first]
        tok, h = first, hidden
        arange = torch.arange(B + 1, dtype=torch.int32, device=first.device)
        for j in range(1, k):
            p = (pos + (j - 1)).long()
            slot = bt.gather(1, (p // bs).view(B, 1)).view(B).long() * bs + p % bs
            mini = _DraftRows(tok, p.int(), slot.int(), arange, (p + 1).int(), bt, bs, inp.layout.MB_cap, max_kv=inp.max_kv + j)
            h = self.draft.forward_mtp(mini, self.draft_kv, h)
            tok = self._propose(h, None)
            out.append(tok)
        return torch.stack(out, 1).reshape(-1)

    # ------------------------------------------------------------------ rank 0
    def _suffix_drafts(self, batch, i: int, seq_id: int) -> List[int]:
        # only what is new since the last step crosses into Python (plus the 32-token context of the lookup)
        n = batch.seq_num_tokens(i)
        fed = self._suffix_fed.get(seq_id, 0)
        if n > fed:
            self.suffix.append(seq_id, batch.seq_tokens_from(i, fed))
            self._suffix_fed[seq_id] = n
        o = self.opt
        d = self.suffix.speculate_scored(batch.seq_tokens_from(i, n - 32), self.k, o.speculative_suffix_max_spec_factor,
                                         o.speculative_suffix_max_spec_offset, o.speculative_suffix_min_token_prob)
        return (list(d) + [0] * self.k)[:self.k]

    def step(self):
        self.bind_thread()
        sch = self.scheduler
        batches = sch.schedule()
        b = batches[0]
        if all(x.empty for x in batches):
            return sch.take_outputs()
        assert self.opt.dp_size == 1, "speculative decoding runs with one attention-DP group"
        entries = b.entries()
        is_decode = b.num_spec > 0
        local = self._publish_spec(batches, entries, is_decode)
        local.wait()
        n_rows = local.n_sample
        toks = local.tokens[:n_rows].numpy()
        extra = local.tokens[n_rows:n_rows + getattr(local, "n_extra", 0)].numpy()
        lps = local.logprobs[:n_rows].numpy() if local.logprobs is not None else None
        if is_decode:
            k1 = self.k + 1
            out = toks.reshape(-1, k1)
            self.stat_draft_tokens += out.shape[0] * self.k
            self.stat_accepted_tokens += int((out >= 0).sum() - out.shape[0])
            sch.process_output(b.id, out, lps.reshape(-1, k1) if lps is not None else None)
        else:
            sch.process_output(b.id, toks, lps)
        # remember the next draft of every sequence that sampled this step
        j = 0
        for e in entries:
            if not e[4]:
                continue
            if self.draft is not None and (j + 1) * self.k <= len(extra):
                self.drafts[e[0]] = [int(t) for t in extra[j * self.k:(j + 1) * self.k]]
            j += 1
        self.step_count += 1
        outs = sch.take_outputs()
        for o in outs:                       # per-sequence draft state ends with the sequence
            if o.finished:
                self.drafts.pop(o.seq_id, None)
                if self.algo == "SUFFIX":
                    self._suffix_fed.pop(o.seq_id, None)
        return outs

    def _publish_spec(self, batches, entries, is_decode):
        """As `_publish`, with the drafts written into the packed token section of decode batches."""
        if not is_decode:
            return self._publish(batches, patch=False)
        b = batches[0]
        drafts: List[List[int]] = []
        for i, e in enumerate(entries):
            if self.algo == "SUFFIX":
                drafts.append(self._suffix_drafts(b, i, e[0]))
            else:
                drafts.append(self.drafts.get(e[0], [0] * self.k))

        def hook(engine, msg, L, off):
            host = msg[CTRL_WORDS + off:CTRL_WORDS + off + L.total_words].numpy()
            q_cu = host[L.q_cu:L.q_cu + len(entries) + 1]
            for i, d in enumerate(drafts):
                start = int(q_cu[i]) + 1
                host[L.tokens + start:L.tokens + start + self.k] = d
        self._pack_hook = hook
        try:
            return self._publish(batches, patch=False)
        finally:
            self._pack_hook = None

    def acceptance_rate(self) -> float:
        return self.stat_accepted_tokens / max(1, self.stat_draft_tokens)


class _RowsLayout:
    def __init__(self, mb_cap: int):
        self.MB_cap = mb_cap


class _DraftRows:
    """Step input of one decode-like row per sequence, built on the device from another step's block tables: what the
    draft module needs to run one more token of every sequence (tokens, positions, KV slots, lengths, block tables)."""

    def __init__(self, tokens, positions, slots, q_cu, kv_lens, block_tables, block_size, mb_cap, max_kv=0):
        B = tokens.shape[0]
        self.tokens, self.positions, self.slots = tokens, positions, slots
        self.q_cu, self.kv_lens, self.block_tables = q_cu, kv_lens, block_tables
        self.n_tokens = self.T = B
        self.n_seqs = self.B = self.n_decode = B
        self.n_prefill = self.n_prefill_tokens = 0
        self.max_q, self.max_kv = 1, max_kv          # an upper bound known on the host (the lengths live on the device)
        self.block_size = block_size
        self.padded = False
        self.has_prefill = False
        self.layout = _RowsLayout(mb_cap)
        self.token_seq = torch.arange(B, dtype=torch.int32, device=tokens.device)


class _TokenView:
    """A StepInput whose token ids are replaced (positions, slots, lengths, block tables shared)."""

    def __init__(self, inp: StepInput, tokens: torch.Tensor):
        self.__dict__.update(inp.__dict__)
        self.tokens = tokens


def _with_tokens(inp: StepInput, tokens: torch.Tensor):
    return _TokenView(inp, tokens)
