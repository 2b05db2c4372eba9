"""Embedding task: one prefill per prompt, last-token pooling + L2 norm (reference:
xllm/core/runtime/embed_worker_impl.cpp, models/llm/qwen3.h:238-247).  The same one-prefill pass also serves the
Qwen3-Reranker score (`mode=2`): the probability of "yes" against "no" at the position after the prompt
(api_service/qwen3_rerank_service_impl.cpp, framework/sampling/sampler.cpp:78-90 of the reference)."""
from __future__ import annotations

from typing import List

from .. import _core
from ..framework.params import RequestOutput, SequenceOutput, Status, Usage


def embed_prompts(master, prompts: List[str], mode: int = 1) -> List[RequestOutput]:
    eng = master.engine
    if max(1, eng.opt.dp_size) > 1:
        raise NotImplementedError("the embedding task runs on engines with one attention-DP rank")
    outs: List[RequestOutput] = []
    ids_list = [p if not isinstance(p, str) else master.tokenizer.encode(p) for p in prompts]
    sched = eng.scheduler
    st = _core.StopCriteria()
    st.max_tokens = 1
    pending = {}
    for i, ids in enumerate(ids_list):
        cid = eng.add_request(ids, None, st)
        pending[cid] = i
    results = [None] * len(prompts)
    # run prefill-only steps; the pooled vector of a sequence is taken at the step that finishes its prompt
    while sched.has_unfinished():
        batches = sched.schedule()
        b = batches[0]
        if b.empty:
            break
        local = eng._publish(batches, patch=False, want_emb=mode)
        import numpy as np
        toks = np.zeros(max(b.num_sample_rows, 1), dtype=np.int32)
        row = 0
        for e in b.entries():
            if e[4]:
                results[pending[e[1]]] = local.embeddings[row].tolist()
                row += 1
        sched.process_output(b.id, toks, None)
        sched.take_outputs()
    for i, ids in enumerate(ids_list):
        outs.append(RequestOutput(prompt=prompts[i] if isinstance(prompts[i], str) else None, prompt_token_ids=list(ids),
                                  status=Status(), finished=True, usage=Usage(len(ids), 0, len(ids)),
                                  outputs=[SequenceOutput(index=0, embeddings=results[i])]))
    return outs


def rerank_scores(master, prompts: List[str]) -> List[float]:
    """P("yes") against P("no") right after each prompt (query + document, as the caller formatted them)."""
    v = master.args.vocab_size
    no_id, yes_id = master.engine.worker.yes_no_ids
    if not (0 <= no_id < v and 0 <= yes_id < v):
        raise ValueError(f"rerank token ids ({no_id}, {yes_id}) are outside the vocabulary of {v} tokens")
    return [float(o.outputs[0].embeddings[0]) for o in embed_prompts(master, prompts, mode=2)]
