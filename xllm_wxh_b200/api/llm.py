"""Offline Python API: `LLM`, `Embedding`, `ArgumentParser`.

Same surface as the reference's pybind layer (xllm/pybind/llm.py:86-485, embedding.py, args.py:4-49;
examples/generate.py, generate_beam_search.py, generate_embedding.py): construct with a model path
and device list, call `generate(prompts, sampling_params)` and read `output.outputs[i].text`,
`finish()` releases the workers.
"""
from __future__ import annotations

import argparse
import dataclasses
import math
from typing import Any, Dict, List, Optional, Sequence, Union

from ..config import Options
from ..framework.params import (BeamSearchParams, PoolingParams, RequestOutput, RequestParams, SamplingParams, SequenceOutput,
                                Status, StatusCode, Usage, to_request_params)
from ..runtime.engine import LLMEngine
from ..runtime.master import LLMMaster


class ArgumentParser:
    """`ArgumentParser().parse_args()` -> namespace usable as `LLM(**vars(ns))` (pybind/args.py:4-49)."""

    def __init__(self):
        p = argparse.ArgumentParser()
        p.add_argument("--model", type=str, required=True)
        p.add_argument("--runner", type=str, choices=["pooling"], default=None)
        p.add_argument("--devices", type=str, default="auto")
        p.add_argument("--draft_model", type=str, default=None)
        p.add_argument("--draft_devices", type=str, default=None)
        p.add_argument("--block_size", type=int, default=128)
        p.add_argument("--max_cache_size", type=int, default=0)
        p.add_argument("--max_memory_utilization", type=float, default=0.9)
        p.add_argument("--disable_prefix_cache", action="store_true")
        p.add_argument("--max_tokens_per_batch", type=int, default=20480)
        p.add_argument("--max_seqs_per_batch", type=int, default=256)
        p.add_argument("--max_tokens_per_chunk_for_prefill", type=int, default=-1)
        p.add_argument("--num_speculative_tokens", type=int, default=0)
        p.add_argument("--num_request_handling_threads", type=int, default=4)
        p.add_argument("--communication_backend", type=str, default="fused")
        p.add_argument("--expert_parallel_degree", type=int, default=0)
        p.add_argument("--disable_chunked_prefill", action="store_true")
        p.add_argument("--enable_prefill_sp", action="store_true")
        p.add_argument("--instance_role", type=str, default="DEFAULT")
        p.add_argument("--nnodes", type=int, default=1)
        p.add_argument("--node_rank", type=int, default=0)
        p.add_argument("--dp_size", type=int, default=1)
        p.add_argument("--ep_size", type=int, default=1)
        p.add_argument("--enable_disagg_pd", action="store_true")
        p.add_argument("--enable_schedule_overlap", action="store_true")
        p.add_argument("--kv_cache_transfer_mode", type=str, default="PUSH")
        p.add_argument("--enable_shm", action="store_true")
        p.add_argument("--task", type=str, default="generate")
        # accepted for scripts written against the reference's parser (pybind/args.py); no counterpart on this backend
        p.add_argument("--rank_tablefile", type=str, default="")
        p.add_argument("--master_node_addr", type=str, default="127.0.0.1:19888")
        p.add_argument("--device_ip", type=str, default="")
        p.add_argument("--transfer_listen_port", type=int, default=26000)
        p.add_argument("--instance_name", type=str, default="")
        p.add_argument("--enable_pd_ooc", action="store_true")
        p.add_argument("--enable_multi_stream_parallel", action="store_true")
        p.add_argument("--disable_ttft_profiling", action="store_true")
        p.add_argument("--enable_forward_interruption", action="store_true")
        p.add_argument("--input_shm_size", type=int, default=1024)
        p.add_argument("--output_shm_size", type=int, default=128)
        p.add_argument("--kv_cache_dtype", type=str, default="auto")
        self._parser = self.parser = p

    def add_argument(self, *a, **kw):
        return self._parser.add_argument(*a, **kw)

    def parse_args(self, args=None):
        return self._parser.parse_args(args)


def _options_from_kwargs(model: str, task: str, devices: str, kw: Dict[str, Any]) -> Options:
    o = Options(model=model, task=task, devices=devices)
    rename = {"disable_prefix_cache": ("enable_prefix_cache", lambda v: not v),
              "disable_chunked_prefill": ("enable_chunked_prefill", lambda v: not v)}
    names = {f.name for f in dataclasses.fields(Options)}
    for k, v in kw.items():
        if v is None:
            continue
        if k in rename:
            setattr(o, rename[k][0], rename[k][1](v))
        elif k in names:
            setattr(o, k, v)
        elif k == "communication_backend":
            o.communication_backend = "nccl" if v == "nccl" else "fused"
        # unknown / backend-specific keywords of the reference signature (rank_tablefile, device_ip, ...) are accepted
    if o.communication_backend not in ("fused", "nccl"):
        o.communication_backend = "fused"
    return o.validate()


def build_sample_jobs(tok, prompts: List[str], selectors: List[Any]):
    """For `LLM.sample` / `/v1/sample`: [(prompt index, hit index, token prefix ending with the selector)], hits per prompt."""
    jobs, hits_per_prompt = [], []
    for i, (pr, sel) in enumerate(zip(prompts, selectors)):
        value = sel["value"] if isinstance(sel, dict) else sel
        sel_ids = tok.encode(value, add_special_tokens=False)
        if len(sel_ids) != 1:
            raise ValueError("Failed to build sample slots. selector.value must be a stable single special token.")
        ids = tok.encode(pr, add_special_tokens=True)
        hits = [j for j, t in enumerate(ids) if t == sel_ids[0]]
        hits_per_prompt.append(len(hits))
        for h, j in enumerate(hits):
            jobs.append((i, h, ids[:j + 1]))
    return jobs, hits_per_prompt


class BeamSearchOutput:
    """Result of `LLM.beam_search` for one prompt: the beams, best first, in `sequences` (pybind/llm.py:62-68)."""

    def __init__(self, output: RequestOutput):
        self.prompt = output.prompt
        self.sequences = output.outputs
        self.outputs = output.outputs
        self.status = output.status
        self.usage = output.usage
        self.finished = output.finished
        self.prompt_token_ids = output.prompt_token_ids
        self.request_output = output


class EmbeddingOutputs:
    def __init__(self, output: RequestOutput):
        embedding = output.outputs[0].embeddings if output.outputs else []
        self.embedding = embedding
        self.embeddings = embedding

    # older callers of this package indexed the list of sequence outputs
    def __getitem__(self, i):
        if i != 0:
            raise IndexError(i)
        return self

    def __len__(self):
        return 1


class EmbeddingOutput:
    """Result of `LLM.embed` for one prompt: `outputs.embedding` is the pooled vector (pybind/llm.py:71-83)."""

    def __init__(self, output: RequestOutput):
        self.prompt = output.prompt
        self.outputs = EmbeddingOutputs(output)
        self.status = output.status
        self.usage = output.usage
        self.finished = output.finished
        self.prompt_token_ids = output.prompt_token_ids
        self.request_output = output


class LLM:
    def __init__(self, model: str, task: str = "generate", runner: Optional[str] = None, devices: str = "auto",
                 draft_model: Optional[str] = None, draft_devices: Optional[str] = None, block_size: int = 128,
                 max_cache_size: int = 0, max_memory_utilization: float = 0.9, disable_prefix_cache: bool = False,
                 max_tokens_per_batch: int = 20480, max_seqs_per_batch: int = 256,
                 max_tokens_per_chunk_for_prefill: int = -1, num_speculative_tokens: int = 0,
                 num_request_handling_threads: int = 4, communication_backend: str = "fused",
                 expert_parallel_degree: int = 0, disable_chunked_prefill: bool = False, enable_prefill_sp: bool = False,
                 instance_role: str = "DEFAULT", nnodes: int = 1, node_rank: int = 0, dp_size: int = 1, ep_size: int = 1,
                 instance_name: str = "", enable_disagg_pd: bool = False, enable_schedule_overlap: bool = False,
                 kv_cache_transfer_mode: str = "PUSH", enable_shm: bool = False, **kwargs: Any) -> None:
        if runner is not None:
            task = {"generate": "generate", "pooling": "embed"}.get(runner, task)
        kw = dict(draft_model=draft_model, draft_devices=draft_devices, block_size=block_size, max_cache_size=max_cache_size,
                  max_memory_utilization=max_memory_utilization, disable_prefix_cache=disable_prefix_cache,
                  max_tokens_per_batch=max_tokens_per_batch, max_seqs_per_batch=max_seqs_per_batch,
                  max_tokens_per_chunk_for_prefill=max_tokens_per_chunk_for_prefill,
                  num_speculative_tokens=num_speculative_tokens, num_request_handling_threads=num_request_handling_threads,
                  communication_backend=communication_backend, expert_parallel_degree=expert_parallel_degree,
                  disable_chunked_prefill=disable_chunked_prefill, enable_prefill_sp=enable_prefill_sp,
                  instance_role=instance_role, nnodes=nnodes, node_rank=node_rank, dp_size=dp_size, ep_size=ep_size,
                  instance_name=instance_name, enable_disagg_pd=enable_disagg_pd,
                  enable_schedule_overlap=enable_schedule_overlap, kv_cache_transfer_mode=kv_cache_transfer_mode,
                  enable_shm=enable_shm)
        kw.update(kwargs)
        engine = kw.pop("engine", None)
        tokenizer = kw.pop("tokenizer", None)
        self.options = _options_from_kwargs(model, task, devices, kw)
        self._procs = []
        if engine is None:
            from ..runtime.launcher import launch_engine
            engine, self._procs = launch_engine(self.options)
        self.master = LLMMaster(self.options, engine, tokenizer)
        self.engine = self.master.engine

    # ------------------------------------------------------------------ generate
    def generate(self, prompts: Union[str, List[str], Dict, List[Dict], List[List[int]]],
                 sampling_params=None, wait_schedule_done: bool = True) -> List[RequestOutput]:
        single = isinstance(prompts, (str, dict)) or (isinstance(prompts, list) and prompts and isinstance(prompts[0], int))
        plist = [prompts] if single else list(prompts)
        if isinstance(sampling_params, list):
            if len(sampling_params) != len(plist):
                raise ValueError("the number of sampling params must match the number of prompts")
            params = [to_request_params(p) for p in sampling_params]
        else:
            params = [to_request_params(sampling_params) for _ in plist]
        outputs: List[Optional[RequestOutput]] = [None] * len(plist)

        def make_cb(i):
            def cb(out: RequestOutput) -> bool:
                if out.finished:
                    outputs[i] = out
                return True
            return cb

        for i, (pr, rp) in enumerate(zip(plist, params)):
            rp.streaming = False
            if isinstance(pr, dict):                                  # vLLM-style {"prompt": ...} / {"prompt_token_ids": ...}
                pr = pr.get("prompt_token_ids") or pr.get("prompt")
            if rp.beam_width > 1:
                outputs[i] = self._beam_search_one(pr, rp)
                continue
            self.master.handle_request(pr, rp, make_cb(i), asynchronous=False)
        self.master.generate(getattr(self, "generate_timeout_s", 3600.0))
        for i, o in enumerate(outputs):
            if o is None:
                outputs[i] = RequestOutput(status=Status(StatusCode.UNKNOWN, "request produced no output"), finished=True)
        return outputs  # type: ignore[return-value]

    def beam_search(self, prompts, params: Optional[BeamSearchParams] = None) -> List[BeamSearchOutput]:
        """`prompts`: strings, token-id lists or `{"prompt": ...}` / `{"prompt_token_ids": ...}` dictionaries."""
        params = params or BeamSearchParams(beam_width=4)
        single = isinstance(prompts, (str, dict)) or (isinstance(prompts, list) and prompts and isinstance(prompts[0], int))
        plist = [prompts] if single else list(prompts)
        outs = []
        for p in plist:
            if isinstance(p, dict):
                p = p.get("prompt_token_ids") or p.get("prompt")
            outs.append(BeamSearchOutput(self._beam_search_one(p, to_request_params(params))))
        return outs

    def _beam_search_one(self, prompt, rp: RequestParams) -> RequestOutput:
        """Beam search driven from the API: each round extends every live beam by one token and keeps the
        `beam_width` best continuations by cumulative log-probability (reference: BeamSearcher,
        framework/sampling/beam_searcher.cpp; examples/generate_beam_search.py).  Beams share their prefix KV
        through the prefix cache."""
        tok = self.master.tokenizer
        ids = list(prompt) if not isinstance(prompt, str) else tok.encode(prompt)
        W = rp.beam_width
        eos = self.master._eos()
        beams = [(0.0, [])]              # (cumulative logprob, generated ids)
        done: List = []
        for _ in range(rp.max_tokens):
            cands = []
            outs = [None] * len(beams)
            for bi, (score, gen) in enumerate(beams):
                p = RequestParams(max_tokens=1, temperature=0.0, logprobs=True, top_logprobs=W, ignore_eos=True)
                def cb(out, bi=bi):
                    if out.finished:
                        outs[bi] = out
                    return True
                self.master.handle_request(ids + gen, p, cb, asynchronous=False)
            self.master.generate(getattr(self, "generate_timeout_s", 3600.0))
            for (score, gen), out in zip(beams, outs):
                lps = out.outputs[0].logprobs if out and out.outputs else None
                if not lps:
                    continue
                lp = lps[0]
                if lp.top_logprobs:
                    for t in lp.top_logprobs:
                        cands.append((score + t.logprob, gen + [t.token_id]))
                else:
                    cands.append((score + lp.logprob, gen + [lp.token_id]))
            cands.sort(key=lambda c: -c[0])
            beams = []
            for sc, g in cands:
                if g[-1] == eos and not rp.ignore_eos:
                    done.append((sc, g))
                else:
                    beams.append((sc, g))
                if len(beams) >= W:
                    break
            if len(done) >= W or not beams:
                break
        done.extend(beams)
        done.sort(key=lambda c: -c[0])
        outs = [SequenceOutput(index=i, text=tok.decode(g, rp.skip_special_tokens), token_ids=g,
                               finish_reason="stop" if g and g[-1] == eos else "length", cumulative_logprob=sc)
                for i, (sc, g) in enumerate(done[:W])]
        gen_total = sum(len(o.token_ids) for o in outs)
        return RequestOutput(prompt=prompt if isinstance(prompt, str) else None, prompt_token_ids=ids, status=Status(),
                             outputs=outs, usage=Usage(len(ids), gen_total, len(ids) + gen_total), finished=True)

    # ------------------------------------------------------------------ embeddings
    # ------------------------------------------------------------------ sample
    def sample(self, prompts: Union[str, List[str]], selector, request_params=None, logprobs: int = 5,
               wait_schedule_done: bool = True) -> List[RequestOutput]:
        """Next-token distribution at every position of a prompt that holds the `selector` token (reference:
        xllm/pybind/llm.py:413-485, examples/sample.py, `/v1/sample`).  One RequestOutput per prompt; its `outputs` hold one
        entry per selector hit, in prompt order, each with the sampled token and its `logprobs` alternatives.

        The reference marks the positions as "sample slots" of one prefill; here every hit becomes a one-token request over
        the prompt prefix that ends with the selector, and the prefix cache makes the hits of one prompt share their KV."""
        plist = [prompts] if isinstance(prompts, str) else list(prompts)
        if not plist:
            return []
        sels = [selector] * len(plist) if isinstance(selector, (str, dict)) else list(selector)
        if len(sels) != len(plist):
            raise ValueError("the number of selectors must match the number of prompts")
        if request_params is None:
            rps = [RequestParams() for _ in plist]
        elif isinstance(request_params, RequestParams):
            rps = [dataclasses.replace(request_params) for _ in plist]
        else:
            rps = list(request_params)
            if len({id(r) for r in rps}) != len(rps):
                raise ValueError("request_params contains duplicated RequestParams objects; create one per prompt")
        jobs, hits_per_prompt = build_sample_jobs(self.master.tokenizer, plist, sels)
        results: Dict[tuple, RequestOutput] = {}

        def make_cb(key):
            def cb(out: RequestOutput) -> bool:
                if out.finished:
                    results[key] = out
                return True
            return cb

        for i, h, prefix in jobs:
            rp = dataclasses.replace(rps[i])
            rp.max_tokens, rp.n, rp.best_of = 1, 1, 1
            rp.logprobs, rp.top_logprobs = True, int(logprobs)
            rp.streaming, rp.ignore_eos = False, True
            self.master.handle_request(prefix, rp, make_cb((i, h)), asynchronous=False)
        self.master.generate(getattr(self, "generate_timeout_s", 3600.0))
        outs: List[RequestOutput] = []
        for i, pr in enumerate(plist):
            o = RequestOutput(prompt=pr, finished=True, outputs=[])
            for h in range(hits_per_prompt[i]):
                r = results.get((i, h))
                if r is None or (r.status is not None and not r.status.ok):
                    raise RuntimeError(f"sample request failed: {r.status.message if r is not None and r.status else 'no output'}")
                so = r.outputs[0]
                so.index = h
                o.outputs.append(so)
                o.usage = r.usage
            outs.append(o)
        return outs

    def embed(self, prompts: Union[str, List[str]], pooling_params=None) -> List[EmbeddingOutput]:
        from ..runtime.embed import embed_prompts
        single = isinstance(prompts, (str, dict))
        plist = [prompts] if single else list(prompts)
        plist = [(p.get("prompt_token_ids") or p.get("prompt")) if isinstance(p, dict) else p for p in plist]
        return [EmbeddingOutput(o) for o in embed_prompts(self.master, plist)]

    def finish(self):
        self.master.stop()
        for p in self._procs:
            try:
                p.wait(timeout=10)
            except Exception:
                p.kill()
        self._procs = []

    def __del__(self):
        try:
            if getattr(self, "_procs", None):
                self.finish()
        except Exception:
            pass


class Embedding(LLM):
    """`Embedding(model, devices).embedding(prompts)` (pybind/embedding.py)."""

    def __init__(self, model: str, devices: str = "auto", **kwargs: Any):
        kwargs.pop("task", None)            # `Embedding(**vars(ArgumentParser().parse_args()))` carries the parser's default
        kwargs.pop("runner", None)
        super().__init__(model, task="embed", devices=devices, **kwargs)

    def embedding(self, prompts, pooling_params=None):
        return self.embed(prompts, pooling_params)
