"""OpenAI-compatible and Anthropic-compatible HTTP API on top of `LLMMaster`.

Endpoints (the reference's REST mappings, xllm/server/xllm_server.cpp:41-54; service logic api_service/*.cpp):
  POST /v1/completions, /v1/chat/completions, /v1/embeddings, /v1/messages (Anthropic), /v1/rerank
  GET  /v1/models, /v2/repository/index, /health, /metrics, /version
  POST /sleep, /wakeup (release / restore device memory of an idle instance)
  POST /fork_master (a second model on the same device, served under its own model id; the models take turns by sleep / wake-up)
  POST /link_d2d, /unlink_d2d (sessions to the weight services of awake instances; /wakeup {"remote_addrs": [...]} copies
       a deep sleeper's weights from one of them instead of reading the checkpoint)
Streaming answers are server-sent events (`data: {...}\\n\\n`, terminated by `data: [DONE]`), with
`delta.content | delta.reasoning_content | delta.tool_calls` for chat (chat_service_impl.cpp:74-155) and the Anthropic
event sequence for `/v1/messages`.  A rate limiter answers 429 above `--max_concurrent_requests`
(core/common/rate_limiter.cpp).  A client that disconnects cancels its request.
"""
from __future__ import annotations

import asyncio
import collections
import json
import threading
import time
import uuid
from typing import Any, Dict, List, Optional

from ..framework.params import RequestOutput, RequestParams, StatusCode
from ..runtime.master import LLMMaster
from ..utils.health import HEALTH
from ..utils.metrics import METRICS
from .function_call import StreamingToolParser, parse_tool_calls, resolve_parser
from .reasoning_parser import ReasoningParser, resolve_reasoning_parser
from .server import HttpServer, Request, Response, StreamingResponse

_HTTP_OF = {StatusCode.INVALID_ARGUMENT: 400, StatusCode.RESOURCE_EXHAUSTED: 503, StatusCode.UNAVAILABLE: 503,
            StatusCode.CANCELLED: 499, StatusCode.DEADLINE_EXCEEDED: 504, StatusCode.UNKNOWN: 500}


class RateLimiter:
    """Concurrent-request bound; also the gate of the sleep state: an instance may only fall asleep with no request in
    flight, and admits none until it is woken (rate_limiter.cpp:61-73 of the reference)."""

    def __init__(self, max_concurrent: int):
        self.max, self.cur, self.lock = max_concurrent, 0, threading.Lock()
        self.sleeping = False

    def try_set_sleeping(self) -> bool:
        with self.lock:
            if self.cur != 0 or self.sleeping:
                return False
            self.sleeping = True
            return True

    def try_wakeup(self) -> bool:
        with self.lock:
            if not self.sleeping:
                return False
            self.sleeping = False
            return True

    def acquire(self) -> bool:
        with self.lock:
            if self.sleeping:
                return False
            if self.max > 0 and self.cur >= self.max:
                return False
            self.cur += 1
            METRICS.set("num_concurrent_requests", self.cur)
            return True

    def release(self):
        with self.lock:
            self.cur = max(0, self.cur - 1)
            METRICS.set("num_concurrent_requests", self.cur)


def _err(message: str, status: int = 400, etype: str = "invalid_request_error") -> Response:
    return Response({"error": {"message": message, "type": etype, "code": status}}, status)


def params_from_body(body: Dict[str, Any], chat: bool) -> RequestParams:
    """completion.proto:10-121 / chat.proto:30-146 fields -> RequestParams."""
    p = RequestParams()
    g = body.get
    p.request_id = g("request_id") or ""
    p.service_request_id = g("service_request_id") or ""
    mt = g("max_completion_tokens", g("max_tokens"))
    if mt is not None:
        p.max_tokens = int(mt)
    for k in ("temperature", "top_p", "frequency_penalty", "presence_penalty", "repetition_penalty"):
        if g(k) is not None:
            setattr(p, k, float(g(k)))
    if g("top_k") is not None:
        p.top_k = int(g("top_k"))
    p.n = int(g("n") or 1)
    if g("best_of") is not None:
        p.best_of = int(g("best_of"))
    p.echo = bool(g("echo", False))
    p.streaming = bool(g("stream", False))
    p.include_usage = bool((g("stream_options") or {}).get("include_usage", False))
    stop = g("stop")
    if stop:
        p.stop = [stop] if isinstance(stop, str) else list(stop)
    if g("stop_token_ids"):
        p.stop_token_ids = [int(x) for x in g("stop_token_ids")]
    p.skip_special_tokens = bool(g("skip_special_tokens", True))
    p.ignore_eos = bool(g("ignore_eos", False))
    if g("seed") is not None:
        p.seed = int(g("seed"))
    p.offline = bool(g("offline", False))
    if g("priority") is not None:
        p.priority = int(g("priority"))
    if g("beam_width"):
        p.beam_width = int(g("beam_width"))
    if g("add_special_tokens") is not None:
        p.add_special_tokens = bool(g("add_special_tokens"))
    for k, a in (("ttft_slo_ms", "ttft_slo_ms"), ("tpot_slo_ms", "tpot_slo_ms"), ("ttlt_slo_ms", "ttlt_slo_ms")):
        if g(k) is not None:
            setattr(p, a, float(g(k)))
    routing = g("routing")
    if isinstance(routing, dict):           # chat.proto field 27 / common.proto:63-67: set by the service layer
        p.decode_name = str(routing.get("decode_name") or "")
        p.decode_address = str(routing.get("decode_address") or "")
    for k in ("ttft_priority_weight", "tpot_priority_weight"):
        if g(k) is not None:
            setattr(p, k, max(1, int(g(k))))
    if chat:
        p.logprobs = bool(g("logprobs", False))
        p.top_logprobs = int(g("top_logprobs") or 0)
        p.tools = g("tools")
        p.tool_choice = g("tool_choice", "auto")
        p.chat_template_kwargs = g("chat_template_kwargs")
    else:
        lp = g("logprobs")
        if lp is not None and lp is not False:
            p.logprobs = True
            p.top_logprobs = int(lp) if not isinstance(lp, bool) else 0
    return p


def _usage(u) -> Dict[str, int]:
    return {"prompt_tokens": u.num_prompt_tokens, "completion_tokens": u.num_generated_tokens, "total_tokens": u.num_total_tokens,
            "prompt_tokens_details": {"cached_tokens": u.num_cached_tokens}}


def _lp_chat(lps) -> Optional[Dict]:
    if not lps:
        return None
    return {"content": [{"token": l.token, "logprob": l.logprob, "bytes": list(l.token.encode()),
                         "top_logprobs": [{"token": t.token, "logprob": t.logprob, "bytes": list(t.token.encode())}
                                          for t in (l.top_logprobs or [])]} for l in lps]}


def _lp_completion(lps) -> Optional[Dict]:
    if not lps:
        return None
    return {"tokens": [l.token for l in lps], "token_logprobs": [l.logprob for l in lps],
            "top_logprobs": [{t.token: t.logprob for t in (l.top_logprobs or [])} for l in lps], "text_offset": []}


class APIService:
    def __init__(self, master: LLMMaster, options):
        self.master = master
        self.opt = options
        self.limiter = RateLimiter(options.max_concurrent_requests)
        mt = master.args.model_type
        self.tool_parser = resolve_parser(options.tool_call_parser, mt) if options.tool_call_parser else ""
        self.reasoning_parser = resolve_reasoning_parser(options.reasoning_parser, mt) if options.reasoning_parser else ""
        self.created = int(time.time())
        # masters forked for other models (model id -> their own service object: master, limiter, parsers)
        self.children: Dict[str, "APIService"] = {}
        self._mail: "collections.deque" = collections.deque()      # (handler, output) pairs on their way to the event loop
        self._mail_scheduled = False

    def _by_model(self, name: str):
        """Handler that hands the request to the service object of the model it names (`model`, or `model_id` for the
        admin calls); requests that name no forked model stay with the first master."""
        async def handler(req: Request):
            svc = self
            if self.children:
                try:
                    body = req.json()
                except ValueError:
                    body = None
                if isinstance(body, dict):
                    svc = self.children.get(body.get("model") or body.get("model_id") or "", self)
            return await getattr(svc, name)(req)
        return handler

    def register(self, srv: HttpServer) -> HttpServer:
        srv.add("POST", "/v1/completions", self._by_model("completions"))
        srv.add("POST", "/v1/chat/completions", self._by_model("chat"))
        srv.add("POST", "/v1/embeddings", self._by_model("embeddings"))
        srv.add("POST", "/v1/messages", self._by_model("anthropic_messages"))
        srv.add("POST", "/v1/sample", self._by_model("sample"))
        srv.add("POST", "/v1/rerank", self._by_model("rerank"))
        srv.add("GET", "/v1/models", self.models)
        srv.add("GET", "/v2/repository/index", self.models)
        srv.add("GET", "/health", self.health)
        srv.add("GET", "/metrics", self.metrics)
        srv.add("GET", "/version", self.version)
        srv.add("POST", "/sleep", self._by_model("sleep"))
        srv.add("POST", "/wakeup", self._by_model("wakeup"))
        srv.add("POST", "/fork_master", self.fork_master)
        srv.add("POST", "/link_d2d", self._by_model("link_d2d"))
        srv.add("POST", "/unlink_d2d", self._by_model("unlink_d2d"))
        return srv

    # ------------------------------------------------------------------ plumbing
    def _post(self, loop, fn, arg) -> None:
        """Hand `fn(arg)` to the event loop from the engine's thread.  The outputs of one engine step (one per streaming
        request) share a single wake-up of the loop: they go into a mailbox, and only the first of a burst schedules the
        drain.  (Append first, then look at the flag; the drain clears the flag before it empties the mailbox: an item
        is either seen by the running drain or schedules the next one.)"""
        self._mail.append((fn, arg))
        if not self._mail_scheduled:
            self._mail_scheduled = True
            loop.call_soon_threadsafe(self._drain_mail)

    def _drain_mail(self) -> None:
        self._mail_scheduled = False
        mail = self._mail
        while mail:
            fn, arg = mail.popleft()
            try:
                fn(arg)
            except Exception:                  # one request's handler must not drop the others' outputs
                import logging
                logging.getLogger("xllm").exception("output handler failed")

    async def _run(self, req: Request, prompt, params: RequestParams, on_output, on_done):
        """Submit to the master; `on_output(RequestOutput)` is called on the event loop for every delta."""
        loop = asyncio.get_event_loop()
        done = asyncio.Event()
        holder: Dict[str, Any] = {"cid": None, "cancel": False}

        def cb(out: RequestOutput) -> bool:
            self._post(loop, _deliver, out)
            return not holder["cancel"]

        def _deliver(out: RequestOutput):
            try:
                on_output(out)
            finally:
                if out.finished:
                    done.set()

        fut = self.master.handle_request(prompt, params, cb, asynchronous=True)

        async def watch_disconnect():
            await req.disconnected.wait()
            holder["cancel"] = True
            try:
                cid = fut.result(timeout=5)
                if cid is not None:
                    self.master.cancel(cid)
            except Exception:
                pass
            done.set()
        watcher = asyncio.ensure_future(watch_disconnect())
        await done.wait()
        watcher.cancel()
        on_done()

    def _limited(self, kind: str) -> Response:
        METRICS.inc("server_request_total_limit")
        if self.limiter.sleeping:
            return _err(f"model '{self.master.model_id}' is currently in sleep state", 503, "model_sleeping")
        return _err("too many concurrent requests", 429, kind)

    def _check(self, body: Dict, need: str) -> Optional[Response]:
        if need not in body or body[need] in (None, "", []):
            return _err(f"'{need}' is required")
        model = body.get("model")
        if model and model not in (self.master.model_id, self.opt.model):
            return _err(f"model '{model}' is not served here (serving '{self.master.model_id}')", 404, "model_not_found")
        return None

    # ------------------------------------------------------------------ /v1/completions
    async def completions(self, req: Request):
        body = req.json()
        bad = self._check(body, "prompt")
        if bad:
            return bad
        if not self.limiter.acquire():
            return self._limited("rate_limit_exceeded")
        p = params_from_body(body, chat=False)
        prompt = body.get("token_ids") or body["prompt"]
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], str):
            prompt = prompt[0]
        rid = p.request_id or "cmpl-" + uuid.uuid4().hex[:24]
        p.request_id = rid
        base = {"id": rid, "object": "text_completion", "created": int(time.time()), "model": self.master.model_id}
        if p.streaming:
            resp = StreamingResponse()

            def on_output(out: RequestOutput):
                if out.status and not out.status.ok:
                    resp.put(f"data: {json.dumps({'error': {'message': out.status.message, 'code': out.status.code.name}})}\n\n")
                for o in out.outputs:
                    chunk = dict(base, choices=[{"index": o.index, "text": o.text, "logprobs": _lp_completion(o.logprobs),
                                                 "finish_reason": o.finish_reason}])
                    resp.put(f"data: {json.dumps(chunk, ensure_ascii=False)}\n\n")
                if out.finished:
                    if p.include_usage and out.usage:
                        resp.put(f"data: {json.dumps(dict(base, choices=[], usage=_usage(out.usage)))}\n\n")
                    resp.put("data: [DONE]\n\n")
                    resp.close()
            asyncio.ensure_future(self._run(req, prompt, p, on_output, self.limiter.release))
            return resp
        final: Dict[str, RequestOutput] = {}
        await self._run(req, prompt, p, lambda out: final.__setitem__("o", out) if out.finished else None, self.limiter.release)
        out = final.get("o")
        if out is None:
            return _err("request was cancelled", 499, "cancelled")
        if out.status and not out.status.ok:
            return _err(out.status.message, _HTTP_OF.get(out.status.code, 500), out.status.code.name.lower())
        return Response(dict(base, choices=[{"index": o.index, "text": o.text, "logprobs": _lp_completion(o.logprobs),
                                             "finish_reason": o.finish_reason} for o in out.outputs], usage=_usage(out.usage)))

    # ------------------------------------------------------------------ /v1/chat/completions
    def _split_message(self, text: str, tools) -> Dict[str, Any]:
        msg: Dict[str, Any] = {"role": "assistant", "content": text}
        if self.reasoning_parser:
            r, c = ReasoningParser(self.reasoning_parser).parse(text)
            msg["content"] = c
            if r:
                msg["reasoning_content"] = r
        if self.tool_parser and tools:
            content, calls = parse_tool_calls(msg["content"] or "", self.tool_parser)
            if calls:
                msg["content"] = content or None
                msg["tool_calls"] = [{"id": c.id, "type": "function", "function": {"name": c.name, "arguments": c.arguments}}
                                     for c in calls]
        return msg

    async def chat(self, req: Request):
        body = req.json()
        bad = self._check(body, "messages")
        if bad:
            return bad
        if not self.limiter.acquire():
            return self._limited("rate_limit_exceeded")
        p = params_from_body(body, chat=True)
        rid = p.request_id or "chatcmpl-" + uuid.uuid4().hex[:24]
        p.request_id = rid
        base = {"id": rid, "object": "chat.completion", "created": int(time.time()), "model": self.master.model_id}
        messages = body["messages"]
        if p.streaming:
            resp = StreamingResponse()
            cbase = dict(base, object="chat.completion.chunk")
            state: Dict[int, Dict[str, Any]] = {}

            def send(index, delta, finish=None, lp=None):
                ch = {"index": index, "delta": delta, "finish_reason": finish}
                if lp:
                    ch["logprobs"] = lp
                resp.put(f"data: {json.dumps(dict(cbase, choices=[ch]), ensure_ascii=False)}\n\n")

            def on_output(out: RequestOutput):
                if out.status and not out.status.ok:
                    resp.put(f"data: {json.dumps({'error': {'message': out.status.message, 'code': out.status.code.name}})}\n\n")
                for o in out.outputs:
                    st = state.get(o.index)
                    if st is None:
                        st = state[o.index] = {"r": ReasoningParser(self.reasoning_parser) if self.reasoning_parser else None,
                                               "t": StreamingToolParser(self.tool_parser) if (self.tool_parser and p.tools) else None,
                                               "calls": False}
                        send(o.index, {"role": "assistant", "content": ""})
                    reasoning, content = ("", o.text)
                    if st["r"] is not None:
                        reasoning, content = st["r"].feed(o.text)
                        if o.finish_reason:
                            r2, c2 = st["r"].flush()
                            reasoning, content = reasoning + r2, content + c2
                    tool_deltas = []
                    if st["t"] is not None:
                        content, tool_deltas = st["t"].feed(content)
                        if o.finish_reason:
                            content += st["t"].flush()
                    if reasoning:
                        send(o.index, {"reasoning_content": reasoning})
                    if content:
                        send(o.index, {"content": content}, lp=_lp_chat(o.logprobs))
                    for d in tool_deltas:
                        st["calls"] = True
                        fn = {"arguments": d.arguments}
                        if d.name is not None:
                            fn["name"] = d.name
                        item = {"index": d.index, "function": fn}
                        if d.id:
                            item.update(id=d.id, type="function")
                        send(o.index, {"tool_calls": [item]})
                    if o.finish_reason:
                        send(o.index, {}, "tool_calls" if st["calls"] and o.finish_reason == "stop" else o.finish_reason)
                if out.finished:
                    if p.include_usage and out.usage:
                        resp.put(f"data: {json.dumps(dict(cbase, choices=[], usage=_usage(out.usage)))}\n\n")
                    resp.put("data: [DONE]\n\n")
                    resp.close()
            asyncio.ensure_future(self._run(req, messages, p, on_output, self.limiter.release))
            return resp
        final: Dict[str, RequestOutput] = {}
        await self._run(req, messages, p, lambda out: final.__setitem__("o", out) if out.finished else None, self.limiter.release)
        out = final.get("o")
        if out is None:
            return _err("request was cancelled", 499, "cancelled")
        if out.status and not out.status.ok:
            return _err(out.status.message, _HTTP_OF.get(out.status.code, 500), out.status.code.name.lower())
        choices = []
        for o in out.outputs:
            msg = self._split_message(o.text, p.tools)
            fr = "tool_calls" if msg.get("tool_calls") and o.finish_reason == "stop" else o.finish_reason
            choices.append({"index": o.index, "message": msg, "logprobs": _lp_chat(o.logprobs), "finish_reason": fr})
        return Response(dict(base, choices=choices, usage=_usage(out.usage)))

    # ------------------------------------------------------------------ Anthropic /v1/messages
    async def anthropic_messages(self, req: Request):
        body = req.json()
        bad = self._check(body, "messages")
        if bad:
            return bad
        if "max_tokens" not in body:
            return _err("'max_tokens' is required")
        if not self.limiter.acquire():
            return self._limited("rate_limit_error")
        messages: List[Dict[str, Any]] = []
        system = body.get("system")
        if system:
            messages.append({"role": "system", "content": system if isinstance(system, str) else
                             "".join(b.get("text", "") for b in system if isinstance(b, dict))})
        for m in body["messages"]:
            c = m.get("content")
            if isinstance(c, list):
                c = "".join(b.get("text", "") for b in c if isinstance(b, dict) and b.get("type") == "text")
            messages.append({"role": m.get("role", "user"), "content": c})
        p = RequestParams(max_tokens=int(body["max_tokens"]), temperature=float(body.get("temperature", 1.0)),
                          top_p=float(body.get("top_p", 1.0)), top_k=int(body.get("top_k", -1)), streaming=bool(body.get("stream", False)))
        if body.get("stop_sequences"):
            p.stop = list(body["stop_sequences"])
        mid = "msg_" + uuid.uuid4().hex[:24]
        p.request_id = mid
        stop_of = {"stop": "end_turn", "length": "max_tokens"}
        if p.streaming:
            resp = StreamingResponse()

            def ev(name, data):
                resp.put(f"event: {name}\ndata: {json.dumps(data, ensure_ascii=False)}\n\n")
            started = {"v": False}

            def on_output(out: RequestOutput):
                if not started["v"]:
                    started["v"] = True
                    ev("message_start", {"type": "message_start", "message": {"id": mid, "type": "message", "role": "assistant", "content": [],
                                                                              "model": self.master.model_id, "stop_reason": None,
                                                                              "usage": {"input_tokens": 0, "output_tokens": 0}}})
                    ev("content_block_start", {"type": "content_block_start", "index": 0, "content_block": {"type": "text", "text": ""}})
                fr = None
                for o in out.outputs:
                    if o.text:
                        ev("content_block_delta", {"type": "content_block_delta", "index": 0, "delta": {"type": "text_delta", "text": o.text}})
                    fr = o.finish_reason or fr
                if out.finished:
                    ev("content_block_stop", {"type": "content_block_stop", "index": 0})
                    u = out.usage
                    ev("message_delta", {"type": "message_delta", "delta": {"stop_reason": stop_of.get(fr, "end_turn"), "stop_sequence": None},
                                         "usage": {"input_tokens": u.num_prompt_tokens if u else 0, "output_tokens": u.num_generated_tokens if u else 0}})
                    ev("message_stop", {"type": "message_stop"})
                    resp.close()
            asyncio.ensure_future(self._run(req, messages, p, on_output, self.limiter.release))
            return resp
        final: Dict[str, RequestOutput] = {}
        await self._run(req, messages, p, lambda out: final.__setitem__("o", out) if out.finished else None, self.limiter.release)
        out = final.get("o")
        if out is None or (out.status and not out.status.ok):
            return Response({"type": "error", "error": {"type": "api_error", "message": out.status.message if out else "cancelled"}}, 500)
        o = out.outputs[0]
        return Response({"id": mid, "type": "message", "role": "assistant", "model": self.master.model_id,
                         "content": [{"type": "text", "text": o.text}], "stop_reason": stop_of.get(o.finish_reason, "end_turn"),
                         "stop_sequence": None, "usage": {"input_tokens": out.usage.num_prompt_tokens,
                                                          "output_tokens": out.usage.num_generated_tokens}})

    # ------------------------------------------------------------------ embeddings / rerank / models / health
    async def embeddings(self, req: Request):
        body = req.json()
        bad = self._check(body, "input")
        if bad:
            return bad
        inputs = body["input"]
        inputs = [inputs] if isinstance(inputs, str) or (inputs and isinstance(inputs[0], int)) else list(inputs)
        from ..runtime.embed import embed_prompts
        loop = asyncio.get_event_loop()
        outs = await loop.run_in_executor(None, lambda: self.master.run_exclusive(lambda: embed_prompts(self.master, inputs)))
        total = sum(o.usage.num_prompt_tokens for o in outs)
        return Response({"object": "list", "model": self.master.model_id,
                         "data": [{"object": "embedding", "index": i, "embedding": o.outputs[0].embeddings} for i, o in enumerate(outs)],
                         "usage": {"prompt_tokens": total, "total_tokens": total}})

    async def rerank(self, req: Request):
        body = req.json()
        if "query" not in body or "documents" not in body:
            return _err("'query' and 'documents' are required")
        from ..runtime.embed import embed_prompts, rerank_scores
        loop = asyncio.get_event_loop()
        if getattr(self.opt, "enable_qwen3_reranker", False):
            # Qwen3-Reranker: one prompt per document, query + document as the client formatted them; the score is the
            # probability of "yes" at the answer position (qwen3_rerank_service_impl.cpp:45-76 of the reference)
            pairs = [body["query"] + d for d in body["documents"]]
            try:
                scores = await loop.run_in_executor(None, lambda: self.master.run_exclusive(lambda: rerank_scores(self.master, pairs)))
            except ValueError as e:
                return _err(str(e))
        else:
            texts = [body["query"]] + list(body["documents"])
            outs = await loop.run_in_executor(None, lambda: self.master.run_exclusive(lambda: embed_prompts(self.master, texts)))
            q = outs[0].outputs[0].embeddings
            scores = [sum(a * b for a, b in zip(q, o.outputs[0].embeddings)) for o in outs[1:]]
        order = sorted(range(len(scores)), key=lambda i: -scores[i])[: int(body.get("top_n") or len(scores))]
        return Response({"model": self.master.model_id, "results": [{"index": i, "relevance_score": scores[i],
                                                                     "document": {"text": body["documents"][i]}} for i in order]})

    async def sample(self, req: Request):
        """`/v1/sample`: next-token distributions at the positions of a selector token (sample_service_impl.cpp)."""
        body = req.json()
        if "prompt" not in body or "selector" not in body:
            return _err("'prompt' and 'selector' are required")
        import dataclasses
        from .llm import build_sample_jobs
        prompts = body["prompt"] if isinstance(body["prompt"], list) else [body["prompt"]]
        sels = body["selector"]
        sels = [sels] * len(prompts) if isinstance(sels, (str, dict)) else list(sels)
        if len(sels) != len(prompts):
            return _err("the number of selectors must match the number of prompts")
        try:
            jobs, hits = build_sample_jobs(self.master.tokenizer, prompts, sels)
        except ValueError as e:
            return _err(str(e))
        base = params_from_body(body, chat=False)
        k = int(body.get("logprobs") or 5)
        loop = asyncio.get_event_loop()
        futs = {}
        for i, h, prefix in jobs:
            rp = dataclasses.replace(base)
            rp.request_id = ""
            rp.max_tokens, rp.n, rp.best_of, rp.logprobs, rp.top_logprobs, rp.streaming, rp.ignore_eos = 1, 1, 1, True, k, False, True
            fut = loop.create_future()
            futs[(i, h)] = fut

            def cb(out: RequestOutput, fut=fut) -> bool:
                if out.finished:
                    loop.call_soon_threadsafe(lambda: fut.done() or fut.set_result(out))
                return True
            self.master.handle_request(prefix, rp, cb, asynchronous=True)
        outs = []
        for i, pr in enumerate(prompts):
            o = RequestOutput(prompt=pr, finished=True, outputs=[])
            for h in range(hits[i]):
                r = await futs[(i, h)]
                if r.status is not None and not r.status.ok:
                    return _err(f"sample request failed: {r.status.message}", 500, "internal_error")
                so = r.outputs[0]
                so.index = h
                o.outputs.append(so)
            outs.append(o)
        data = []
        for i, o in enumerate(outs):
            data.append({"index": i, "samples": [{
                "sample_id": so.index, "token": so.text, "token_ids": so.token_ids, "finish_reason": so.finish_reason,
                "top_logprobs": [{"token": t.token, "token_id": t.token_id, "logprob": t.logprob}
                                 for t in ((so.logprobs or [None])[0].top_logprobs or [])] if so.logprobs else []}
                for so in o.outputs]})
        return Response({"object": "sample", "model": self.master.model_id, "data": data})

    async def models(self, req: Request):
        every = [self] + list(self.children.values())
        return Response({"object": "list", "data": [{"id": s.master.model_id, "object": "model", "created": s.created,
                                                     "owned_by": "xllm", "max_model_len": s.master.args.max_position_embeddings,
                                                     "sleeping": s.master.is_sleeping()} for s in every]})

    async def health(self, req: Request):
        ok, why = HEALTH.status()
        return Response({"status": "ok" if ok else "unhealthy", "reason": why}, 200 if ok else 503)

    async def metrics(self, req: Request):
        return Response(METRICS.prometheus_text(), content_type="text/plain; version=0.0.4")

    async def version(self, req: Request):
        from .. import __version__
        return Response({"version": __version__})

    async def sleep(self, req: Request):
        """POST /sleep {"master_status": 1 | 2 | "LIGHT_SLEEP" | "DEEP_SLEEP"} (api_service.cpp:977-1045 of the reference)."""
        body = req.json()
        status = body.get("master_status", 1)
        level = {"LIGHT_SLEEP": 1, "DEEP_SLEEP": 2}.get(status, status)
        if level not in (1, 2):
            return _err("Invalid sleep status")
        if self.master.is_sleeping():
            return _err("Master for model is already sleeping", 409)
        if not self.limiter.try_set_sleeping():
            return _err("Cannot sleep model with in-flight requests", 409)
        loop = asyncio.get_event_loop()
        ok = await loop.run_in_executor(None, self.master.sleep, int(level))
        if not ok:
            self.limiter.try_wakeup()
            return _err("Failed to sleep model", 500, "internal_error")
        return Response({"ok": True, "master_status": int(level), "bytes_released": self.master.engine.bytes_released_by_sleep})

    async def wakeup(self, req: Request):
        if not self.master.is_sleeping():
            return _err("Master for model is not sleeping", 409)
        loop = asyncio.get_event_loop()
        try:
            body = req.json() or {}
        except ValueError:
            body = {}
        remote = [str(a) for a in (body.get("remote_addrs") or [])]
        ok = await loop.run_in_executor(None, lambda: self.master.wakeup(remote))
        if not ok:
            return _err("Failed to wakeup model", 500, "internal_error")
        self.limiter.try_wakeup()
        return Response({"ok": True, "weights_pulled_bytes": int(getattr(self.master.engine, "weights_pulled_bytes", 0)),
                         "weights_pull_ms": float(getattr(self.master.engine, "weights_pull_ms", 0.0))})

    async def link_d2d(self, req: Request):
        """POST /link_d2d {"model_id": ..., "device_ips": ["host:port", ...]} (LinkD2DHttp in the reference): open sessions to
        the weight services of awake instances of this model."""
        addrs = [str(a) for a in (req.json().get("device_ips") or [])]
        if not addrs:
            return _err("'device_ips' is required")
        loop = asyncio.get_event_loop()
        try:
            await loop.run_in_executor(None, self.master.link_d2d, addrs)
        except (OSError, ConnectionError, TimeoutError) as e:
            return _err(f"Failed to link d2d: {e}", 502, "bad_gateway")
        return Response({"ok": True, "linked": sorted(self.master.weight_sources)})

    async def unlink_d2d(self, req: Request):
        addrs = [str(a) for a in (req.json().get("device_ips") or [])]
        if not addrs:
            return _err("'device_ips' is required")
        n = self.master.unlink_d2d(addrs)
        return Response({"ok": True, "unlinked": n, "linked": sorted(self.master.weight_sources)})

    async def fork_master(self, req: Request):
        """POST /fork_master {"model_path": dir, "master_status": 0 | 1 | 2} (ForkMasterHttp, api_service.cpp:892-975 of the
        reference): load another model beside the first one and serve it under the name of its directory."""
        import os
        from ..runtime.master import fork_master
        body = req.json()
        path = str(body.get("model_path") or "")
        if not path:
            return _err("'model_path' is required")
        status = body.get("master_status", 0)
        status = {"WAKEUP": 0, "LIGHT_SLEEP": 1, "DEEP_SLEEP": 2}.get(status, status)
        if status not in (0, 1, 2):
            return _err("Invalid master_status")
        model_id = path[7:] if path.startswith("preset:") else os.path.basename(os.path.normpath(path))
        if model_id == self.master.model_id or model_id in self.children:
            return Response({"ok": True, "model_id": model_id, "message": "master for this model already exists"})
        overrides = {k: body[k] for k in ("max_memory_utilization", "max_cache_size", "num_kv_blocks") if k in body}
        loop = asyncio.get_event_loop()
        try:
            new = await loop.run_in_executor(None, lambda: fork_master(self.master, path, model_id, int(status), **overrides))
        except (FileNotFoundError, ValueError, KeyError) as e:
            return _err(f"Failed to parse fork master request: {e}")
        except NotImplementedError as e:
            return _err(str(e), 501, "not_implemented")
        except Exception as e:                                   # out of memory, broken checkpoint, ...
            return _err(f"Failed to fork master: {type(e).__name__}: {e}", 500, "internal_error")
        child = APIService(new, new.opt)
        if new.is_sleeping():
            child.limiter.try_set_sleeping()                     # no request in flight yet: cannot fail
        self.children[model_id] = child
        return Response({"ok": True, "model_id": model_id, "master_status": int(status), "server_idx": new.server_idx})



async def serve(master: LLMMaster, options, ready: Optional[threading.Event] = None):
    srv = APIService(master, options).register(HttpServer())
    server = await srv.start(options.host, options.port)
    if ready is not None:
        ready.set()
    async with server:
        await server.serve_forever()
