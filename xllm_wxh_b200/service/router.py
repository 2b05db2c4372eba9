"""The service in front of several engine instances: registry endpoints, load-balance policies, request forwarding.

Role of the xllm-service master that the reference's XServiceClient talks to (runtime/xservice_client.cpp: register /
heartbeat / watch; docs/en/features/global_kvcache.md and disagg_pd.md: cache-aware routing, prefill / decode pairing).
HTTP + JSON stand where the reference uses etcd and brpc.

Endpoints
    POST /xservice/register      {"info": InstanceInfo, "ttl_s": 3}
    POST /xservice/heartbeat     {"name", "incarnation_id", "load_metrics", "latency_metrics", "cache_event"}
    POST /xservice/deregister    {"name"}
    GET  /xservice/instances     ?type=PREFILL        -> names and infos
    GET  /xservice/instance      ?name=...            -> one info with its current load
    GET  /xservice/watch         ?revision=N&timeout=S  (long poll)
    POST /v1/completions, /v1/chat/completions        forwarded to the instance the policy picks (SSE passes through)
"""
from __future__ import annotations

import asyncio
import http.client
import itertools
import json
import threading
from typing import Any, Dict, List, Optional, Sequence, Tuple

from .. import _core
from ..api.server import HttpServer, Request, Response, StreamingResponse
from .registry import InstanceInfo, InstanceState, Registry


# ----------------------------------------------------------------------------- policies
class RoundRobin:
    name = "RR"

    def __init__(self):
        self._it = itertools.count()

    def pick(self, candidates: Sequence[InstanceState], tokens: Optional[Sequence[int]]) -> InstanceState:
        ordered = sorted(candidates, key=lambda s: s.info.name)
        return ordered[next(self._it) % len(ordered)]


class CacheAwareRouting:
    """Score = share of the prompt's prefix blocks the instance already caches, minus its load.

    The prefix index is built from the instances' cache events: keys are the same chained 128-bit block hashes the
    engines' prefix caches use, so the router can tell how many leading blocks of a prompt an instance holds without
    asking it."""
    name = "CAR"

    def __init__(self, load_weight: float = 0.5, max_waiting: int = 64):
        self.load_weight, self.max_waiting = load_weight, max_waiting

    @staticmethod
    def matched_blocks(st: InstanceState, tokens: Sequence[int]) -> Tuple[int, int]:
        keys = _core.prefix_block_keys(list(tokens), st.info.block_size, st.info.hash_seed)
        n = 0
        for k in keys:
            if (int(k[0]), int(k[1])) not in st.cached_keys:
                break
            n += 1
        return n, len(keys)

    def score(self, st: InstanceState, tokens: Optional[Sequence[int]]) -> float:
        hit = 0.0
        if tokens:
            n, total = self.matched_blocks(st, tokens)
            hit = n / total if total else 0.0
        load = min(1.0, (st.waiting_requests + st.inflight) / max(1, self.max_waiting)) * 0.5 + 0.5 * min(1.0, st.cache_usage)
        return hit - self.load_weight * load

    def pick(self, candidates: Sequence[InstanceState], tokens: Optional[Sequence[int]]) -> InstanceState:
        return max(sorted(candidates, key=lambda s: s.info.name), key=lambda s: self.score(s, tokens))


class SloAware:
    """Least recent latency first (recent_max_ttft for prefill-capable roles, recent_max_tbt for decode), then load."""
    name = "SLO_AWARE"

    def pick(self, candidates: Sequence[InstanceState], tokens: Optional[Sequence[int]]) -> InstanceState:
        def key(s: InstanceState):
            lat = s.recent_max_tbt_ms if s.info.type == "DECODE" else s.recent_max_ttft_ms
            return (lat, s.waiting_requests + s.inflight, s.info.name)
        return min(candidates, key=key)


POLICIES = {"RR": RoundRobin, "CAR": CacheAwareRouting, "SLO_AWARE": SloAware}


# ----------------------------------------------------------------------------- service
class XllmService:
    def __init__(self, policy: str = "CAR", tokenizer=None, chat_template=None, lease_sweep_s: float = 0.5):
        self.registry = Registry()
        self.policy = POLICIES[policy]()
        self.tokenizer = tokenizer
        self.chat_template = chat_template
        self.lease_sweep_s = lease_sweep_s
        self._stop = threading.Event()
        self._sweeper: Optional[threading.Thread] = None
        self.forwarded: Dict[str, int] = {}

    # ------------------------------------------------------------------ routing decisions
    def prompt_tokens(self, body: Dict[str, Any], chat: bool) -> Optional[List[int]]:
        """Token ids of the request as the engine will see them (needed for the prefix keys); None when unknown."""
        try:
            if chat:
                if self.tokenizer is None or self.chat_template is None:
                    return None
                text = self.chat_template.apply(body.get("messages") or [], tools=body.get("tools"),
                                                kwargs=body.get("chat_template_kwargs"))
                return self.tokenizer.encode(text, add_special_tokens=False)
            p = body.get("prompt")
            if isinstance(p, list) and p and all(isinstance(x, int) for x in p):
                return list(p)
            if isinstance(p, str) and self.tokenizer is not None:
                return self.tokenizer.encode(p)
        except Exception:
            return None
        return None

    def choose(self, tokens: Optional[Sequence[int]], model: str = "") -> Tuple[Optional[InstanceState], Optional[InstanceState]]:
        """(instance that takes the request, decode partner or None).  With PREFILL and DECODE instances present the
        request goes to a prefill instance and names the decode instance that will continue it.  When instances of several
        models are registered, a request that names one of them stays among that model's instances."""
        self.registry.expire()

        def of_model(states):
            mine = [st for st in states if model and st.info.model == model]
            return mine or ([] if model and model in served else states)
        served = {st.info.model for st in self.registry.instances() if st.info.model}
        prefill, decode = of_model(self.registry.instances("PREFILL")), of_model(self.registry.instances("DECODE"))
        if prefill and decode:
            return self.policy.pick(prefill, tokens), SloAware().pick(decode, None)
        pool = of_model(self.registry.instances("DEFAULT") + self.registry.instances("MIX"))
        if not pool:
            return None, None
        return self.policy.pick(pool, tokens), None

    # ------------------------------------------------------------------ HTTP
    def register(self, srv: HttpServer) -> HttpServer:
        reg = self.registry

        @srv.route("POST", "/xservice/register")
        async def _register(req: Request):
            b = req.json()
            try:
                return Response(reg.register(InstanceInfo.from_json(b.get("info") or {}), float(b.get("ttl_s", 3.0))))
            except (ValueError, TypeError) as e:
                return Response({"ok": False, "error": str(e)}, 400)

        @srv.route("POST", "/xservice/heartbeat")
        async def _heartbeat(req: Request):
            b = req.json()
            return Response(reg.heartbeat(str(b.get("name", "")), str(b.get("incarnation_id", "")), b))

        @srv.route("POST", "/xservice/deregister")
        async def _deregister(req: Request):
            return Response({"ok": reg.deregister(str(req.json().get("name", "")))})

        @srv.route("GET", "/xservice/instances")
        async def _instances(req: Request):
            reg.expire()
            role = (req.query.get("type") or [None])[0]
            return Response({"revision": reg.revision, "instances": [s.info.to_json() for s in reg.instances(role)]})

        @srv.route("GET", "/xservice/instance")
        async def _instance(req: Request):
            st = reg.get((req.query.get("name") or [""])[0])
            if st is None:
                return Response({"error": "unknown instance"}, 404)
            return Response({"info": st.info.to_json(), "load": {"gpu_cache_usage_perc": st.cache_usage,
                             "waiting_requests_num": st.waiting_requests, "inflight": st.inflight,
                             "recent_max_ttft": st.recent_max_ttft_ms, "recent_max_tbt": st.recent_max_tbt_ms,
                             "cached_blocks": len(st.cached_keys)}})

        @srv.route("GET", "/xservice/watch")
        async def _watch(req: Request):
            since = int((req.query.get("revision") or ["0"])[0])
            timeout = min(30.0, float((req.query.get("timeout") or ["10"])[0]))
            loop = asyncio.get_event_loop()
            rev, events = await loop.run_in_executor(None, reg.wait_for_change, since, timeout)
            return Response({"revision": rev, "events": [{"revision": r, "type": k, "key": key} for r, k, key in events]})

        async def _forward(req: Request, chat: bool, with_tokens: bool = True):
            body = req.json()
            tokens = self.prompt_tokens(body, chat) if with_tokens else None
            target, partner = self.choose(tokens, str(body.get("model") or ""))
            if target is None:
                return Response({"error": {"message": "no instance is registered", "type": "service_unavailable"}}, 503)
            if partner is not None:
                body["routing"] = {"prefill_name": target.info.name, "decode_name": partner.info.name,
                                   "decode_address": partner.info.rpc_address}
            name = target.info.name
            self.forwarded[name] = self.forwarded.get(name, 0) + 1
            reg.track(name, +1)
            host, _, port = target.info.rpc_address.rpartition(":")
            payload = json.dumps(body).encode()
            loop = asyncio.get_event_loop()
            if not body.get("stream"):
                def call():
                    try:
                        c = http.client.HTTPConnection(host, int(port), timeout=600)
                        c.request("POST", req.path, payload, {"Content-Type": "application/json", "Connection": "close"})
                        r = c.getresponse()
                        return r.status, r.read()
                    except OSError as e:
                        return 503, json.dumps({"error": {"message": f"instance {name} unreachable: {e}",
                                                          "type": "service_unavailable"}}).encode()
                    finally:
                        reg.track(name, -1)
                status, data = await loop.run_in_executor(None, call)
                return Response(data, status, headers={"X-Xllm-Instance": name})
            out = StreamingResponse(headers={"X-Xllm-Instance": name})

            def pump():
                try:
                    c = http.client.HTTPConnection(host, int(port), timeout=600)
                    c.request("POST", req.path, payload, {"Content-Type": "application/json", "Connection": "close"})
                    r = c.getresponse()
                    while not out.closed:
                        chunk = r.read1(65536)
                        if not chunk:
                            break
                        out.put(chunk)
                except OSError as e:
                    out.put(f"data: {json.dumps({'error': {'message': str(e)}})}\n\n")
                finally:
                    reg.track(name, -1)
                    out.close()
            threading.Thread(target=pump, daemon=True).start()
            return out

        @srv.route("POST", "/v1/completions")
        async def _completions(req: Request):
            return await _forward(req, False)

        @srv.route("POST", "/v1/chat/completions")
        async def _chat(req: Request):
            return await _forward(req, True)

        # requests without a generation phase: any instance of the model will do (no decode partner is named for them)
        for path in ("/v1/embeddings", "/v1/rerank", "/v1/sample", "/v1/messages"):
            async def _plain(req: Request):
                return await _forward(req, False, with_tokens=False)
            srv.add("POST", path, _plain)

        @srv.route("GET", "/v1/models")
        async def _models(req: Request):
            reg.expire()
            seen: Dict[str, int] = {}
            for st in reg.instances():
                if st.info.model:
                    seen[st.info.model] = seen.get(st.info.model, 0) + 1
            return Response({"object": "list", "data": [{"id": m, "object": "model", "owned_by": "xllm", "instances": n}
                                                        for m, n in sorted(seen.items())]})

        @srv.route("GET", "/metrics")
        async def _metrics(req: Request):
            reg.expire()
            lines = ["# TYPE xllm_service_instances gauge"]
            for role in ("DEFAULT", "MIX", "PREFILL", "DECODE"):
                lines.append(f'xllm_service_instances{{type="{role}"}} {len(reg.instances(role))}')
            lines.append("# TYPE xllm_service_forwarded_requests_total counter")
            for name, n in sorted(self.forwarded.items()):
                lines.append(f'xllm_service_forwarded_requests_total{{instance="{name}"}} {n}')
            lines.append("# TYPE xllm_service_inflight_requests gauge")
            for st in reg.instances():
                lines.append(f'xllm_service_inflight_requests{{instance="{st.info.name}"}} {st.inflight}')
                lines.append(f'xllm_service_instance_cache_usage{{instance="{st.info.name}"}} {st.cache_usage}')
                lines.append(f'xllm_service_instance_waiting_requests{{instance="{st.info.name}"}} {st.waiting_requests}')
            lines.append(f"xllm_service_registry_revision {reg.revision}")
            return Response("\n".join(lines) + "\n", content_type="text/plain; version=0.0.4")

        @srv.route("GET", "/health")
        async def _health(req: Request):
            return Response({"status": "ok", "instances": len(reg.instances())})
        return srv

    # ------------------------------------------------------------------ lifecycle
    def start_sweeper(self):
        def loop():
            while not self._stop.wait(self.lease_sweep_s):
                self.registry.expire()
        self._sweeper = threading.Thread(target=loop, daemon=True)
        self._sweeper.start()

    def stop(self):
        self._stop.set()


async def serve(service: XllmService, host: str, port: int, ready: Optional[threading.Event] = None):
    srv = service.register(HttpServer())
    server = await srv.start(host, port)
    service.start_sweeper()
    if ready is not None:
        ready.set()
    async with server:
        await server.serve_forever()


def main(argv: Optional[List[str]] = None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="xllm-service", description="registry and router in front of xllm instances")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=9888)
    ap.add_argument("--load_balance_policy", default="CAR", choices=sorted(POLICIES))
    ap.add_argument("--tokenizer_path", default="", help="model directory (tokenizer + chat template) for cache-aware routing")
    ns = ap.parse_args(argv)
    tok = tpl = None
    if ns.tokenizer_path:
        from ..api.chat_template import JinjaChatTemplate
        from ..utils.tokenizer import load_tokenizer
        tok = load_tokenizer(ns.tokenizer_path)
        if getattr(tok, "chat_template", None):
            tpl = JinjaChatTemplate(tok.chat_template, tok)
    asyncio.run(serve(XllmService(ns.load_balance_policy, tok, tpl), ns.host, ns.port))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
