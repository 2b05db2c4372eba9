"""Service layer: registry with leases and watches, load-balance policies, the instance-side client, and two CPU engine
instances behind the router (cache-aware routing by real prefix-cache events).

The reference's counterpart is XServiceClient + etcd + the xllm-service master (xservice_client.cpp); failures are made on
the host: a lease that runs out, a service that forgets an instance, an unreachable address.
"""
import asyncio
import json
import socket
import threading
import time

import pytest
import requests
import torch

from xllm_wxh_b200 import _core
from xllm_wxh_b200.api.openai_service import APIService
from xllm_wxh_b200.api.server import HttpServer
from xllm_wxh_b200.config import Options
from xllm_wxh_b200.models.args import preset
from xllm_wxh_b200.models.qwen import QwenForCausalLM
from xllm_wxh_b200.runtime.engine import LLMEngine
from xllm_wxh_b200.runtime.master import LLMMaster
from xllm_wxh_b200.runtime.xservice_client import XServiceClient
from xllm_wxh_b200.service.registry import InstanceInfo, InstanceState, Registry
from xllm_wxh_b200.service.router import CacheAwareRouting, RoundRobin, SloAware, XllmService
from xllm_wxh_b200.utils.tokenizer import IdTokenizer


class Clock:
    def __init__(self):
        self.t = 100.0

    def __call__(self):
        return self.t


# ------------------------------------------------------------------ registry
def test_registry_lease_heartbeat_and_expiry():
    ck = Clock()
    r = Registry(clock=ck)
    a = InstanceInfo(name="a", rpc_address="127.0.0.1:1", type="PREFILL", incarnation_id="i1")
    out = r.register(a, ttl_s=3.0)
    assert out["ok"] and out["key"] == "XLLM:PREFILL:a" and r.names("PREFILL") == ["a"] and r.names("DECODE") == []
    ck.t += 2.0
    assert r.heartbeat("a", "i1", {"load_metrics": {"gpu_cache_usage_perc": 0.25, "waiting_requests_num": 3},
                                   "latency_metrics": {"recent_max_ttft": 120, "recent_max_tbt": 9},
                                   "cache_event": {"stored_cache": [[1, 2], [3, 4]], "removed_cache": []}})["registered"]
    st = r.get("a")
    assert st.cache_usage == 0.25 and st.waiting_requests == 3 and st.recent_max_ttft_ms == 120 and st.cached_keys == {(1, 2), (3, 4)}
    ck.t += 2.5                                     # 4.5 s after registration, 2.5 s after the heartbeat: still alive
    assert r.expire() == [] and r.names() == ["a"]
    r.heartbeat("a", "i1", {"cache_event": {"stored_cache": [], "removed_cache": [[1, 2]]}})
    assert r.get("a").cached_keys == {(3, 4)}
    ck.t += 3.5
    assert r.expire() == ["a"] and r.names() == []
    # a heartbeat after the lease ran out asks the instance to register again
    assert r.heartbeat("a", "i1", {}) == {"ok": False, "registered": False}
    with pytest.raises(ValueError):
        r.register(InstanceInfo(name="x", type="WORKER"))
    with pytest.raises(ValueError):
        r.register(InstanceInfo(name="", type="DEFAULT"))


def test_registry_restart_under_the_same_name_drops_the_old_cache_view():
    r = Registry(clock=Clock())
    r.register(InstanceInfo(name="a", type="DEFAULT", incarnation_id="old"))
    r.heartbeat("a", "old", {"cache_event": {"stored_cache": [[7, 7]]}})
    assert r.heartbeat("a", "new", {})["registered"] is False          # another process claims the name
    r.register(InstanceInfo(name="a", type="DEFAULT", incarnation_id="new"))
    assert r.get("a").cached_keys == set()
    assert r.heartbeat("a", "old", {})["registered"] is False          # the old incarnation is fenced off


def test_registry_watch_wakes_on_change():
    r = Registry()
    rev0 = r.revision
    got = {}

    def waiter():
        got["v"] = r.wait_for_change(rev0, 5.0)
    th = threading.Thread(target=waiter)
    th.start()
    time.sleep(0.1)
    r.register(InstanceInfo(name="d0", type="DECODE", incarnation_id="x"))
    th.join(5)
    rev, events = got["v"]
    assert rev == rev0 + 1 and events == [(rev, "PUT", "XLLM:DECODE:d0")]
    t0 = time.monotonic()
    rev2, ev2 = r.wait_for_change(rev, 0.2)                             # nothing happens: bounded wait
    assert rev2 == rev and ev2 == [] and time.monotonic() - t0 < 2.0
    r.deregister("d0")
    assert r.wait_for_change(rev, 0.1)[1][0][1:] == ("DELETE", "XLLM:DECODE:d0")


# ------------------------------------------------------------------ policies
def _state(name, role="DEFAULT", **kw):
    st = InstanceState(info=InstanceInfo(name=name, type=role, rpc_address=f"127.0.0.1:{hash(name) % 1000 + 1000}",
                                         block_size=4, hash_seed=1024), lease_deadline=1e18, ttl_s=3)
    for k, v in kw.items():
        setattr(st, k, v)
    return st


def test_cache_aware_routing_follows_the_prefix_and_backs_off_under_load():
    toks = list(range(50, 66))                                          # 4 blocks of 4
    keys = [tuple(k) for k in _core.prefix_block_keys(toks, 4, 1024)]
    a, b = _state("a"), _state("b", cached_keys=set(keys[:3]))
    car = CacheAwareRouting(load_weight=0.5, max_waiting=8)
    assert car.matched_blocks(b, toks) == (3, 4) and car.matched_blocks(a, toks) == (0, 4)
    assert car.pick([a, b], toks).info.name == "b"
    # a hole in the chain ends the match: blocks 0 and 2 cached means one usable block
    c = _state("c", cached_keys={keys[0], keys[2]})
    assert car.matched_blocks(c, toks) == (1, 4)
    # other prompts go to the less loaded instance
    b.waiting_requests = 6
    assert car.pick([a, b], list(range(900, 916))).info.name == "a"
    # a saturated cache holder loses even its own prefix
    b.waiting_requests, b.cache_usage = 8, 1.0
    assert car.score(b, toks) < car.score(a, toks) + 0.75 + 1e-9
    assert CacheAwareRouting(load_weight=2.0, max_waiting=8).pick([a, b], toks).info.name == "a"
    # different block size / seed on the instance side changes the keys: no false hits
    d = _state("d", cached_keys=set(keys))
    d.info.hash_seed = 7
    assert car.matched_blocks(d, toks)[0] == 0


def test_round_robin_slo_policy_and_prefill_decode_pairing():
    rr = RoundRobin()
    pool = [_state("b"), _state("a"), _state("c")]
    assert [rr.pick(pool, None).info.name for _ in range(4)] == ["a", "b", "c", "a"]
    slo = SloAware()
    assert slo.pick([_state("x", recent_max_ttft_ms=300), _state("y", recent_max_ttft_ms=80)], None).info.name == "y"
    svc = XllmService(policy="RR")
    assert svc.choose(None) == (None, None)
    for n, role in (("p0", "PREFILL"), ("p1", "PREFILL"), ("d0", "DECODE"), ("d1", "DECODE")):
        svc.registry.register(InstanceInfo(name=n, type=role, incarnation_id=n, rpc_address="127.0.0.1:9"), ttl_s=60)
    svc.registry.heartbeat("d0", "d0", {"latency_metrics": {"recent_max_tbt": 40}})
    svc.registry.heartbeat("d1", "d1", {"latency_metrics": {"recent_max_tbt": 12}})
    t, partner = svc.choose(None)
    assert t.info.type == "PREFILL" and partner.info.name == "d1"
    # instances of two models: a request that names a served model stays among that model's instances
    two = XllmService(policy="RR")
    for n, m in (("a0", "alpha"), ("a1", "alpha"), ("b0", "beta")):
        two.registry.register(InstanceInfo(name=n, type="DEFAULT", incarnation_id=n, rpc_address="127.0.0.1:9", model=m), ttl_s=60)
    assert {two.choose(None, "alpha")[0].info.name for _ in range(4)} == {"a0", "a1"}
    assert {two.choose(None, "beta")[0].info.name for _ in range(3)} == {"b0"}
    assert {two.choose(None, "")[0].info.name for _ in range(6)} == {"a0", "a1", "b0"}            # no model named: any instance
    assert {two.choose(None, "an-alias")[0].info.name for _ in range(6)} == {"a0", "a1", "b0"}    # unknown name: left to the instance
    assert svc.prompt_tokens({"prompt": [1, 2, 3]}, chat=False) == [1, 2, 3]
    assert svc.prompt_tokens({"prompt": "text"}, chat=False) is None          # no tokenizer configured


# ------------------------------------------------------------------ client against a live service
def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _wait(cond, timeout=10.0):
    deadline = time.time() + timeout
    while not cond():
        assert time.time() < deadline, "condition not reached"
        time.sleep(0.005)


def _serve(register_fn):
    """Run an HttpServer on its own loop thread; returns (port, stop)."""
    port = _free_port()
    loop = asyncio.new_event_loop()
    ready = threading.Event()

    def run():
        asyncio.set_event_loop(loop)
        srv = register_fn(HttpServer())
        loop.run_until_complete(srv.start("127.0.0.1", port))
        ready.set()
        loop.run_forever()
    th = threading.Thread(target=run, daemon=True)
    th.start()
    assert ready.wait(10)

    def stop():
        loop.call_soon_threadsafe(loop.stop)
        th.join(5)
    return port, stop


def test_client_registers_heartbeats_and_recovers_after_the_service_forgets_it():
    svc = XllmService(policy="RR")
    port, stop = _serve(svc.register)
    try:
        c = XServiceClient(f"127.0.0.1:{port}", heart_beat_interval=0.05, ttl_s=1.0)
        events = {"stored": [(1, 1), (2, 2)], "removed": []}
        c._load_fn = lambda: {"gpu_cache_usage_perc": 0.5, "waiting_requests_num": 2, "running_requests_num": 1}
        c._latency_fn = lambda: {"recent_max_ttft": 33.0, "recent_max_tbt": 4.0}

        def take():
            s, r = events["stored"], events["removed"]
            events["stored"], events["removed"] = [], []
            return s, r
        c._cache_events_fn = take
        assert c.register_instance(InstanceInfo(name="inst", rpc_address="127.0.0.1:1", type="DECODE"))
        assert c.get_static_decode_list() == ["inst"] and c.get_static_prefill_list() == []
        assert c.heartbeat_once()
        st = svc.registry.get("inst")
        assert st.cached_keys == {(1, 1), (2, 2)} and st.waiting_requests == 2 and st.recent_max_ttft_ms == 33.0
        info = c.get_instance_info("inst")
        assert info.type == "DECODE" and info.incarnation_id == c.incarnation_id
        # the service loses the instance (restart, or a lease that ran out during a stall)
        svc.registry.deregister("inst")
        assert c.heartbeat_once() is False                       # refused -> registered again at once, cache view replayed
        assert c.num_registrations == 2
        st = svc.registry.get("inst")
        assert st is not None and st.cached_keys == {(1, 1), (2, 2)}
        # background thread keeps the lease alive well past its TTL
        c.start()
        time.sleep(1.6)
        assert svc.registry.expire() == [] and svc.registry.get("inst") is not None
        rev, ev = c.watch(svc.registry.revision, timeout_s=0.2)
        assert ev == []
        c.stop()
        assert svc.registry.get("inst") is None                  # deregistered on the way out
    finally:
        stop()


def test_client_survives_an_unreachable_service():
    c = XServiceClient(f"127.0.0.1:{_free_port()}", heart_beat_interval=0.05, timeout_s=0.2)
    assert c.register_instance(InstanceInfo(name="x", type="DEFAULT"), retries=2, backoff_s=0.01) is False
    assert c.heartbeat_once() is False and c.get_static_decode_list() == []
    c.start()
    time.sleep(0.2)
    c.stop()


# ------------------------------------------------------------------ two engines behind the router
@pytest.fixture(scope="module")
def cluster():
    svc = XllmService(policy="CAR", tokenizer=IdTokenizer(1024))
    sport, sstop = _serve(svc.register)
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    nodes, stops = [], [sstop]
    for i in range(2):
        port = _free_port()
        opts = Options(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=128, dtype="float32", port=port,
                       host="127.0.0.1", model_id="tiny-qwen2", enable_service_routing=True, etcd_addr=f"127.0.0.1:{sport}",
                       instance_name=f"node{i}", heart_beat_interval=0.05)
        eng = LLMEngine(opts, model_args=args, model=model)
        master = LLMMaster(opts, eng, IdTokenizer(args.vocab_size))
        master.run()
        api = APIService(master, opts)
        p2, stop = _serve(lambda srv, api=api: api.register(srv))
        # the API listens on p2, not on opts.port: tell the service where
        master.xservice.info.rpc_address = f"127.0.0.1:{p2}"
        master.xservice.register_instance(master.xservice.info)
        nodes.append(master)
        stops.append(stop)
    yield {"svc": svc, "url": f"http://127.0.0.1:{sport}", "nodes": nodes}
    for m in nodes:
        m.stop()
    for s in stops:
        s()


def test_router_sends_a_repeated_prompt_to_the_instance_that_cached_it(cluster):
    svc, url = cluster["svc"], cluster["url"]
    assert sorted(i["name"] for i in requests.get(url + "/xservice/instances").json()["instances"]) == ["node0", "node1"]
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, 1024, (64,), generator=g).tolist()
    body = {"model": "tiny-qwen2", "prompt": prompt, "max_tokens": 4, "temperature": 0}
    r1 = requests.post(url + "/v1/completions", json=body)
    assert r1.status_code == 200, r1.text
    first = r1.headers["X-Xllm-Instance"]
    text1 = r1.json()["choices"][0]["text"]
    # the instance reports the new prefix blocks with its next heartbeats
    deadline = time.time() + 5
    while time.time() < deadline and len(svc.registry.get(first).cached_keys) < 4:
        time.sleep(0.05)
    assert len(svc.registry.get(first).cached_keys) >= 4
    other = "node1" if first == "node0" else "node0"
    assert len(svc.registry.get(other).cached_keys) == 0
    for _ in range(3):
        r = requests.post(url + "/v1/completions", json=body)
        assert r.headers["X-Xllm-Instance"] == first and r.json()["choices"][0]["text"] == text1
        assert r.json()["usage"]["prompt_tokens"] == 64
    # a stream passes through the router unchanged
    with requests.post(url + "/v1/completions", json={**body, "stream": True}, stream=True) as rs:
        chunks = [l for l in rs.iter_lines() if l.startswith(b"data: ")]
    assert chunks[-1] == b"data: [DONE]" and len(chunks) >= 2
    # an unrelated prompt is free to go to the idle instance; both stay registered through all of it
    r = requests.post(url + "/v1/completions", json={**body, "prompt": torch.randint(0, 1024, (64,), generator=g).tolist()})
    assert r.status_code == 200
    info = requests.get(url + f"/xservice/instance?name={first}").json()
    assert info["load"]["cached_blocks"] >= 4 and info["load"]["inflight"] == 0
    assert requests.get(url + "/health").json()["instances"] == 2
    # the service's own listing and metrics, and a request without a generation phase
    models = requests.get(url + "/v1/models").json()["data"]
    assert models == [{"id": "tiny-qwen2", "object": "model", "owned_by": "xllm", "instances": 2}]
    emb = requests.post(url + "/v1/embeddings", json={"model": "tiny-qwen2", "input": [[1, 2, 3, 4]]})
    assert emb.status_code == 200 and len(emb.json()["data"]) == 1 and emb.headers["X-Xllm-Instance"] in ("node0", "node1")
    text = requests.get(url + "/metrics").text
    assert 'xllm_service_instances{type="DEFAULT"} 2' in text and f'xllm_service_forwarded_requests_total{{instance="{first}"}}' in text
    assert f'xllm_service_inflight_requests{{instance="{first}"}} 0' in text


def test_router_reports_unreachable_instances_and_empty_pools(cluster):
    svc = XllmService(policy="RR")
    port, stop = _serve(svc.register)
    try:
        url = f"http://127.0.0.1:{port}"
        r = requests.post(url + "/v1/completions", json={"prompt": [1, 2], "max_tokens": 1})
        assert r.status_code == 503
        svc.registry.register(InstanceInfo(name="ghost", type="DEFAULT", incarnation_id="g",
                                           rpc_address=f"127.0.0.1:{_free_port()}"), ttl_s=60)
        r = requests.post(url + "/v1/completions", json={"prompt": [1, 2], "max_tokens": 1})
        assert r.status_code == 503 and "unreachable" in r.json()["error"]["message"]
        assert svc.registry.get("ghost").inflight == 0
    finally:
        stop()


# ------------------------------------------------------------------ prefill instance follows the decode membership
def test_prefill_instance_links_and_drops_decode_instances_with_the_registry():
    """Two DECODE instances register with the service; a prefill instance that starts with no link finds them through the
    registry, connects to the control port each published, and serves a request through each.  When one registration goes
    away the link is dropped and only the other instance is used; when it returns it is linked again."""
    from xllm_wxh_b200.framework.params import RequestParams
    from xllm_wxh_b200.parallel.kv_transfer import LocalCopyTransfer
    from xllm_wxh_b200.runtime.disagg_pd import DecodeCoordinator, PrefillCoordinator
    from xllm_wxh_b200.runtime.pd_discovery import DecodeLinker
    svc = XllmService(policy="RR")
    sport, sstop = _serve(svc.register)
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)

    def opts(**kw):
        return Options(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=128, dtype="float32",
                       enable_disagg_pd=True, **kw)
    socks, d_masters, clients = [], {}, {}
    try:
        for i in range(2):
            eng = LLMEngine(opts(instance_role="DECODE", instance_name=f"d{i}"), model_args=args, model=model)
            dm = LLMMaster(eng.opt, eng)
            pd_port = _free_port()
            socks.append(DecodeCoordinator(dm).serve(pd_port))
            c = XServiceClient(f"127.0.0.1:{sport}", heart_beat_interval=0.05, ttl_s=30.0)
            assert c.register_instance(InstanceInfo(name=f"d{i}", type="DECODE", rpc_address=f"127.0.0.1:{_free_port()}",
                                                    pd_port=pd_port))
            d_masters[f"d{i}"], clients[f"d{i}"] = dm, c
        p_eng = LLMEngine(opts(instance_role="PREFILL"), model_args=args, model=model)
        p_master = LLMMaster(p_eng.opt, p_eng)
        pre = PrefillCoordinator(p_master)                       # no link yet
        out = []
        p_master.handle_request([1, 2, 3], RequestParams(max_tokens=2, request_id="early"), lambda o: out.append(o) or True)
        _wait(lambda: out and out[-1].finished)
        assert out[-1].status.code.name == "UNAVAILABLE" and "no decode instance" in out[-1].status.message

        def on_link(idx, info):                                  # CPU engines: KV blocks are copied between the two caches
            xfer = LocalCopyTransfer(p_eng.worker.kv_caches, d_masters[info.name].engine.worker.kv_caches)
            if idx == 0:
                p_eng.kv_transfer = xfer
            else:
                p_eng.kv_transfer_peers[idx] = xfer
        me = XServiceClient(f"127.0.0.1:{sport}")
        linker = DecodeLinker(pre, me, on_link=on_link)
        assert linker.sync_once() == {"d0": 0, "d1": 1}
        assert [l["info"]["instance_name"] for l in pre.links] == ["d0", "d1"]
        assert linker.sync_once() == {"d0": 0, "d1": 1}          # nothing new: no second link to the same instance
        assert len(pre.links) == 2

        def run(name, rid, n=4):
            res = []
            p_master.handle_request(list(range(5, 30)), RequestParams(temperature=0.0, max_tokens=n, ignore_eos=True,
                                                                      request_id=rid, decode_name=name),
                                    lambda o: res.append(o) or True)
            for _ in range(400):
                p_master.step()
                for dm in d_masters.values():
                    dm.step()
                if res and res[-1].finished:
                    break
                time.sleep(0.002)
            return res[-1]
        a, b = run("d0", "a"), run("d1", "b")
        assert a.finished and b.finished and a.status.ok and b.status.ok
        assert a.outputs[0].token_ids == b.outputs[0].token_ids and len(a.outputs[0].token_ids) == 4
        assert d_masters["d0"].engine.scheduler.stats()["generated_tokens"] == 3
        assert d_masters["d1"].engine.scheduler.stats()["generated_tokens"] == 3
        # d1 leaves the registry: its link is dropped, requests named for it are refused, d0 keeps serving
        clients["d1"].deregister()
        assert linker.sync_once() == {"d0": 0}
        assert not pre.links[1]["alive"]
        gone = run("d1", "c")
        assert gone.status.code.name == "UNAVAILABLE"
        assert run("d0", "d").status.ok
        # d1 registers again: a new link (index 2) is made
        assert clients["d1"].register_instance(clients["d1"].info)
        assert linker.sync_once() == {"d0": 0, "d1": 2}
        back = run("d1", "e")
        assert back.status.ok and back.outputs[0].token_ids == a.outputs[0].token_ids
        # the background thread does the same on its own
        linker.start(poll_s=0.2)
        clients["d0"].deregister()
        _wait(lambda: not pre.links[0]["alive"])
        linker.stop()
    finally:
        for s in socks:
            s.close()
        sstop()
