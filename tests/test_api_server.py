"""HTTP front-end against a tiny CPU model: completions, chat (plain, SSE, reasoning + tool-call deltas), Anthropic
messages, embeddings, models, health, metrics, rate limiting, error paths and cancel on client disconnect."""
import asyncio
import json
import socket
import threading
import time

import pytest
import requests
import torch

from oracle import greedy_generate
from xllm_wxh_b200.api.openai_service import APIService
from xllm_wxh_b200.api.server import HttpServer
from xllm_wxh_b200.config import Options
from xllm_wxh_b200.models.args import preset
from xllm_wxh_b200.models.qwen import QwenForCausalLM
from xllm_wxh_b200.runtime.engine import LLMEngine
from xllm_wxh_b200.runtime.master import LLMMaster
from xllm_wxh_b200.utils.tokenizer import IdTokenizer


class ScriptTokenizer(IdTokenizer):
    """Ids as text, except that decoding follows a script: token i of a reply decodes to `script[i]`, so that a
    random-weight model 'writes' think blocks and tool calls."""
    script = None
    slice_decodable = False          # what a token decodes to depends on its position in the reply

    def encode(self, text, add_special_tokens=True):
        return [int(t) % self._v for t in text.split() if t.isdigit()]

    def decode(self, ids, skip_special_tokens=True):
        if self.script is None:
            return super().decode(ids, skip_special_tokens)
        return "".join(self.script[i % len(self.script)] for i in range(len(ids)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.fixture(scope="module")
def server():
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    port = _free_port()
    opts = Options(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=256, dtype="float32", port=port,
                   host="127.0.0.1", max_concurrent_requests=4, model_id="tiny-qwen2", reasoning_parser="qwen3", tool_call_parser="qwen25")
    eng = LLMEngine(opts, model_args=args, model=model)
    tok = ScriptTokenizer(args.vocab_size)
    master = LLMMaster(opts, eng, tok)
    master.run()
    svc = APIService(master, opts)
    loop = asyncio.new_event_loop()
    ready = threading.Event()

    def run():
        asyncio.set_event_loop(loop)
        srv = svc.register(HttpServer())
        loop.run_until_complete(srv.start("127.0.0.1", port))
        ready.set()
        loop.run_forever()
    th = threading.Thread(target=run, daemon=True)
    th.start()
    assert ready.wait(10)
    yield {"url": f"http://127.0.0.1:{port}", "args": args, "sd": model.state_dict(), "tok": tok, "svc": svc, "master": master}
    loop.call_soon_threadsafe(loop.stop)
    th.join(5)
    master.stop()


def _sse(resp):
    events = []
    for line in resp.iter_lines():
        if line.startswith(b"data: "):
            data = line[6:].decode()
            events.append(data if data == "[DONE]" else json.loads(data))
    return events


def test_models_health_metrics(server):
    u = server["url"]
    r = requests.get(u + "/v1/models").json()
    assert r["data"][0]["id"] == "tiny-qwen2"
    assert requests.get(u + "/health").status_code == 200
    assert requests.get(u + "/v2/repository/index").status_code == 200
    m = requests.get(u + "/metrics")
    assert m.status_code == 200 and "text/plain" in m.headers["content-type"]
    assert requests.get(u + "/nope").status_code == 404
    assert requests.post(u + "/v1/models").status_code == 405


def test_completion_matches_oracle(server):
    prompt = torch.randint(0, 1024, (20,), generator=torch.Generator().manual_seed(1)).tolist()
    r = requests.post(server["url"] + "/v1/completions", json={
        "model": "tiny-qwen2", "prompt": " ".join(map(str, prompt)), "max_tokens": 12, "temperature": 0, "ignore_eos": True, "logprobs": 2})
    assert r.status_code == 200, r.text
    body = r.json()
    want = greedy_generate(server["sd"], server["args"], prompt, 12)
    assert body["choices"][0]["text"] == "".join(f" {t}" for t in want)
    assert body["choices"][0]["finish_reason"] == "length"
    assert body["usage"] == {"prompt_tokens": 20, "completion_tokens": 12, "total_tokens": 32, "prompt_tokens_details": {"cached_tokens": 0}}
    lp = body["choices"][0]["logprobs"]
    assert len(lp["tokens"]) == 12 and all(len(t) == 2 for t in lp["top_logprobs"])


def test_completion_stream_and_usage(server):
    prompt = torch.randint(0, 1024, (10,), generator=torch.Generator().manual_seed(2)).tolist()
    r = requests.post(server["url"] + "/v1/completions", stream=True, json={
        "prompt": " ".join(map(str, prompt)), "max_tokens": 8, "temperature": 0, "ignore_eos": True, "stream": True,
        "stream_options": {"include_usage": True}})
    ev = _sse(r)
    assert ev[-1] == "[DONE]"
    text = "".join(c["text"] for e in ev[:-1] for c in e.get("choices", []))
    want = greedy_generate(server["sd"], server["args"], prompt, 8)
    assert text == "".join(f" {t}" for t in want)
    assert ev[-2]["usage"]["completion_tokens"] == 8
    finals = [c["finish_reason"] for e in ev[:-1] for c in e.get("choices", []) if c["finish_reason"]]
    assert finals == ["length"]


def test_bad_requests(server):
    u = server["url"]
    assert requests.post(u + "/v1/completions", json={"max_tokens": 3}).status_code == 400
    assert requests.post(u + "/v1/completions", data="{not json").status_code == 400
    assert requests.post(u + "/v1/completions", json={"prompt": "1 2", "model": "other"}).status_code == 404
    r = requests.post(u + "/v1/completions", json={"prompt": "1 2", "max_tokens": 2, "top_p": 7.0})
    assert r.status_code == 400 and "top_p" in r.json()["error"]["message"]
    assert requests.post(u + "/v1/messages", json={"messages": [{"role": "user", "content": "1"}]}).status_code == 400


def test_chat_reasoning_and_tool_calls(server):
    tok = server["tok"]
    call = '{"name": "get_weather", "arguments": {"city": "Paris"}}'
    pieces = ["<think>", "hm", "m</think>", "Sure.", "<tool_call>\n"] + [call[i:i + 5] for i in range(0, len(call), 5)] + ["\n</tool_call>"]
    tok.script = pieces
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}}]
    try:
        body = {"messages": [{"role": "user", "content": "5 6 7"}], "max_tokens": len(pieces), "temperature": 0, "ignore_eos": True, "tools": tools}
        r = requests.post(server["url"] + "/v1/chat/completions", json=body)
        assert r.status_code == 200, r.text
        ch = r.json()["choices"][0]
        assert ch["message"]["reasoning_content"] == "hmm"
        assert ch["message"]["content"] == "Sure."
        tc = ch["message"]["tool_calls"][0]
        assert tc["function"]["name"] == "get_weather" and json.loads(tc["function"]["arguments"]) == {"city": "Paris"}
        assert ch["finish_reason"] in ("tool_calls", "length")

        r = requests.post(server["url"] + "/v1/chat/completions", json=dict(body, stream=True), stream=True)
        ev = _sse(r)
        assert ev[-1] == "[DONE]"
        deltas = [c["delta"] for e in ev[:-1] for c in e["choices"]]
        assert deltas[0].get("role") == "assistant"
        assert "".join(d.get("reasoning_content", "") for d in deltas) == "hmm"
        assert "".join(d.get("content") or "" for d in deltas) == "Sure."
        calls = [t for d in deltas for t in d.get("tool_calls", [])]
        assert calls[0]["function"]["name"] == "get_weather" and calls[0]["id"]
        assert json.loads("".join(t["function"]["arguments"] for t in calls)) == {"city": "Paris"}
    finally:
        tok.script = None


def test_anthropic_messages(server):
    body = {"model": "tiny-qwen2", "max_tokens": 5, "temperature": 0, "system": "9", "messages": [{"role": "user", "content": [{"type": "text", "text": "1 2 3"}]}]}
    r = requests.post(server["url"] + "/v1/messages", json=body)
    assert r.status_code == 200, r.text
    m = r.json()
    assert m["type"] == "message" and m["role"] == "assistant" and m["content"][0]["type"] == "text"
    assert m["usage"]["output_tokens"] <= 5 and m["stop_reason"] in ("max_tokens", "end_turn")
    r = requests.post(server["url"] + "/v1/messages", json=dict(body, stream=True), stream=True)
    names = [l[7:].decode() for l in r.iter_lines() if l.startswith(b"event: ")]
    assert names[0] == "message_start" and names[1] == "content_block_start" and names[-1] == "message_stop"
    assert "content_block_delta" in names and names[-2] == "message_delta"


def test_embeddings(server):
    r = requests.post(server["url"] + "/v1/embeddings", json={"input": ["1 2 3 4", "9 8 7"]})
    assert r.status_code == 200, r.text
    d = r.json()["data"]
    assert len(d) == 2 and len(d[0]["embedding"]) == server["args"].hidden_size
    assert abs(sum(x * x for x in d[0]["embedding"]) - 1.0) < 1e-3


def test_sample_endpoint(server):
    ids = torch.randint(0, 1024, (12,), generator=torch.Generator().manual_seed(5)).tolist()
    ids[4] = ids[9] = 1000
    r = requests.post(server["url"] + "/v1/sample", json={"model": "tiny-qwen2", "prompt": " ".join(map(str, ids)),
                                                          "selector": "1000", "logprobs": 4})
    assert r.status_code == 200, r.text
    samples = r.json()["data"][0]["samples"]
    assert [s["sample_id"] for s in samples] == [0, 1]
    for s, end in zip(samples, (5, 10)):
        assert s["token_ids"] == greedy_generate(server["sd"], server["args"], ids[:end], 1)
        assert len(s["top_logprobs"]) == 4
    bad = requests.post(server["url"] + "/v1/sample", json={"prompt": "1 2", "selector": "3 4"})
    assert bad.status_code == 400


def test_rate_limit(server):
    lim = server["svc"].limiter
    for _ in range(4):
        assert lim.acquire()
    try:
        r = requests.post(server["url"] + "/v1/completions", json={"prompt": "1 2 3", "max_tokens": 2})
        assert r.status_code == 429
    finally:
        for _ in range(4):
            lim.release()
    assert requests.post(server["url"] + "/v1/completions", json={"prompt": "1 2 3", "max_tokens": 2}).status_code == 200


def test_metrics_catalogue_after_traffic(server):
    """After some requests `/metrics` carries the reference's catalogue (core/common/metrics.h:110-210) in Prometheus text
    form: request counters, token counters and per-request histograms, latency histograms, scheduler and KV gauges."""
    u = server["url"]
    requests.post(u + "/v1/completions", json={"model": "tiny-qwen2", "prompt": "1 2 3 4 5", "max_tokens": 3})
    text = requests.get(u + "/metrics").text
    for name in ("server_request_in_total", "server_request_total_ok", "request_status_total", "prompt_tokens_total",
                 "generated_tokens_total", "num_prompt_tokens_per_request_count", "num_generated_tokens_per_request_count",
                 "time_to_first_token_latency_milliseconds_count", "end_2_end_latency_milliseconds_count",
                 "scheduling_latency_seconds_count", "execution_latency_seconds_model_count", "engine_latency_seconds_count",
                 "tokenization_latency_seconds_count", "num_running_requests", "num_waiting_requests", "num_pending_requests",
                 "num_preempted_requests", "num_running_sequences", "kv_cache_utilization_perc", "num_free_blocks",
                 "num_used_blocks", "num_blocks_in_prefix_cache", "prefix_cache_block_matched_rate", "num_concurrent_requests",
                 "weight_size_in_kilobytes", "total_kv_cache_size_in_kilobytes"):
        assert ("\n" + name) in ("\n" + text), name
    assert "# TYPE time_to_first_token_latency_milliseconds histogram" in text


def test_disconnect_cancels_stream(server):
    u = server["url"]
    r = requests.post(u + "/v1/completions", stream=True, json={"prompt": "1 2 3", "max_tokens": 900, "ignore_eos": True, "stream": True})
    it = r.iter_lines()
    next(it)
    r.close()
    eng = server["master"].engine
    deadline = time.time() + 20
    while eng.has_unfinished() and time.time() < deadline:
        time.sleep(0.05)
    assert not eng.has_unfinished(), "the request of a vanished client keeps running"
    assert server["svc"].limiter.cur == 0
