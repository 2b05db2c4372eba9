"""Sleep / wake-up of an idle engine: device memory is released (KV cache, graphs, weights to host or dropped) and comes
back with identical behaviour; requests are refused while asleep.  Reference: master.h:38-55, llm_engine.cpp:1252-1350,
api_service.cpp:977-1130."""
import asyncio
import socket
import threading

import pytest
import requests
import torch

from oracle import greedy_generate
from xllm_wxh_b200 import LLM, SamplingParams
from xllm_wxh_b200.api.openai_service import APIService, RateLimiter
from xllm_wxh_b200.api.server import HttpServer
from xllm_wxh_b200.config import Options
from xllm_wxh_b200.models.args import preset
from xllm_wxh_b200.models.qwen import QwenForCausalLM
from xllm_wxh_b200.runtime.engine import LLMEngine
from xllm_wxh_b200.runtime.master import LLMMaster
from xllm_wxh_b200.runtime.sleep import iter_weight_slots
from xllm_wxh_b200.utils.tokenizer import IdTokenizer


def _engine(**kw):
    args = preset("tiny-qwen2")
    opts = dict(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=64, dtype="float32", random_seed=0)
    opts.update(kw)
    return args, LLMEngine(Options(**opts), model_args=args)


def _prompts(n=3, length=40, seed=2):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 1024, (length,), generator=g).tolist() for _ in range(n)]


def test_weight_walker_finds_every_tensor_once_per_slot():
    args, eng = _engine()
    m = eng.worker.model
    slots = list(iter_weight_slots(m))
    tensors = [g() for g, _ in slots if g() is not None]
    total = sum(t.numel() * t.element_size() for t in {t.data_ptr(): t for t in tensors}.values())
    assert total == m.weight_bytes()
    assert any(g() is m.embed for g, _ in slots) and any(g() is m.layers[-1].mlp.down_w for g, _ in slots)


@pytest.mark.parametrize("level", [1, 2])
def test_sleep_releases_memory_and_wakeup_restores_behaviour(level):
    args, eng = _engine(host_blocks_factor=2.0)
    llm = LLM(model="preset:tiny-qwen2", devices="cpu", engine=eng)
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    prompts = _prompts()
    before = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    weight_bytes = eng.worker.model.weight_bytes()
    kv_bytes = sum(t.numel() * t.element_size() for layer in eng.worker.kv_caches for t in layer)
    assert eng.sleep(3) is False                                  # unknown level
    assert eng.sleep(level) is True and eng.sleep_level == level
    assert eng.sleep(level) is False                              # already asleep
    assert eng.bytes_released_by_sleep == weight_bytes + kv_bytes
    assert eng.worker.kv_caches == []
    if level == 2:
        assert eng.worker.model.embed is None and eng.worker.model.layers[0].attn.qkv_w is None
    bm = eng.scheduler.block_manager(0)
    assert bm.num_blocks_in_prefix_cache == 0                     # the device copies are gone ...
    assert len(eng.scheduler.host_manager(0).match(prompts[0])) == 2      # ... the host tier still has the prefixes
    eng.scheduler.host_manager(0).release(eng.scheduler.host_manager(0).match(prompts[0]) * 2)
    eng.add_request(prompts[0])
    with pytest.raises(RuntimeError):
        eng.step()                                                # no forward without memory
    for rid in eng.scheduler.waiting_ids():
        eng.cancel(rid)
    assert eng.wakeup() is True and eng.sleep_level == 0 and eng.wakeup() is False
    while eng.has_unfinished():
        eng.step()
    loaded0 = eng.scheduler.stats()["host_loaded_blocks"]
    after = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert after == before
    assert eng.scheduler.stats()["host_loaded_blocks"] > loaded0   # prefixes came back from host memory, not recomputed
    assert eng.worker.model.weight_bytes() == weight_bytes


def test_engine_with_work_in_flight_does_not_fall_asleep():
    args, eng = _engine()
    eng.add_request(_prompts(1)[0])
    eng.step()
    assert eng.sleep(1) is False and eng.sleep_level == 0
    while eng.has_unfinished():
        eng.step()
    assert eng.sleep(1) is True
    eng.wakeup()


def test_rate_limiter_sleep_gate():
    r = RateLimiter(4)
    assert r.acquire()
    assert r.try_set_sleeping() is False          # a request is in flight
    r.release()
    assert r.try_set_sleeping() is True and r.try_set_sleeping() is False
    assert r.acquire() is False                   # nothing is admitted while asleep
    assert r.try_wakeup() is True and r.try_wakeup() is False
    assert r.acquire()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_sleep_and_wakeup_over_http():
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    port = _free_port()
    opts = Options(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=64, dtype="float32", port=port,
                   host="127.0.0.1", model_id="tiny-qwen2")
    master = LLMMaster(opts, LLMEngine(opts, model_args=args, model=model), IdTokenizer(args.vocab_size))
    master.run()
    api = APIService(master, opts)
    loop = asyncio.new_event_loop()
    ready = threading.Event()

    def run():
        asyncio.set_event_loop(loop)
        srv = api.register(HttpServer())
        loop.run_until_complete(srv.start("127.0.0.1", port))
        ready.set()
        loop.run_forever()
    th = threading.Thread(target=run, daemon=True)
    th.start()
    assert ready.wait(10)
    url = f"http://127.0.0.1:{port}"
    try:
        body = {"model": "tiny-qwen2", "prompt": "1 2 3 4 5 6 7 8", "max_tokens": 4, "temperature": 0}
        t1 = requests.post(url + "/v1/completions", json=body).json()["choices"][0]["text"]
        assert requests.post(url + "/wakeup", json={}).status_code == 409          # not sleeping
        assert requests.post(url + "/sleep", json={"master_status": 7}).status_code == 400
        r = requests.post(url + "/sleep", json={"master_status": "LIGHT_SLEEP"})
        assert r.status_code == 200 and r.json()["bytes_released"] > 0 and master.is_sleeping()
        assert requests.post(url + "/sleep", json={"master_status": 1}).status_code == 409
        assert requests.post(url + "/v1/completions", json=body).status_code == 503
        assert requests.get(url + "/health").status_code == 200
        assert requests.post(url + "/wakeup", json={}).status_code == 200 and not master.is_sleeping()
        assert requests.post(url + "/v1/completions", json=body).json()["choices"][0]["text"] == t1
        # weight sessions: a served instance links and unlinks; an unreachable one is reported
        from xllm_wxh_b200.runtime.weight_transfer import WeightServer
        wport = _free_port()
        ws = WeightServer(master)
        ws.serve(wport, "127.0.0.1")
        try:
            assert requests.post(url + "/link_d2d", json={}).status_code == 400
            r = requests.post(url + "/link_d2d", json={"device_ips": [f"127.0.0.1:{wport}"]})
            assert r.status_code == 200 and r.json()["linked"] == [f"127.0.0.1:{wport}"]
            assert requests.post(url + "/sleep", json={"master_status": 2}).status_code == 200
            # its own weight service sleeps with it, so this wake-up reads the preset again; the call shape is what is checked
            r = requests.post(url + "/wakeup", json={"remote_addrs": [f"127.0.0.1:{wport}"]})
            assert r.status_code == 200 and r.json()["weights_pulled_bytes"] == 0
            r = requests.post(url + "/unlink_d2d", json={"device_ips": [f"127.0.0.1:{wport}"]})
            assert r.json()["unlinked"] == 1 and r.json()["linked"] == []
            assert requests.post(url + "/link_d2d", json={"device_ips": [f"127.0.0.1:{_free_port()}"]}).status_code == 502
        finally:
            ws.close()
    finally:
        loop.call_soon_threadsafe(loop.stop)
        th.join(5)
        master.stop()


def _write_checkpoint(path, seed):
    """A qwen2 checkpoint directory in the HF layout with random weights."""
    import json
    from xllm_wxh_b200.utils.safetensors_io import save_safetensors
    args = preset("tiny-qwen2")
    m = QwenForCausalLM(args, device="cpu").init_random(seed=seed)
    path.mkdir()
    save_safetensors(str(path / "model.safetensors"), m.state_dict())
    (path / "config.json").write_text(json.dumps({
        "model_type": "qwen2", "hidden_size": args.hidden_size, "num_hidden_layers": args.n_layers,
        "num_attention_heads": args.n_heads, "num_key_value_heads": args.n_kv_heads,
        "intermediate_size": args.intermediate_size, "vocab_size": args.vocab_size, "rms_norm_eps": args.rms_norm_eps,
        "rope_theta": args.rope_theta, "max_position_embeddings": args.max_position_embeddings,
        "tie_word_embeddings": args.tie_word_embeddings, "head_dim": args.head_dim, "torch_dtype": "float32"}))
    return m


def test_fork_master_serves_a_second_model_by_turns(tmp_path):
    """POST /fork_master loads a second checkpoint beside the first model; requests reach the model they name; each model
    sleeps and wakes on its own; a forked model that starts asleep answers 503 until it is woken."""
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    second = _write_checkpoint(tmp_path / "second-model", seed=11)
    _write_checkpoint(tmp_path / "third-model", seed=12)
    port = _free_port()
    opts = Options(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=64, dtype="float32", port=port,
                   host="127.0.0.1", model_id="tiny-qwen2")
    master = LLMMaster(opts, LLMEngine(opts, model_args=args, model=model), IdTokenizer(args.vocab_size))
    master.run()
    api = APIService(master, opts)
    loop = asyncio.new_event_loop()
    ready = threading.Event()

    def run():
        asyncio.set_event_loop(loop)
        srv = api.register(HttpServer())
        loop.run_until_complete(srv.start("127.0.0.1", port))
        ready.set()
        loop.run_forever()
    th = threading.Thread(target=run, daemon=True)
    th.start()
    assert ready.wait(10)
    url = f"http://127.0.0.1:{port}"
    prompt = list(range(3, 40))

    def ask(model_id):
        return requests.post(url + "/v1/completions", json={"model": model_id, "prompt": prompt, "max_tokens": 6, "temperature": 0})
    try:
        assert requests.post(url + "/fork_master", json={}).status_code == 400
        assert requests.post(url + "/fork_master", json={"model_path": str(tmp_path / "missing")}).status_code == 400
        assert ask("second-model").status_code == 404                               # not forked yet
        r = requests.post(url + "/fork_master", json={"model_path": str(tmp_path / "second-model"), "num_kv_blocks": 48})
        assert r.status_code == 200 and r.json()["model_id"] == "second-model" and r.json()["server_idx"] >= 1
        again = requests.post(url + "/fork_master", json={"model_path": str(tmp_path / "second-model")})
        assert again.status_code == 200 and "already exists" in again.json()["message"] and len(api.children) == 1
        ids = {m["id"]: m for m in requests.get(url + "/v1/models").json()["data"]}
        assert set(ids) == {"tiny-qwen2", "second-model"} and not ids["second-model"]["sleeping"]
        child = api.children["second-model"].master
        assert child.engine.num_blocks == 48 and child.opt.port == opts.port
        a, b = ask("tiny-qwen2"), ask("second-model")
        assert a.status_code == 200 and b.status_code == 200
        assert a.json()["model"] == "tiny-qwen2" and b.json()["model"] == "second-model"
        # the second model really is another set of weights: its answer equals its own greedy continuation
        from xllm_wxh_b200 import LLM, SamplingParams
        eng2 = LLMEngine(Options(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=64, dtype="float32"),
                         model_args=args, model=second)
        want = LLM(model="preset:tiny-qwen2", devices="cpu", engine=eng2).generate(
            [prompt], SamplingParams(temperature=0.0, max_tokens=6))[0].outputs[0].token_ids
        got = child.tokenizer.encode(b.json()["choices"][0]["text"]) if hasattr(child.tokenizer, "encode") else None
        assert got == want
        assert a.json()["choices"][0]["text"] != b.json()["choices"][0]["text"]
        # by turns: the first model sleeps while the second serves, then the other way round
        assert requests.post(url + "/sleep", json={"model_id": "tiny-qwen2", "master_status": 1}).status_code == 200
        assert master.is_sleeping() and not child.is_sleeping()
        assert ask("tiny-qwen2").status_code == 503 and ask("second-model").json()["choices"][0]["text"] == b.json()["choices"][0]["text"]
        assert requests.post(url + "/sleep", json={"model_id": "second-model", "master_status": 2}).status_code == 200
        assert requests.post(url + "/wakeup", json={"model_id": "tiny-qwen2"}).status_code == 200
        assert ask("tiny-qwen2").json()["choices"][0]["text"] == a.json()["choices"][0]["text"]
        assert ask("second-model").status_code == 503
        # a deep sleep dropped the second model's weights; the wake-up reads its checkpoint again
        assert requests.post(url + "/wakeup", json={"model_id": "second-model"}).status_code == 200
        assert ask("second-model").json()["choices"][0]["text"] == b.json()["choices"][0]["text"]
        # a model forked asleep
        r = requests.post(url + "/fork_master", json={"model_path": str(tmp_path / "third-model"), "master_status": "LIGHT_SLEEP"})
        assert r.status_code == 200 and api.children["third-model"].master.is_sleeping()
        assert ask("third-model").status_code == 503
        assert requests.post(url + "/wakeup", json={"model_id": "third-model"}).status_code == 200
        assert ask("third-model").status_code == 200
    finally:
        loop.call_soon_threadsafe(loop.stop)
        th.join(5)
        for c in api.children.values():
            c.master.stop()
        master.stop()


def test_deep_sleeper_wakes_up_from_the_weights_of_an_awake_instance(tmp_path):
    """Two instances of one checkpoint.  The second one sleeps deeply, its checkpoint directory is then emptied, and it still
    wakes up: the weights come from the first instance's weight service (layout compared first, then the bytes).  A source
    with another layout is refused and the sleeper falls back to its checkpoint."""
    import os
    from xllm_wxh_b200 import LLM, SamplingParams
    from xllm_wxh_b200.runtime.weight_transfer import WeightPuller, WeightServer
    _write_checkpoint(tmp_path / "m", seed=21)

    def make():
        o = Options(model=str(tmp_path / "m"), devices="cpu", block_size=16, num_kv_blocks=64, dtype="float32")
        e = LLMEngine(o)
        return LLMMaster(o, e, IdTokenizer(e.args.vocab_size))
    a, b = make(), make()
    port = _free_port()
    srv = WeightServer(a)
    srv.serve(port, "127.0.0.1")
    sp = SamplingParams(temperature=0.0, max_tokens=6)
    prompt = list(range(7, 50))

    def tokens(master):
        llm = LLM(model="x", devices="cpu", engine=master.engine)
        llm.master = master
        return llm.generate([prompt], sp)[0].outputs[0].token_ids
    try:
        want = tokens(b)
        assert want == tokens(a)
        assert b.sleep(2) and b.is_sleeping()
        hidden = tmp_path / "m" / "model.safetensors"
        os.rename(hidden, tmp_path / "moved.safetensors")          # the checkpoint can no longer be read
        addr = f"127.0.0.1:{port}"
        assert list(b.link_d2d([addr])) == [addr] and isinstance(b.weight_sources[addr], WeightPuller)
        assert b.wakeup([addr]) and not b.is_sleeping()
        pulled = b.weight_sources[addr].bytes_pulled
        n_bytes = sum(p.numel() * p.element_size() for p in {id(t): t for t in a.engine.worker.model.state_dict().values()}.values())
        assert pulled > 0 and pulled == srv.bytes_served == b.engine.weights_pulled_bytes and pulled >= 0.9 * n_bytes
        assert tokens(b) == want
        # tied weights stay tied after the pull
        m = b.engine.worker.model
        assert m.lm_head.data_ptr() == m.embed.data_ptr()
        # light sleep does not need a source, and ignores one
        assert b.sleep(1) and b.wakeup([addr]) and b.weight_sources[addr].bytes_pulled == pulled and tokens(b) == want
        # a source that sleeps holds no weights: the sleeper reads its checkpoint (restored here) instead
        os.rename(tmp_path / "moved.safetensors", hidden)
        assert b.sleep(2) and a.sleep(2)
        assert b.wakeup([addr]) and b.weight_sources[addr].bytes_pulled == pulled and b.engine.weights_pulled_bytes == 0
        assert tokens(b) == want
        assert a.wakeup() and tokens(a) == want
        # an unreachable source is skipped
        assert b.sleep(2) and b.wakeup([f"127.0.0.1:{_free_port()}", addr]) and b.engine.weights_pulled_bytes == pulled
        assert b.unlink_d2d([addr]) == 1 and b.weight_sources == {}
    finally:
        srv.close()
        a.stop()
        b.stop()


@pytest.mark.gpu
@pytest.mark.parametrize("level", [1, 2])
def test_sleep_frees_device_memory_on_gpu(level):
    from xllm_wxh_b200.models.args import ModelArgs
    args = ModelArgs(model_type="qwen3", vocab_size=2048, hidden_size=512, n_layers=3, n_heads=8, n_kv_heads=2, head_dim=128,
                     intermediate_size=1536, qk_norm=True, rope_theta=1e6, max_position_embeddings=4096, dtype="bfloat16")
    eng = LLMEngine(Options(model="preset:x", devices="cuda:0", block_size=16, num_kv_blocks=256, host_blocks_factor=1.0,
                            max_tokens_per_batch=2048, max_seqs_per_batch=64, random_seed=0), model_args=args)
    llm = LLM(model="preset:x", devices="cuda:0", engine=eng)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    prompts = _prompts(4, 80)
    before = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    before2 = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]        # graphs captured on the second sighting
    assert before2 == before
    torch.cuda.synchronize()
    used = torch.cuda.memory_allocated()
    assert eng.sleep(level)
    released = used - torch.cuda.memory_allocated()
    assert released >= 0.9 * eng.bytes_released_by_sleep > 0
    assert eng.wakeup()
    after = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    same = sum(x == y for a, b in zip(after, before) for x, y in zip(a, b))
    assert same >= 0.9 * sum(len(a) for a in before)          # bf16: a prompt split at a loaded prefix may flip a near-tie
    assert eng.scheduler.stats()["host_loaded_blocks"] > 0
    from xllm_wxh_b200.ops import cuda_ops
    assert cuda_ops.read_status() == 0
    llm.finish()


@pytest.mark.gpu
def test_deep_sleeper_pulls_weights_over_cuda_ipc(tmp_path):
    """An awake instance in another process (on the second GPU when there is one) serves its weights; this process holds
    a model with other weights, sleeps deeply and wakes up from the source: device-to-device copies through CUDA-IPC
    mappings, after which its greedy tokens are those of the source's model."""
    import os
    import subprocess
    import sys
    import time
    import torch
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(here, "helpers"))
    import weight_source_worker as wsw
    port = _free_port()
    out = str(tmp_path / "source.pt")
    src_gpu = 1 if torch.cuda.device_count() > 1 else 0
    proc = subprocess.Popen([sys.executable, os.path.join(here, "helpers", "weight_source_worker.py"), str(src_gpu), str(port), out],
                            env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    try:
        master = wsw.make(0, seed=9)
        mine = wsw.tokens(master)
        deadline = time.time() + 120
        while not os.path.exists(out):
            assert proc.poll() is None and time.time() < deadline, "the weight source did not come up"
            time.sleep(0.05)
        want = torch.load(out)["tokens"]
        assert mine != want                                   # other weights before the pull
        assert master.sleep(2)
        free_asleep = torch.cuda.mem_get_info(0)[0]
        assert master.wakeup([f"127.0.0.1:{port}"]) and not master.is_sleeping()
        eng = master.engine
        assert eng.weights_pulled_bytes > 0 and torch.cuda.mem_get_info(0)[0] < free_asleep
        print(f"weight pull: {eng.weights_pulled_bytes / 1e9:.3f} GB in {eng.weights_pull_ms:.3f} ms of device time "
              f"({eng.weights_pulled_bytes / 1e6 / max(eng.weights_pull_ms, 1e-6):.1f} GB/s), source on GPU {src_gpu}")
        assert wsw.tokens(master) == want
        from xllm_wxh_b200.ops import cuda_ops
        assert cuda_ops.read_status() == 0
        master.stop()
    finally:
        open(out + ".stop", "w").close()
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
