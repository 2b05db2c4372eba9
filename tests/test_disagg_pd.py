"""Prefill / decode disaggregation: a PREFILL engine and a DECODE engine in one process (in-process transport, tensor
copies for the KV blocks).  Tokens must equal those of a single colocated engine."""
import pytest
import torch

from xllm_wxh_b200 import LLM, SamplingParams
from xllm_wxh_b200.config import Options
from xllm_wxh_b200.models.args import preset
from xllm_wxh_b200.models.qwen import QwenForCausalLM
from xllm_wxh_b200.parallel.kv_transfer import LocalCopyTransfer
from xllm_wxh_b200.runtime.disagg_pd import DecodeCoordinator, InProcTransport, PrefillCoordinator
from xllm_wxh_b200.runtime.engine import LLMEngine
from xllm_wxh_b200.runtime.master import LLMMaster


def _opts(**kw):
    o = dict(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=128, dtype="float32")
    o.update(kw)
    return Options(**o)


def test_pd_pair_matches_colocated_engine():
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (20, 45, 7, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in
            LLM(model="preset:tiny-qwen2", devices="cpu", engine=LLMEngine(_opts(), model_args=args, model=model)).generate(prompts, sp)]

    p_eng = LLMEngine(_opts(enable_disagg_pd=True, instance_role="PREFILL"), model_args=args, model=model)
    d_eng = LLMEngine(_opts(enable_disagg_pd=True, instance_role="DECODE"), model_args=args, model=model)
    p_master, d_master = LLMMaster(p_eng.opt, p_eng), LLMMaster(d_eng.opt, d_eng)
    tp, td = InProcTransport.pair()
    dec = DecodeCoordinator(d_master)
    dec.attach(td)
    pre = PrefillCoordinator(p_master, tp)
    p_eng.kv_transfer = LocalCopyTransfer(p_eng.worker.kv_caches, d_eng.worker.kv_caches)
    p_master.idle_wait = lambda: d_master.step()

    llm = LLM(model="preset:tiny-qwen2", devices="cpu", engine=p_eng)
    llm.master = p_master
    outs = llm.generate(prompts, sp)
    got = [o.outputs[0].token_ids for o in outs]
    assert got == want
    assert all(o.outputs[0].finish_reason == "length" for o in outs)
    assert p_eng.kv_transfer.bytes_moved > 0
    # the prefill instance never decoded: every request left it after one token
    assert p_eng.scheduler.stats()["generated_tokens"] == len(prompts)
    # all blocks returned on both sides
    assert d_eng.scheduler.block_manager(0).num_used_blocks == 0 and p_eng.scheduler.block_manager(0).num_used_blocks == 0


def test_pd_pull_mode_decode_instance_fetches_the_blocks():
    """`--kv_cache_transfer_mode PULL`: the prefill instance pushes nothing; `first_generation` names its blocks and the
    decode instance copies them before it activates the request.  Chunked prompts, same tokens as a colocated engine."""
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (50, 9, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in
            LLM(model="preset:tiny-qwen2", devices="cpu", engine=LLMEngine(_opts(), model_args=args, model=model)).generate(prompts, sp)]
    kw = dict(enable_disagg_pd=True, kv_cache_transfer_mode="PULL", max_tokens_per_chunk_for_prefill=16, max_tokens_per_batch=32)
    p_eng = LLMEngine(_opts(instance_role="PREFILL", **kw), model_args=args, model=model)
    d_eng = LLMEngine(_opts(instance_role="DECODE", **kw), model_args=args, model=model)
    p_master, d_master = LLMMaster(p_eng.opt, p_eng), LLMMaster(d_eng.opt, d_eng)
    tp, td = InProcTransport.pair()
    dec = DecodeCoordinator(d_master)
    dec.attach(td)
    pre = PrefillCoordinator(p_master, tp)
    assert pre.pull
    d_eng.kv_sources[0] = LocalCopyTransfer(p_eng.worker.kv_caches, d_eng.worker.kv_caches)
    p_master.idle_wait = lambda: d_master.step()
    llm = LLM(model="preset:tiny-qwen2", devices="cpu", engine=p_eng)
    llm.master = p_master
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == want
    assert p_eng.kv_transfer is None and d_eng.kv_sources[0].bytes_moved > 0
    assert not dec._reserved
    assert d_eng.scheduler.block_manager(0).num_used_blocks == 0 and p_eng.scheduler.block_manager(0).num_used_blocks == 0


def test_pd_long_prompts_leave_chunk_by_chunk_and_layer_by_layer():
    """A prompt prefilled in several chunks: each chunk's blocks are pushed in the step that computes them (the partly
    filled block again with the next chunk), every layer right after its attention; with a prefix that the prefill side
    already caches, the cached blocks travel with the first chunk.  Tokens equal those of a colocated engine."""
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, args.vocab_size, (40,), generator=g).tolist()
    prompts = [shared + torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (37, 5)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in
            LLM(model="preset:tiny-qwen2", devices="cpu", engine=LLMEngine(_opts(), model_args=args, model=model)).generate(prompts, sp)]
    kw = dict(enable_disagg_pd=True, max_tokens_per_chunk_for_prefill=16, max_tokens_per_batch=32)
    p_eng = LLMEngine(_opts(instance_role="PREFILL", **kw), model_args=args, model=model)
    d_eng = LLMEngine(_opts(instance_role="DECODE", **kw), model_args=args, model=model)
    p_master, d_master = LLMMaster(p_eng.opt, p_eng), LLMMaster(d_eng.opt, d_eng)
    tp, td = InProcTransport.pair()
    DecodeCoordinator(d_master).attach(td)
    PrefillCoordinator(p_master, tp)
    calls = []

    class Recording(LocalCopyTransfer):
        def push(self, pairs, layer=-1):
            calls.append((layer, len(pairs)))
            super().push(pairs, layer)
    p_eng.kv_transfer = Recording(p_eng.worker.kv_caches, d_eng.worker.kv_caches)
    p_master.idle_wait = lambda: d_master.step()
    llm = LLM(model="preset:tiny-qwen2", devices="cpu", engine=p_eng)
    llm.master = p_master
    got = [o.outputs[0].token_ids for o in llm.generate([prompts[0]], sp)]
    got += [o.outputs[0].token_ids for o in llm.generate([prompts[1]], sp)]      # its first 32 tokens are cached on the prefill side
    assert got == want
    n_layers = args.n_layers
    assert all(0 <= layer < n_layers for layer, _ in calls), "pushes go layer by layer"
    steps = len(calls) // n_layers
    assert steps >= 5 + 1                       # 77 tokens in 16-token chunks, then the second prompt's remaining tokens
    assert d_eng.scheduler.block_manager(0).num_used_blocks == 0 and p_eng.scheduler.block_manager(0).num_used_blocks == 0


def test_pd_decode_refuses_when_out_of_blocks():
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    p_eng = LLMEngine(_opts(enable_disagg_pd=True, instance_role="PREFILL"), model_args=args, model=model)
    d_eng = LLMEngine(_opts(enable_disagg_pd=True, instance_role="DECODE", num_kv_blocks=3), model_args=args, model=model)
    p_master, d_master = LLMMaster(p_eng.opt, p_eng), LLMMaster(d_eng.opt, d_eng)
    tp, td = InProcTransport.pair()
    DecodeCoordinator(d_master).attach(td)
    PrefillCoordinator(p_master, tp)
    llm = LLM(model="preset:tiny-qwen2", devices="cpu", engine=p_eng)
    llm.master = p_master
    outs = llm.generate([list(range(100))], SamplingParams(max_tokens=4))
    assert outs[0].status.code.name == "RESOURCE_EXHAUSTED"


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("mode", ["PUSH", "PULL"])
def test_pd_two_processes_nvlink_push(tmp_path, mode):
    """PREFILL on GPU 0 and DECODE on GPU 1 as separate processes: TCP control plane, CUDA-IPC mapped decode cache,
    KV blocks written by the push kernel over NVLink (PUSH), or the prefill cache mapped by the decode instance, which
    reads the blocks with peer loads when the first token arrives (PULL)."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    worker = os.path.join(here, "helpers", "pd_worker.py")
    port = 27811
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    co = str(tmp_path / "co.pt")
    logs = {k: open(str(tmp_path / f"{k}.log"), "w") for k in ("co", "d", "p")}

    def tail(k):
        logs[k].flush()
        return open(str(tmp_path / f"{k}.log")).read()[-3000:]
    r = subprocess.run([sys.executable, worker, "colocated", "0", str(port), co], env=env, timeout=180, stdout=logs["co"], stderr=subprocess.STDOUT)
    assert r.returncode == 0, tail("co")
    d_out, p_out = str(tmp_path / "d.pt"), str(tmp_path / "p.pt")
    d = subprocess.Popen([sys.executable, worker, "decode", "1", str(port), d_out, mode], env=env, stdout=logs["d"], stderr=subprocess.STDOUT)
    try:
        try:
            p = subprocess.run([sys.executable, worker, "prefill", "0", str(port), p_out, mode], env=env, timeout=180, stdout=logs["p"],
                               stderr=subprocess.STDOUT)
        except subprocess.TimeoutExpired:
            raise AssertionError("prefill instance timed out\n--- prefill\n" + tail("p") + "\n--- decode\n" + tail("d"))
        assert p.returncode == 0, "--- prefill\n" + tail("p") + "\n--- decode\n" + tail("d")
    finally:
        open(d_out + ".stop", "w").close()
        try:
            d.wait(timeout=60)
        except subprocess.TimeoutExpired:
            d.kill()
    want, got, dec = torch.load(co), torch.load(p_out), torch.load(d_out)
    assert got["status"] == 0 and dec["status"] == 0
    assert (got["moved"] > 0 and dec["pulled"] == 0) if mode == "PUSH" else (got["moved"] == 0 and dec["pulled"] > 0)
    assert got["tokens"] == want["tokens"]
    assert dec["generated"] > 0


def _pair(num_kv_blocks=128):
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    p_eng = LLMEngine(_opts(enable_disagg_pd=True, instance_role="PREFILL"), model_args=args, model=model)
    d_eng = LLMEngine(_opts(enable_disagg_pd=True, instance_role="DECODE", num_kv_blocks=num_kv_blocks), model_args=args, model=model)
    p_master, d_master = LLMMaster(p_eng.opt, p_eng), LLMMaster(d_eng.opt, d_eng)
    tp, td = InProcTransport.pair()
    dec = DecodeCoordinator(d_master)
    dec.attach(td)
    pre = PrefillCoordinator(p_master, tp)
    p_eng.kv_transfer = LocalCopyTransfer(p_eng.worker.kv_caches, d_eng.worker.kv_caches)
    return args, p_master, d_master, pre, dec, tp, td


def _until(cond, what, timeout=10.0):
    import time
    deadline = time.time() + timeout
    while not cond():
        assert time.time() < deadline, what
        time.sleep(0.005)


def test_decode_side_cleans_up_after_a_vanished_prefill_instance():
    """The prefill instance disappears (its connection closes) with one request reserved and one already decoding on
    the decode side: both are released there, and the decode instance stays healthy and usable."""
    from xllm_wxh_b200.framework.params import RequestParams
    from xllm_wxh_b200.utils.health import HEALTH
    args, p_master, d_master, pre, dec, tp, td = _pair()
    d_eng = d_master.engine
    results = []
    # request A runs until the hand-over and a few decode steps on the decode side
    p_master.handle_request(list(range(30)), RequestParams(max_tokens=50, ignore_eos=True, request_id="A"), results.append)
    _until(lambda: len(pre.remote) == 1, "request A was not taken in")       # intake runs on the master's thread pool
    for _ in range(3):
        p_master.step()
    for _ in range(3):
        d_master.step()
    assert d_eng.scheduler.num_running == 1
    # request B has only reserved its blocks there (its prefill has not run yet)
    p_master.handle_request(list(range(100, 140)), RequestParams(max_tokens=50, ignore_eos=True, request_id="B"), results.append)
    _until(lambda: len(dec._owner) == 2, "request B did not reserve its blocks")
    assert d_eng.scheduler.block_manager(0).num_used_blocks > 0
    was_healthy = HEALTH.healthy if hasattr(HEALTH, "healthy") else True
    td.closed = True
    assert dec.unlink(td) == 2                      # what the transport's close callback does
    d_master.step()
    d_master.step()
    assert dec._owner == {} and dec.transports == []
    assert d_eng.scheduler.num_running == 0 and not d_eng.scheduler.has_unfinished()
    assert d_eng.scheduler.block_manager(0).num_used_blocks == 0
    # the decode instance still serves requests of its own
    out = LLM(model="preset:tiny-qwen2", devices="cpu", engine=d_eng)
    out.master = d_master
    d_master._emit = dec._orig_emit
    got = out.generate([list(range(9))], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
    assert got[0].status.ok and len(got[0].outputs[0].token_ids) == 3


def test_prefill_side_fails_its_requests_when_the_decode_instance_vanishes():
    from xllm_wxh_b200.framework.params import RequestParams
    from xllm_wxh_b200.utils.health import HEALTH
    args, p_master, d_master, pre, dec, tp, td = _pair()
    results = []
    p_master.handle_request(list(range(30)), RequestParams(max_tokens=50, ignore_eos=True, request_id="A"), results.append)
    _until(lambda: len(pre.remote) == 1, "request A was not taken in")
    for _ in range(3):
        p_master.step()
    assert len(pre.remote) == 1
    tp.close()                                      # both ends see the link go down
    assert pre.remote == {} and dec._owner == {}
    final = [r for r in results if r.finished]
    assert final and final[-1].status.code.name == "UNAVAILABLE"
    ok, why = HEALTH.status() if hasattr(HEALTH, "status") else (False, "")
    assert not ok
    # a new request is refused at once instead of waiting for a peer that is gone
    p_master.handle_request(list(range(5)), RequestParams(max_tokens=5, request_id="C"), results.append)
    _until(lambda: any(r.request_id == "C" and r.finished for r in results), "request C was not answered")
    c = [r for r in results if r.request_id == "C" and r.finished]
    assert c and c[0].status.code.name == "UNAVAILABLE"
    HEALTH.set_healthy() if hasattr(HEALTH, "set_healthy") else None


def test_routing_names_the_decode_instance():
    """`routing.decode_name` from the service layer: accepted when it is the linked decode instance, refused otherwise."""
    from xllm_wxh_b200.api.openai_service import params_from_body
    from xllm_wxh_b200.framework.params import RequestParams
    p = params_from_body({"prompt": [1, 2], "routing": {"prefill_name": "p0", "decode_name": "d7", "decode_address": "h:1"}}, chat=False)
    assert p.decode_name == "d7" and p.decode_address == "h:1"
    args, p_master, d_master, pre, dec, tp, td = _pair()
    pre.peer_info["instance_name"] = "d0"
    results = []
    p_master.handle_request(list(range(9)), RequestParams(max_tokens=2, request_id="X", decode_name="d7"), results.append)
    _until(lambda: any(r.request_id == "X" and r.finished for r in results), "request X was not answered")
    assert results[-1].status.code.name == "UNAVAILABLE" and "d7" in results[-1].status.message
    p_master.handle_request(list(range(9)), RequestParams(max_tokens=2, request_id="Y", decode_name="d0", ignore_eos=True), results.append)
    _until(lambda: len(pre.remote) == 1, "request Y was not taken in")


def test_one_prefill_instance_feeds_two_decode_instances():
    """Two decode instances behind one prefill instance: requests go to the instance `routing.decode_name` names (or to the
    links in turn), each decode instance receives the KV of its own requests only, tokens equal a colocated engine, and
    the loss of one decode instance fails only its requests."""
    from xllm_wxh_b200.framework.params import RequestParams
    from xllm_wxh_b200.utils.health import HEALTH
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (20, 33, 18, 41)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in
            LLM(model="preset:tiny-qwen2", devices="cpu", engine=LLMEngine(_opts(), model_args=args, model=model)).generate(prompts, sp)]

    p_eng = LLMEngine(_opts(enable_disagg_pd=True, instance_role="PREFILL"), model_args=args, model=model)
    p_master = LLMMaster(p_eng.opt, p_eng)
    d_masters, decs = [], []
    pre = None
    for i in range(2):
        d_eng = LLMEngine(_opts(enable_disagg_pd=True, instance_role="DECODE", instance_name=f"d{i}"), model_args=args, model=model)
        dm = LLMMaster(d_eng.opt, d_eng)
        tp, td = InProcTransport.pair()
        dec = DecodeCoordinator(dm)
        dec.attach(td)
        if pre is None:
            pre = PrefillCoordinator(p_master, tp)
            p_eng.kv_transfer = LocalCopyTransfer(p_eng.worker.kv_caches, d_eng.worker.kv_caches)
        else:
            assert pre.add_decode_link(tp) == 1
            p_eng.kv_transfer_peers[1] = LocalCopyTransfer(p_eng.worker.kv_caches, d_eng.worker.kv_caches)
        d_masters.append(dm)
        decs.append(dec)
    assert [l["info"]["instance_name"] for l in pre.links] == ["d0", "d1"]
    results = {}

    def cb(out):
        results.setdefault(out.request_id, []).append(out)
        return True
    names = ["d1", "d0", "d1", ""]                       # the last one names no decode instance: links take turns
    for i, (pr, name) in enumerate(zip(prompts, names)):
        p_master.handle_request(pr, RequestParams(temperature=0.0, max_tokens=6, ignore_eos=True, request_id=f"r{i}",
                                                  decode_name=name), cb)
    _until(lambda: len(pre.remote) == 4, "requests were not taken in")
    by_link = {i: [info["link"] for cid, info in pre.remote.items() if p_master._states[cid].ext_id == f"r{i}"][0] for i in range(4)}
    assert by_link[0] == 1 and by_link[1] == 0 and by_link[2] == 1 and by_link[3] in (0, 1)
    for _ in range(40):
        p_master.step()
        for dm in d_masters:
            dm.step()
        if all(any(o.finished for o in results.get(f"r{i}", [])) for i in range(4)):
            break
    got = []
    for i in range(4):
        toks = []
        for o in results[f"r{i}"]:
            for so in (o.outputs or []):
                toks = so.token_ids if o.finished and so.token_ids and len(so.token_ids) >= len(toks) else toks
        got.append(toks)
    assert got == want
    # each decode instance served its own requests only
    n0 = d_masters[0].engine.scheduler.stats()["generated_tokens"]
    n1 = d_masters[1].engine.scheduler.stats()["generated_tokens"]
    assert n0 + n1 == 4 * 5 and n0 in (5, 10) and n1 == 20 - n0      # five decoded tokens per request, where it was routed
    assert p_eng.kv_transfer.bytes_moved > 0 and p_eng.kv_transfer_peers[1].bytes_moved > 0
    # one decode instance goes away: only its requests fail, the instance stays in service through the other link
    HEALTH.set_healthy()
    p_master.handle_request(prompts[0], RequestParams(max_tokens=50, ignore_eos=True, request_id="x1", decode_name="d1"), cb)
    p_master.handle_request(prompts[1], RequestParams(max_tokens=50, ignore_eos=True, request_id="x0", decode_name="d0"), cb)
    _until(lambda: len(pre.remote) == 2, "second wave was not taken in")
    pre.links[1]["t"].close()
    assert any(o.finished and o.status.code.name == "UNAVAILABLE" for o in results["x1"])
    assert len(pre.remote) == 1 and HEALTH.status()[0]
    p_master.handle_request(prompts[2], RequestParams(max_tokens=2, request_id="x2", decode_name="d1"), cb)
    _until(lambda: any(o.finished for o in results.get("x2", [])), "x2 was not answered")
    assert results["x2"][-1].status.code.name == "UNAVAILABLE"


def test_link_plan_between_different_tp_degrees():
    """Which destination ranks a source rank writes when every rank holds the same cache (MLA): all destinations are served
    exactly once, by a rank that exists, and the PULL-mode inverse names the same pairing."""
    from xllm_wxh_b200.parallel.kv_transfer import plan_links, plan_source
    assert [plan_links(2, 4, r) for r in range(2)] == [[0, 2], [1, 3]]          # the stride rule of merge_kv_blocks
    assert [plan_links(4, 2, r) for r in range(4)] == [[0], [1], [], []]
    assert [plan_links(1, 8, 0)] == [list(range(8))]
    for src in (1, 2, 3, 4, 8):
        for dst in (1, 2, 4, 6, 8):
            served = sorted(d for r in range(src) for d in plan_links(src, dst, r))
            assert served == list(range(dst)), (src, dst, served)
            for r in range(src):
                assert all(plan_source(src, dst, d) == r for d in plan_links(src, dst, r))
    with pytest.raises(ValueError):
        plan_links(2, 4, 2)


def test_one_source_rank_serves_two_destination_ranks():
    """MultiTransfer: the blocks of one prefill rank land in the caches of both ranks of a TP-2 decode instance, whole
    step or layer by layer."""
    from xllm_wxh_b200.parallel.kv_transfer import MultiTransfer, plan_links
    g = torch.Generator().manual_seed(0)
    src = [(torch.randn(8, 4, 6, generator=g),) for _ in range(3)]                       # 3 layers, one latent tensor each
    dsts = [[(torch.zeros(10, 4, 6),) for _ in range(3)] for _ in range(2)]
    t = MultiTransfer([LocalCopyTransfer(src, dsts[d]) for d in plan_links(1, 2, 0)])
    pairs = [(1, 7), (5, 2)]
    t.push(pairs)
    for layer in range(3):
        t.push_layer_async([(2, 9)], layer)
    t.join()
    t.wait()
    for d in dsts:
        for ls, ld in zip(src, d):
            assert torch.equal(ld[0][7], ls[0][1]) and torch.equal(ld[0][2], ls[0][5]) and torch.equal(ld[0][9], ls[0][2])
            assert float(ld[0][0].abs().sum()) == 0.0
    assert t.bytes_moved == 2 * (2 + 1) * 3 * 4 * 6 * 4
    none = MultiTransfer([])
    none.push(pairs)
    none.wait()
    assert none.bytes_moved == 0


def test_link_to_an_instance_of_another_tp_degree_is_refused_for_head_sharded_caches():
    """A Qwen cache is sharded by KV head, so an instance with another number of ranks cannot be linked; the refusal says so
    (an MLA model, whose ranks all hold the same latent cache, takes the plan of `plan_links` instead)."""
    args = preset("tiny-qwen2")
    eng = LLMEngine(_opts(enable_disagg_pd=True, instance_role="PREFILL"), model_args=args,
                    model=QwenForCausalLM(args, device="cpu").init_random(seed=0))
    with pytest.raises(ValueError, match="same on every rank"):
        eng.link_kv_peer([[], []])
    from xllm_wxh_b200.models.deepseek_impl import DeepseekForCausalLM
    assert DeepseekForCausalLM.kv_replicated_over_tp and not getattr(QwenForCausalLM, "kv_replicated_over_tp", False)
