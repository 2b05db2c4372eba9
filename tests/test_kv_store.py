"""Shared KV-block store (third tier): the store itself, the scheduler's adoption of fetched blocks, and two engines that
share prefixes through it.  The reference's counterpart is KVCacheStore over Mooncake (kv_cache_store.cpp) with
prefetch_from_storage (hierarchy_block_manager_pool.cpp:209-262)."""
import threading

import torch

from test_core_scheduler import make, stop
from xllm_wxh_b200 import LLM, SamplingParams
from xllm_wxh_b200.config import Options
from xllm_wxh_b200.models.args import preset
from xllm_wxh_b200.models.qwen import QwenForCausalLM
from xllm_wxh_b200.runtime.engine import LLMEngine
from xllm_wxh_b200.service.kv_store import KvStore, KvStoreClient, KvStoreServer, block_key, model_namespace


def test_store_keeps_the_most_recently_used_blocks_within_its_capacity():
    st = KvStore(capacity_bytes=1000)
    assert st.put("a", b"x" * 400) and st.put("b", b"y" * 400)
    assert st.get("a") == b"x" * 400                      # "a" is now newer than "b"
    assert st.put("c", b"z" * 400)                        # evicts "b"
    assert st.exist("a") and not st.exist("b") and st.exist("c") and st.used == 800
    assert st.put("a", b"w" * 100) and st.used == 500     # overwrite replaces the bytes
    assert not st.put("huge", b"0" * 2000)
    s = st.stats()
    assert s["evictions"] == 1 and s["blocks"] == 2 and s["hits"] == 1


def test_client_and_server_move_raw_records_and_survive_a_lost_store():
    srv = KvStoreServer("127.0.0.1", 0, 1 << 20).start()
    try:
        c = KvStoreClient(f"127.0.0.1:{srv.port}")
        rec = torch.arange(4096, dtype=torch.uint8)
        assert c.batch_put(["k1", "k2"], [memoryview(rec.numpy()), b"abc"]) == 2
        assert c.batch_exist(["k1", "nope", "k2"]) == [True, False, True]
        got = c.batch_get(["nope", "k1", "k2"])
        assert got[0] is None and bytes(got[1]) == rec.numpy().tobytes() and bytes(got[2]) == b"abc"
        # several threads share one client
        errs = []

        def worker(i):
            for j in range(20):
                key = f"t{i}-{j}"
                if c.batch_put([key], [bytes([i]) * 64]) != 1 or bytes(c.batch_get([key])[0]) != bytes([i]) * 64:
                    errs.append(key)
        ths = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
        [t.start() for t in ths]
        [t.join() for t in ths]
        assert not errs and c.stats()["puts"] == 2 + 80
    finally:
        srv.stop()
    dead = KvStoreClient("127.0.0.1:1", timeout_s=0.2)
    assert dead.batch_exist(["a"]) == [False] and dead.batch_get(["a"]) == [None] and dead.batch_put(["a"], [b"x"]) == 0
    assert dead.failures == 3
    assert block_key((5, 9), 1, 2, "ns:") == "ns:00000000000000090000000000000005/1/2"
    a = preset("tiny-qwen2")
    assert model_namespace("m", a, 16, 100) != model_namespace("m", a, 32, 100) != model_namespace("n", a, 16, 100)


def test_scheduler_adopts_fetched_blocks_into_the_host_tier():
    s = make(num_blocks=9, block_size=4, prefix=True, host_blocks_factor=2.0, max_tokens_per_batch=64)
    prompt = list(range(200, 221))                           # 21 tokens: 5 full blocks can be reused
    assert s.prefix_presence(0, prompt) == (0, 0)
    got = s.host_adopt(0, prompt, 0, 3)
    assert [i for i, _ in got] == [0, 1, 2] and len({h for _, h in got}) == 3
    assert s.prefix_presence(0, prompt) == (0, 3) and s.stats()["host_adopted_blocks"] == 3
    hm = s.host_manager(0)
    keys = [hm.block_hash(h) for _, h in got]
    from xllm_wxh_b200 import _core
    assert keys == _core.prefix_block_keys(prompt[:12], 4, 1024) and hm.block_hash(got[0][1]) != (0, 0)
    # the store held blocks from 4 on, but the host prefix ends at 3: nothing is adopted (there would be a hole)
    assert s.host_adopt(0, prompt, 4, 5) == [] and s.prefix_presence(0, prompt) == (0, 3)
    # extend from where the host tier stands
    more = s.host_adopt(0, prompt, 3, 5)
    assert [i for i, _ in more] == [3, 4] and s.prefix_presence(0, prompt) == (0, 5)
    assert s.host_adopt(0, prompt, 0, 5) == []               # nothing missing any more
    # a request for this prompt loads the adopted blocks like any host-tier hit
    s.add_request(prompt, stop=stop(2))
    b = s.schedule()[0]
    offs, loads = s.take_transfers()[0]
    assert [h for h, _ in loads] == [h for _, h in got + more] and offs == []
    assert b.num_seqs == 1 and s.stats()["host_loaded_blocks"] == 5
    # more blocks than the host tier can take: refused as a whole
    big = list(range(1000, 1000 + 4 * 40))
    assert s.host_adopt(0, big, 0, 39) == []


def _engine(args, model, port, **kw):
    o = dict(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=24, dtype="float32", host_blocks_factor=2.0,
             enable_kvcache_store=True, store_master_server_address=f"127.0.0.1:{port}", max_tokens_per_batch=256)
    o.update(kw)
    return LLMEngine(Options(**o), model_args=args, model=model)


def test_second_instance_completes_its_prompt_from_the_store():
    """Instance A serves a prompt; its blocks reach the host tier and from there the store.  Instance B (same model, empty
    caches) gets the same prompt: the blocks come out of the store into B's host tier, B loads them instead of computing
    them, and its tokens equal A's.  Another model's instance shares the store without meeting A's blocks."""
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    srv = KvStoreServer("127.0.0.1", 0, 64 << 20).start()
    try:
        g = torch.Generator().manual_seed(3)
        prompt = torch.randint(0, args.vocab_size, (100,), generator=g).tolist()      # 6 full blocks
        sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
        a = _engine(args, model, srv.port)
        assert a.kv_store is not None and a.host_tier.store is a.kv_store
        want = LLM(model="x", devices="cpu", engine=a).generate([prompt], sp)[0].outputs[0].token_ids
        a.host_tier.flush_store()
        st = srv.store.stats()
        assert st["blocks"] == 6 and a.host_tier.blocks_put == 6 and st["bytes"] == 6 * a.host_tier.stride
        assert a.store_prefetched_blocks == 0
        # the same prompt again on A: everything is local, nothing is fetched or sent
        LLM(model="x", devices="cpu", engine=a).generate([prompt], sp)
        a.host_tier.flush_store()
        assert a.store_prefetched_blocks == 0 and srv.store.stats()["puts"] == 6

        b = _engine(args, model, srv.port)
        out = LLM(model="x", devices="cpu", engine=b).generate([prompt], sp)[0]
        assert out.outputs[0].token_ids == want
        assert b.store_prefetched_blocks == 6 and b.host_tier.blocks_filled == 6
        sb = b.scheduler.stats()
        assert sb["host_adopted_blocks"] == 6 and sb["host_loaded_blocks"] == 6
        assert out.usage.num_cached_tokens == 96                                        # 6 blocks were not computed
        # a longer prompt with the same beginning, served by A first: B has the shared part in its own tiers and fetches
        # only the two blocks that A added
        longer = prompt + torch.randint(0, args.vocab_size, (40,), generator=g).tolist()
        ref = LLM(model="x", devices="cpu", engine=a).generate([longer], sp)[0].outputs[0].token_ids
        a.host_tier.flush_store()
        assert srv.store.stats()["blocks"] == 9                 # 140 prompt + 4 generated tokens with KV = 9 full blocks
        assert LLM(model="x", devices="cpu", engine=b).generate([longer], sp)[0].outputs[0].token_ids == ref
        assert b.store_prefetched_blocks == 8 and b.host_tier.blocks_filled == 8

        # another model (other weights under another name) uses the same store and never sees A's blocks
        other = QwenForCausalLM(args, device="cpu").init_random(seed=7)
        c = _engine(args, other, srv.port, model_id="other-model")
        own = LLM(model="x", devices="cpu", engine=LLMEngine(Options(model="preset:tiny-qwen2", devices="cpu", block_size=16,
                  num_kv_blocks=24, dtype="float32"), model_args=args, model=other)).generate([prompt], sp)[0].outputs[0].token_ids
        assert LLM(model="x", devices="cpu", engine=c).generate([prompt], sp)[0].outputs[0].token_ids == own
        assert c.store_prefetched_blocks == 0

        # the store goes away: instances keep serving from their own tiers and by computing
        srv.stop()
        fresh = torch.randint(0, args.vocab_size, (70,), generator=g).tolist()
        ref = LLM(model="x", devices="cpu", engine=a).generate([fresh], sp)[0].outputs[0].token_ids
        assert LLM(model="x", devices="cpu", engine=b).generate([fresh], sp)[0].outputs[0].token_ids == ref
    finally:
        try:
            srv.stop()
        except Exception:
            pass


def test_store_prefetch_under_a_running_serving_loop():
    """Requests arrive on several threads while the scheduling thread runs: the look-up and the adoption take the step lock,
    every request ends with the tokens of a store-less engine, and the shared prefix was fetched, not computed."""
    import time
    from xllm_wxh_b200.framework.params import RequestParams
    from xllm_wxh_b200.runtime.master import LLMMaster
    from xllm_wxh_b200.utils.tokenizer import IdTokenizer
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    srv = KvStoreServer("127.0.0.1", 0, 64 << 20).start()
    try:
        g = torch.Generator().manual_seed(5)
        shared = torch.randint(0, args.vocab_size, (64,), generator=g).tolist()         # 4 blocks every prompt starts with
        prompts = [shared + torch.randint(0, args.vocab_size, (10 + i,), generator=g).tolist() for i in range(8)]
        sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
        plain = LLMEngine(Options(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=64, dtype="float32"),
                          model_args=args, model=model)
        want = [o.outputs[0].token_ids for o in LLM(model="x", devices="cpu", engine=plain).generate(prompts, sp)]
        a = _engine(args, model, srv.port, num_kv_blocks=64)
        LLM(model="x", devices="cpu", engine=a).generate([prompts[0]], sp)
        a.host_tier.flush_store()
        assert srv.store.stats()["blocks"] >= 4
        b = _engine(args, model, srv.port, num_kv_blocks=64)
        master = LLMMaster(b.opt, b, IdTokenizer(args.vocab_size))
        assert b.external_step_lock is master._step_lock
        master.run()
        done = {}

        def submit(i):
            def cb(out):
                if out.finished:
                    done[i] = out
                return True
            master.handle_request(prompts[i], RequestParams(temperature=0.0, max_tokens=4, ignore_eos=True, request_id=f"r{i}"), cb)
        ths = [threading.Thread(target=submit, args=(i,)) for i in range(8)]
        [t.start() for t in ths]
        [t.join() for t in ths]
        deadline = time.time() + 60
        while len(done) < 8 and time.time() < deadline:
            time.sleep(0.01)
        master.stop()
        assert len(done) == 8 and [done[i].outputs[0].token_ids for i in range(8)] == want
        assert b.store_prefetched_blocks >= 4 and b.scheduler.stats()["host_loaded_blocks"] >= 4
    finally:
        srv.stop()


import pytest  # noqa: E402


@pytest.mark.gpu
def test_store_tier_on_gpu_two_engines_share_a_prefix():
    """On the device: engine A's blocks go device -> pinned host record -> store; engine B fetches them into its host
    pool and loads them through the pack kernel instead of computing them.  Tokens equal a store-less engine's."""
    from xllm_wxh_b200.models.args import ModelArgs
    from xllm_wxh_b200.ops import cuda_ops
    args = ModelArgs(model_type="qwen3", vocab_size=2048, hidden_size=512, n_layers=3, n_heads=8, n_kv_heads=2, head_dim=128,
                     intermediate_size=1536, qk_norm=True, rope_theta=1e6, max_position_embeddings=4096, dtype="bfloat16")
    srv = KvStoreServer("127.0.0.1", 0, 256 << 20).start()
    try:
        g = torch.Generator().manual_seed(11)
        prompts = [torch.randint(0, args.vocab_size, (130,), generator=g).tolist() for _ in range(3)]       # 8 full blocks each
        sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)

        def engine(store):
            kw = dict(enable_kvcache_store=True, store_master_server_address=f"127.0.0.1:{srv.port}") if store else {}
            return LLMEngine(Options(model="preset:x", devices="cuda:0", block_size=16, num_kv_blocks=40, host_blocks_factor=2.0,
                                     max_tokens_per_batch=512, max_seqs_per_batch=4, random_seed=0, **kw), model_args=args)
        want = [o.outputs[0].token_ids for o in LLM(model="preset:x", devices="cuda:0", engine=engine(False)).generate(prompts, sp)]
        a = engine(True)
        assert [o.outputs[0].token_ids for o in LLM(model="preset:x", devices="cuda:0", engine=a).generate(prompts, sp)] == want
        a.host_tier.drain()
        a.host_tier.flush_store()
        assert srv.store.stats()["blocks"] == 24 and a.host_tier.blocks_put == 24
        b = engine(True)
        outs = LLM(model="preset:x", devices="cuda:0", engine=b).generate(prompts, sp)
        assert [o.outputs[0].token_ids for o in outs] == want
        assert b.store_prefetched_blocks == 24 and b.scheduler.stats()["host_loaded_blocks"] == 24
        assert all(o.usage.num_cached_tokens == 128 for o in outs)
        assert cuda_ops.read_status() == 0
    finally:
        srv.stop()


def test_store_under_cache_pressure_keeps_tokens_exact():
    """Small device caches and small host tiers on two engines that take turns on prompts with shared beginnings, a store
    that itself evicts: blocks move device -> host -> store -> other host -> other device all the time, host blocks are
    reused while their records are being sent, and every answer must still be the one a plain engine gives."""
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    g = torch.Generator().manual_seed(9)
    stems = [torch.randint(0, args.vocab_size, (48 + 16 * i,), generator=g).tolist() for i in range(4)]
    prompts = []
    for r in range(24):
        stem = stems[int(torch.randint(0, 4, (1,), generator=g))]
        tail = torch.randint(0, args.vocab_size, (int(torch.randint(1, 30, (1,), generator=g)),), generator=g).tolist()
        prompts.append(stem + tail)
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    plain = LLMEngine(Options(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=256, dtype="float32"),
                      model_args=args, model=model)
    want = [o.outputs[0].token_ids for o in LLM(model="x", devices="cpu", engine=plain).generate(prompts, sp)]
    rec = 2 * args.n_layers * 16 * args.n_kv_heads * args.head_dim * 4
    srv = KvStoreServer("127.0.0.1", 0, 14 * rec).start()                   # room for 14 blocks only
    try:
        engines = [_engine(args, model, srv.port, num_kv_blocks=14, host_blocks_factor=0.8, max_seqs_per_batch=2) for _ in range(2)]
        llms = [LLM(model="x", devices="cpu", engine=e) for e in engines]
        got = []
        for i in range(0, len(prompts), 2):
            k = (i // 2) % 2
            got += [o.outputs[0].token_ids for o in llms[k].generate(prompts[i:i + 2], sp)]
        assert got == want
        for e in engines:
            e.host_tier.flush_store()
        st = srv.store.stats()
        assert st["evictions"] > 0 and st["puts"] > 14
        assert sum(e.store_prefetched_blocks for e in engines) > 0
        assert sum(e.scheduler.stats()["host_loaded_blocks"] for e in engines) > 0
        for e in engines:
            while e.scheduler.has_pending_transfers:                        # blocks still held for copies of the last steps
                e.scheduler.schedule()
                e._publish_transfers_only(1)
            assert e.scheduler.block_manager(0).num_used_blocks == 0
    finally:
        srv.stop()
