"""Tiny Qwen2 configuration end to end on CPU in fp32: 4 prompts x 32 tokens, greedy, 32 new tokens,
block size 16, checked token for token against the independent oracle."""
import pytest
import torch

from oracle import greedy_generate
from xllm_wxh_b200 import LLM, SamplingParams
from xllm_wxh_b200.config import Options
from xllm_wxh_b200.models.args import preset
from xllm_wxh_b200.models.qwen import QwenForCausalLM
from xllm_wxh_b200.runtime.engine import LLMEngine


def _prompts(seed=0, n=4, length=32, vocab=1024):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


@pytest.fixture(scope="module")
def tiny():
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    return args, model, model.state_dict()


def _llm(args, model, **kw):
    opts = dict(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=256, dtype="float32")
    opts.update(kw)
    o = Options(**opts)
    return LLM(model="preset:tiny-qwen2", devices="cpu", engine=LLMEngine(o, model_args=args, model=model))


@pytest.mark.parametrize("mode", ["chunked", "prefill_first", "small_chunks", "overlap", "mix", "mix_overlap"])
def test_greedy_matches_oracle(tiny, mode):
    args, model, sd = tiny
    kw = {}
    if mode == "prefill_first":
        kw["enable_chunked_prefill"] = False
    if mode == "small_chunks":
        kw.update(max_tokens_per_chunk_for_prefill=7, max_tokens_per_batch=24)
    if mode in ("overlap", "mix_overlap"):
        kw["enable_schedule_overlap"] = True
    if mode.startswith("mix"):        # urgency-ordered single queue with small chunks and a per-token target
        kw.update(use_mix_scheduler=True, max_tokens_per_batch=40, max_global_tpot_ms=50.0)
    llm = _llm(args, model, **kw)
    prompts = _prompts()
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=32, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.status.ok
        assert o.outputs[0].token_ids == greedy_generate(sd, args, p, 32)
        assert o.outputs[0].finish_reason == "length"
        assert o.usage.num_prompt_tokens == 32 and o.usage.num_generated_tokens == 32


def test_prefix_cache_reuse_keeps_outputs(tiny):
    args, model, sd = tiny
    llm = _llm(args, model)
    prompts = _prompts(seed=3, n=2, length=48)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    first = llm.generate(prompts, sp)
    again = llm.generate(prompts, sp)          # same prompts: served from the prefix cache
    for a, b, p in zip(first, again, prompts):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids == greedy_generate(sd, args, p, 8)
    assert again[0].usage.num_cached_tokens >= 32
    bm = llm.engine.scheduler.block_manager(0)
    assert bm.match_hits > 0


def test_sample_at_selector_positions_matches_oracle(tiny):
    """`LLM.sample`: one output per selector hit, each the greedy next token after the prefix that ends with the hit."""
    args, model, sd = tiny
    llm = _llm(args, model)
    prompts = ["5 9 77 3 4 77 8", "1 77", "2 3 4"]
    outs = llm.sample(prompts, selector="77", logprobs=3)
    assert [len(o.outputs) for o in outs] == [2, 1, 0]
    ids = [int(t) for t in prompts[0].split()]
    for h, end in enumerate((3, 6)):
        want = greedy_generate(sd, args, ids[:end], 1)
        so = outs[0].outputs[h]
        assert so.index == h and so.token_ids == want and so.finish_reason == "length"
        assert len(so.logprobs) == 1 and len(so.logprobs[0].top_logprobs) == 3
        assert so.logprobs[0].top_logprobs[0].token_id == want[0]          # greedy token leads the alternatives
    with pytest.raises(ValueError):
        llm.sample(["1 2"], selector="7 8")                                 # selector must be a single token


def test_example_scripts_run_on_cpu():
    """The scripts under examples/ run as a user would run them (random-weight preset on CPU)."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    for name, marker in (("generate.py", "Generated text"), ("sample.py", "sample_id=0"),
                         ("generate_embedding.py", "dim 256"), ("generate_beam_search.py", "best beam")):
        p = subprocess.run([sys.executable, os.path.join(root, "examples", name), "--model=preset:tiny-qwen2", "--devices=cpu"],
                           env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
        assert p.returncode == 0 and marker in p.stdout, (name, p.stdout[-2000:])


def test_host_trace_and_chrome_export(tiny, tmp_path):
    import json
    args, model, _ = tiny
    llm = _llm(args, model)
    llm.generate(_prompts(n=2, length=8), SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    eng = llm.engine
    summ = eng.host_trace_summary()
    assert set(summ) == {"schedule_ms", "pack_publish_ms", "kernel_issue_ms", "collect_wait_ms"} and summ["kernel_issue_ms"] > 0
    n = eng.export_chrome_trace(str(tmp_path / "trace.json"))
    ev = json.load(open(tmp_path / "trace.json"))["traceEvents"]
    assert n >= 4 and len(ev) == 4 * n and ev[0]["ph"] == "X"


def test_top_logprobs_with_schedule_overlap_match_the_plain_run(tiny):
    """The alternatives of every generated token must come back with schedule overlap on too, equal to the run without
    it, and nothing of them may stay behind in the engine: neither for co-batched requests that asked for none nor after
    the requests have finished."""
    args, model, sd = tiny
    prompts = _prompts(seed=5, n=3, length=20)
    with_lp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, logprobs=True, top_logprobs=3)
    without = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    results = {}
    for overlap in (False, True):
        llm = _llm(args, model, enable_schedule_overlap=overlap)
        outs = llm.generate(prompts, [with_lp, without, with_lp])
        results[overlap] = outs
        assert llm.engine.top_logprobs == {}, "alternatives left behind in the engine"
        assert outs[1].outputs[0].logprobs in (None, [])
    for a, b in zip(results[False], results[True]):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids
    for i in (0, 2):
        plain, over = results[False][i].outputs[0].logprobs, results[True][i].outputs[0].logprobs
        assert len(plain) == len(over) == 6
        for x, y in zip(plain, over):
            assert len(y.top_logprobs) == 3
            assert [t.token_id for t in x.top_logprobs] == [t.token_id for t in y.top_logprobs]
            assert y.top_logprobs[0].token_id == y.token_id
            for t, u in zip(x.top_logprobs, y.top_logprobs):
                assert abs(t.logprob - u.logprob) < 1e-5


def test_penalties_follow_the_tokens_as_they_arrive(tiny):
    """The per-sequence token counts behind the penalties grow step by step (chunked prefill adds the prompt in pieces,
    every decode step one token): greedy decoding under repetition, frequency and presence penalties equals a
    step-by-step recomputation from the oracle's logits.  (With schedule overlap the newest token is still a placeholder
    on the host when the next step's list is built, so its penalty starts one step later; that run is only required to
    finish with the same number of tokens.)"""
    from oracle import forward_full
    args, model, sd = tiny
    prompts = _prompts(seed=7, n=3, length=40, vocab=64)          # few distinct ids: repeats are certain
    rep, freq, pres = 1.3, 0.4, 0.6
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True, repetition_penalty=rep, frequency_penalty=freq,
                        presence_penalty=pres)
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(24):
            lg = forward_full(sd, args, toks)[-1].float().clone()
            gen = toks[len(p):]
            for t in set(gen):                                   # frequency and presence first (generated tokens only) ...
                lg[t] -= freq * gen.count(t) + pres
            seen = torch.tensor(sorted(set(toks)))               # ... then the repetition penalty on every token seen
            v = lg[seen]
            lg[seen] = torch.where(v < 0, v * rep, v / rep)
            toks.append(int(lg.argmax()))
        want.append(toks[len(p):])
    for kw in (dict(), dict(max_tokens_per_chunk_for_prefill=16, max_tokens_per_batch=64)):
        got = [o.outputs[0].token_ids for o in _llm(args, model, **kw).generate(prompts, sp)]
        assert got == want, kw
    late = [o.outputs[0].token_ids for o in _llm(args, model, enable_schedule_overlap=True).generate(prompts, sp)]
    assert [len(t) for t in late] == [24, 24, 24] and [t[0] for t in late] == [t[0] for t in want]


def test_outputs_of_a_request_that_was_scheduled_before_its_state_was_registered_are_not_lost(tiny):
    """A request becomes schedulable inside `engine.add_request`; the serving loop may run whole steps before the
    submitting thread gets to register the request's state.  Its outputs must wait for that, not be dropped (a dropped
    final output left the request unfinished for ever)."""
    import threading
    import time
    from xllm_wxh_b200.framework.params import RequestParams
    from xllm_wxh_b200.runtime.master import LLMMaster
    args, model, sd = tiny
    eng = LLMEngine(Options(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=64, dtype="float32"),
                    model_args=args, model=model)
    master = LLMMaster(eng.opt, eng)
    real = eng.add_request

    def slow_add(*a, **kw):
        cid = real(*a, **kw)
        master._wake.set()
        time.sleep(0.5)                       # the loop thread runs the request to its end meanwhile
        return cid
    eng.add_request = slow_add
    master.run()
    got, done = [], threading.Event()

    def cb(out):
        got.append(out)
        if out.finished:
            done.set()
        return True
    try:
        prompt = _prompts(seed=9, n=1, length=12)[0]
        master.handle_request(prompt, RequestParams(max_tokens=3, temperature=0.0, ignore_eos=True), cb, asynchronous=False)
        assert done.wait(10), "the request never finished"
        assert got[-1].outputs[0].token_ids == greedy_generate(sd, args, prompt, 3)
    finally:
        master.stop()
