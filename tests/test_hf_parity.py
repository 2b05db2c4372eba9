"""Model families against the Hugging Face implementations on CPU: a random model saved with `save_pretrained` is loaded
by the engine from its directory, and its greedy tokens must be those HF computes (llama, mistral, qwen2, qwen3, qwen3_moe,
deepseek_v3); the rope scaling variants (llama3, linear, yarn) are compared with HF's own frequency tables."""
import json

import pytest
import torch

from xllm_wxh_b200 import LLM, SamplingParams
from xllm_wxh_b200.config import Options
from xllm_wxh_b200.models.args import args_from_hf_config, load_model_args
from xllm_wxh_b200.ops import reference as ref
from xllm_wxh_b200.runtime.engine import LLMEngine

transformers = pytest.importorskip("transformers")


def _hf_greedy(model, prompt, n):
    ids = torch.tensor([prompt])
    out = []
    with torch.no_grad():
        for _ in range(n):
            nxt = int(model(ids).logits[0, -1].argmax())
            out.append(nxt)
            ids = torch.cat([ids, torch.tensor([[nxt]])], dim=1)
    return out


def _engine(path):
    o = Options(model=str(path), devices="cpu", block_size=16, num_kv_blocks=64, dtype="float32")
    return LLMEngine(o)


@pytest.mark.parametrize("kind", ["llama", "llama3_rope", "mistral_window"])
def test_llama_family_matches_hugging_face(tmp_path, kind):
    torch.manual_seed(0)
    common = dict(vocab_size=512, hidden_size=128, intermediate_size=344, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, max_position_embeddings=512, rms_norm_eps=1e-5, tie_word_embeddings=False,
                  torch_dtype="float32")
    if kind == "mistral_window":
        cfg = transformers.MistralConfig(sliding_window=24, rope_theta=10000.0, **common)
        model = transformers.MistralForCausalLM(cfg)
    else:
        extra = {}
        if kind == "llama3_rope":
            extra["rope_scaling"] = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                     "original_max_position_embeddings": 64}
        cfg = transformers.LlamaConfig(rope_theta=10000.0, **common, **extra)
        model = transformers.LlamaForCausalLM(cfg)
    model = model.float().eval()
    with torch.no_grad():
        for p in model.parameters():
            p.mul_(3.0)                       # sharper logits than the default init: greedy ties would make the check moot
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    args = load_model_args(str(tmp_path))
    assert args.model_type == ("mistral" if kind == "mistral_window" else "llama") and not args.qk_norm and not args.attention_bias
    if kind == "llama3_rope":
        assert args.rope_scaling_type == "llama3" and args.rope_scaling_factor == 8.0 and args.rope_original_max_position == 64
    if kind == "mistral_window":
        assert args.sliding_window == 24
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (5, 40, 90)]
    eng = _engine(tmp_path)
    outs = LLM(model=str(tmp_path), devices="cpu", engine=eng).generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == _hf_greedy(model, p, 8)


def test_rope_scaling_tables_match_hugging_face():
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    base = dict(model_type="llama", hidden_size=256, num_attention_heads=4, num_hidden_layers=1, max_position_embeddings=4096,
                rope_theta=500000.0)
    cases = {
        "llama3": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                   "original_max_position_embeddings": 1024},
        "linear": {"rope_type": "linear", "factor": 4.0},
        "yarn": {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 1024},
    }
    for kind, rs in cases.items():
        a = args_from_hf_config(dict(base, rope_scaling=rs))
        assert a.rope_scaling_type == kind
        table = ref.scaled_cos_sin_cache(a, 64)
        cfg = transformers.LlamaConfig(hidden_size=256, num_attention_heads=4, num_hidden_layers=1, max_position_embeddings=4096,
                                       rope_theta=500000.0, rope_scaling=dict(rs))
        inv, att = ROPE_INIT_FUNCTIONS[kind](cfg, "cpu")
        t = torch.arange(4096, dtype=torch.float32)
        fr = torch.outer(t, inv.float())
        want = torch.cat([fr.cos() * att, fr.sin() * att], dim=-1)
        assert torch.allclose(table, want, atol=2e-4), kind
    with pytest.raises(ValueError):
        args_from_hf_config(dict(base, rope_scaling={"rope_type": "longrope", "factor": 2.0}))


@pytest.mark.parametrize("kind", ["qwen2", "qwen3", "qwen3_moe"])
def test_qwen_family_matches_hugging_face(tmp_path, kind):
    """The same check for the Qwen families, whose block adds the qkv bias (qwen2), per-head q / k norms (qwen3) and the
    routed experts (qwen3_moe)."""
    torch.manual_seed(0)
    common = dict(vocab_size=512, hidden_size=128, intermediate_size=344, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, max_position_embeddings=512, rms_norm_eps=1e-6, tie_word_embeddings=False,
                  torch_dtype="float32", rope_theta=1000000.0)
    if kind == "qwen2":
        model = transformers.Qwen2ForCausalLM(transformers.Qwen2Config(**common))
    elif kind == "qwen3":
        model = transformers.Qwen3ForCausalLM(transformers.Qwen3Config(head_dim=32, **common))
    else:
        model = transformers.Qwen3MoeForCausalLM(transformers.Qwen3MoeConfig(
            head_dim=32, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=96, norm_topk_prob=True,
            decoder_sparse_step=1, mlp_only_layers=[], **common))
    model = model.float().eval()
    with torch.no_grad():
        for p in model.parameters():
            p.mul_(2.0)
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    args = load_model_args(str(tmp_path))
    assert args.model_type == kind
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (7, 50)]
    eng = _engine(tmp_path)
    outs = LLM(model=str(tmp_path), devices="cpu", engine=eng).generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == _hf_greedy(model, p, 8)


def test_deepseek_v3_matches_hugging_face(tmp_path):
    """Multi-head latent attention with the decoupled rope part, yarn scaling, sigmoid routing with group-limited top-k and
    the score-correction bias, shared expert, dense first layer."""
    torch.manual_seed(0)
    cfg = transformers.DeepseekV3Config(
        vocab_size=512, hidden_size=128, intermediate_size=256, moe_intermediate_size=64, num_hidden_layers=3,
        num_attention_heads=4, num_key_value_heads=4, n_shared_experts=1, n_routed_experts=8, routed_scaling_factor=2.5,
        kv_lora_rank=32, q_lora_rank=48, qk_rope_head_dim=16, v_head_dim=32, qk_nope_head_dim=32, n_group=4, topk_group=2,
        num_experts_per_tok=2, first_k_dense_replace=1, norm_topk_prob=True, max_position_embeddings=512, rms_norm_eps=1e-6,
        rope_theta=10000.0, tie_word_embeddings=False, torch_dtype="float32",
        rope_scaling={"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 128, "beta_fast": 32, "beta_slow": 1,
                      "mscale": 1.0, "mscale_all_dim": 1.0})
    model = transformers.DeepseekV3ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.mul_(2.0)
            if n.endswith("e_score_correction_bias"):
                p.copy_(torch.randn_like(p) * 0.1)
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    args = load_model_args(str(tmp_path))
    assert args.model_type == "deepseek_v3" and args.kv_lora_rank == 32 and args.rope_scaling_type == "yarn"
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (6, 45, 150)]
    eng = _engine(tmp_path)
    outs = LLM(model=str(tmp_path), devices="cpu", engine=eng).generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == _hf_greedy(model, p, 8)


def test_embedding_matches_hugging_face_hidden_state(tmp_path):
    """The embedding task returns the L2-normalised final hidden state (after the last norm) of the prompt's last token."""
    torch.manual_seed(0)
    cfg = transformers.Qwen3Config(vocab_size=512, hidden_size=128, intermediate_size=344, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=32, max_position_embeddings=512, rms_norm_eps=1e-6,
                                   tie_word_embeddings=False, torch_dtype="float32", rope_theta=1000000.0)
    model = transformers.Qwen3ForCausalLM(cfg).float().eval()
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (3, 37, 80)]
    llm = LLM(model=str(tmp_path), devices="cpu", engine=_engine(tmp_path))
    outs = llm.embed(prompts)
    for p, o in zip(prompts, outs):
        with torch.no_grad():
            h = model.model(torch.tensor([p])).last_hidden_state[0, -1]
        want = torch.nn.functional.normalize(h, dim=-1)
        got = torch.tensor(o.outputs[0].embeddings)
        assert got.shape == want.shape and torch.allclose(got, want, atol=2e-4)


def test_config_keys_with_null_values_and_newer_names():
    base = {"model_type": "deepseek_v2", "hidden_size": 128, "num_attention_heads": 4, "num_hidden_layers": 2}
    assert args_from_hf_config(dict(base, q_lora_rank=None)).q_lora_rank == 0          # DeepSeek-V2-Lite: no low-rank q
    assert args_from_hf_config(dict(base, q_lora_rank=48)).q_lora_rank == 48
    assert args_from_hf_config(base).q_lora_rank == 1536
    moe = {"model_type": "qwen3_moe", "hidden_size": 128, "num_attention_heads": 4, "num_hidden_layers": 2}
    assert args_from_hf_config(dict(moe, num_local_experts=8)).n_routed_experts == 8
    assert args_from_hf_config(dict(moe, num_experts=16)).n_routed_experts == 16
    ds = args_from_hf_config(dict(base, rope_parameters={"rope_type": "yarn", "factor": 4.0, "rope_theta": 5000.0,
                                                          "original_max_position_embeddings": 128}))
    assert ds.rope_scaling_type == "yarn" and ds.rope_theta == 5000.0 and ds.rope_original_max_position == 128


def test_sliding_window_with_chunked_prefill_and_cached_prefixes(tmp_path):
    """Mistral's attention window against HF when the prompt is prefilled in 32-token chunks and when its beginning comes
    out of the prefix cache on the second pass."""
    torch.manual_seed(0)
    cfg = transformers.MistralConfig(vocab_size=512, hidden_size=128, intermediate_size=344, num_hidden_layers=2,
                                     num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512, rms_norm_eps=1e-5,
                                     tie_word_embeddings=False, torch_dtype="float32", sliding_window=24, rope_theta=10000.0)
    model = transformers.MistralForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for p in model.parameters():
            p.mul_(3.0)
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (90, 130)]
    want = [_hf_greedy(model, p, 8) for p in prompts]
    eng = LLMEngine(Options(model=str(tmp_path), devices="cpu", block_size=16, num_kv_blocks=64, dtype="float32", max_tokens_per_batch=32))
    llm = LLM(model=str(tmp_path), devices="cpu", engine=eng)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    first = llm.generate(prompts, sp)
    second = llm.generate(prompts, sp)
    assert [o.outputs[0].token_ids for o in first] == want and [o.outputs[0].token_ids for o in second] == want
    assert [o.usage.num_cached_tokens for o in first] == [0, 0] and [o.usage.num_cached_tokens for o in second] == [80, 128]


def test_logprobs_match_hugging_face(tmp_path):
    """Log-probabilities of the sampled tokens and the top alternatives against HF's log-softmax of the same positions."""
    torch.manual_seed(0)
    cfg = transformers.Qwen3Config(vocab_size=512, hidden_size=128, intermediate_size=344, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=32, max_position_embeddings=512, rms_norm_eps=1e-6,
                                   tie_word_embeddings=False, torch_dtype="float32", rope_theta=1000000.0)
    model = transformers.Qwen3ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for p in model.parameters():
            p.mul_(2.0)
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 512, (40,), generator=g).tolist()
    llm = LLM(model=str(tmp_path), devices="cpu", engine=_engine(tmp_path))
    out = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True, logprobs=True, top_logprobs=3))[0].outputs[0]
    ids = torch.tensor([prompt])
    for i, tok in enumerate(out.token_ids):
        with torch.no_grad():
            lp = torch.log_softmax(model(ids).logits[0, -1].float(), -1)
        top = torch.topk(lp, 3)
        mine = out.logprobs[i]
        assert abs(mine.logprob - float(lp[tok])) < 1e-3
        assert [t.token_id for t in mine.top_logprobs] == [int(t) for t in top.indices]
        assert all(abs(t.logprob - float(v)) < 1e-3 for t, v in zip(mine.top_logprobs, top.values))
        ids = torch.cat([ids, torch.tensor([[tok]])], dim=1)


def test_repetition_penalty_matches_hugging_face(tmp_path):
    """Greedy decoding under a repetition penalty (prompt and generated tokens count) against HF's logits processor; the small
    vocabulary makes repeats certain."""
    torch.manual_seed(0)
    cfg = transformers.Qwen3Config(vocab_size=64, hidden_size=128, intermediate_size=344, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=32, max_position_embeddings=512, rms_norm_eps=1e-6,
                                   tie_word_embeddings=False, torch_dtype="float32", rope_theta=1000000.0)
    model = transformers.Qwen3ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for p in model.parameters():
            p.mul_(2.0)
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 64, (30,), generator=g).tolist()
    llm = LLM(model=str(tmp_path), devices="cpu", engine=_engine(tmp_path))
    plain = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))[0].outputs[0].token_ids
    got = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True, repetition_penalty=1.5))[0].outputs[0].token_ids
    proc = transformers.RepetitionPenaltyLogitsProcessor(1.5)
    ids, want = torch.tensor([prompt]), []
    with torch.no_grad():
        for _ in range(12):
            nxt = int(proc(ids, model(ids).logits[:, -1].float())[0].argmax())
            want.append(nxt)
            ids = torch.cat([ids, torch.tensor([[nxt]])], dim=1)
    assert got == want and got != plain


@pytest.mark.parametrize("rs", [{"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 128},
                                {"rope_type": "linear", "factor": 2.0}], ids=["yarn", "linear"])
def test_qwen3_with_scaled_rope_matches_hugging_face(tmp_path, rs):
    """Long-context configurations of the dense models (positions beyond the original context) against HF."""
    torch.manual_seed(0)
    cfg = transformers.Qwen3Config(vocab_size=512, hidden_size=128, intermediate_size=344, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=32, max_position_embeddings=512, rms_norm_eps=1e-6,
                                   tie_word_embeddings=False, torch_dtype="float32", rope_theta=10000.0, rope_scaling=dict(rs))
    model = transformers.Qwen3ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for p in model.parameters():
            p.mul_(2.0)
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    assert load_model_args(str(tmp_path)).rope_scaling_type == rs["rope_type"]
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (20, 200)]
    outs = LLM(model=str(tmp_path), devices="cpu", engine=_engine(tmp_path)).generate(
        prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == _hf_greedy(model, p, 6)


def test_beam_search_matches_a_beam_over_hugging_face_logits(tmp_path):
    """Width-3 beam search: the surviving beams and their cumulative log-probabilities equal a plain beam search carried out
    on HF's log-softmax outputs."""
    from xllm_wxh_b200.api.llm import BeamSearchParams
    torch.manual_seed(0)
    cfg = transformers.Qwen3Config(vocab_size=512, hidden_size=128, intermediate_size=344, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=32, max_position_embeddings=512, rms_norm_eps=1e-6,
                                   tie_word_embeddings=False, torch_dtype="float32", rope_theta=1000000.0)
    model = transformers.Qwen3ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for p in model.parameters():
            p.mul_(2.0)
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 512, (25,), generator=g).tolist()
    eng = LLMEngine(Options(model=str(tmp_path), devices="cpu", block_size=16, num_kv_blocks=128, dtype="float32"))
    out = LLM(model=str(tmp_path), devices="cpu", engine=eng).beam_search([prompt], BeamSearchParams(beam_width=3, max_tokens=5))[0]
    beams = [([], 0.0)]
    for _ in range(5):
        cand = []
        for toks, score in beams:
            with torch.no_grad():
                lp = torch.log_softmax(model(torch.tensor([prompt + toks])).logits[0, -1].float(), -1)
            top = torch.topk(lp, 3)
            cand += [(toks + [int(i)], score + float(v)) for v, i in zip(top.values, top.indices)]
        beams = sorted(cand, key=lambda x: -x[1])[:3]
    assert [o.token_ids for o in out.outputs] == [t for t, _ in beams]
    for o, (_, score) in zip(out.outputs, beams):
        assert abs(o.cumulative_logprob - score) < 1e-2


def test_frequency_and_presence_penalties_count_generated_tokens_only(tmp_path):
    """OpenAI semantics (and the reference's count map): logits of a token drop by frequency x (times it was generated) and
    by presence once it was generated at all; tokens that only occur in the prompt are not penalised."""
    torch.manual_seed(0)
    cfg = transformers.Qwen3Config(vocab_size=64, hidden_size=128, intermediate_size=344, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=32, max_position_embeddings=512, rms_norm_eps=1e-6,
                                   tie_word_embeddings=False, torch_dtype="float32", rope_theta=1000000.0)
    model = transformers.Qwen3ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for p in model.parameters():
            p.mul_(1.2)
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 64, (30,), generator=g).tolist()
    llm = LLM(model=str(tmp_path), devices="cpu", engine=_engine(tmp_path))
    n, fr, pr = 40, 0.6, 0.4
    base = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True))[0].outputs[0].token_ids
    got = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True, frequency_penalty=fr,
                                                presence_penalty=pr))[0].outputs[0].token_ids
    ids, gen = list(prompt), []
    with torch.no_grad():
        for _ in range(n):
            lg = model(torch.tensor([ids])).logits[0, -1].float()
            cnt = torch.bincount(torch.tensor(gen, dtype=torch.long), minlength=64).float()
            nxt = int((lg - fr * cnt - pr * (cnt > 0).float()).argmax())
            gen.append(nxt)
            ids.append(nxt)
    assert got == gen and got != base and len(set(got)) > len(set(base))


def test_qwen3_reranker_score_is_p_yes_against_p_no(tmp_path):
    """`--enable_qwen3_reranker`: the score of query + document is softmax(logit[no], logit[yes])[yes] at the position
    that would generate the answer, from one prefill; checked against Hugging Face logits, directly and through
    `/v1/rerank` (sorted, top_n)."""
    import asyncio
    from xllm_wxh_b200.api.openai_service import APIService
    from xllm_wxh_b200.api.server import Request
    from xllm_wxh_b200.runtime.embed import rerank_scores
    from xllm_wxh_b200.runtime.master import LLMMaster
    torch.manual_seed(0)
    cfg = transformers.Qwen3Config(vocab_size=512, hidden_size=128, intermediate_size=344, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=32, max_position_embeddings=512, rms_norm_eps=1e-6,
                                   tie_word_embeddings=False, torch_dtype="float32", rope_theta=1000000.0)
    model = transformers.Qwen3ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for p in model.parameters():
            p.mul_(1.5)
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    opts = Options(model=str(tmp_path), devices="cpu", block_size=16, num_kv_blocks=128, dtype="float32", enable_qwen3_reranker=True,
                   rerank_no_token_id=17, rerank_yes_token_id=301)
    eng = LLMEngine(opts)
    master = LLMMaster(opts, eng)
    query = "7 8 9 10 "
    docs = ["1 2 3 4 5", "400 401 402", "33 33 33 33 33 33 33", "250"]

    def hf_score(text):
        ids = master.tokenizer.encode(text)
        with torch.no_grad():
            lg = model(torch.tensor([ids])).logits[0, -1].float()
        return float(torch.softmax(lg[[17, 301]], -1)[1])
    want = [hf_score(query + d) for d in docs]
    got = rerank_scores(master, [query + d for d in docs])
    assert len(set(round(w, 4) for w in want)) > 1
    for a, b in zip(got, want):
        assert abs(a - b) < 1e-4, (got, want)
    svc = APIService(master, opts)
    body = {"model": master.model_id, "query": query, "documents": docs, "top_n": 3}
    import json as _json
    resp = asyncio.new_event_loop().run_until_complete(svc.rerank(Request("POST", "/v1/rerank", {}, {}, _json.dumps(body).encode())))
    res = _json.loads(resp.body)["results"]
    order = sorted(range(len(docs)), key=lambda i: -want[i])[:3]
    assert [r["index"] for r in res] == order
    for r in res:
        assert abs(r["relevance_score"] - want[r["index"]]) < 1e-4 and r["document"]["text"] == docs[r["index"]]
    # ids outside the vocabulary are refused with a message, not an index error inside a step
    eng.worker.yes_no_ids = (2152, 9693)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        rerank_scores(master, [query + docs[0]])
    master.stop()
