"""Host-only tests of the remaining C++ core parts and their Python front ends: byte-level BPE tokenizer (against the
HF `tokenizers` library on the same tokenizer.json), incremental detokenisation, safetensors reader, checkpoint
loader, suffix-tree drafter, chat template, request-parameter checks, rate limiter, shared-memory channel.

Same tier as the reference's fast_tokenizer_tests.cpp, hf_model_loader_test.cpp, suffix_decoding_cache_test.cpp,
jinja_chat_template_test.cpp, sampling_params_test.cpp and rate_limiter_test.cpp.
"""
import json
import os
import struct
import threading

import numpy as np
import pytest
import torch

from xllm_wxh_b200 import _core
from xllm_wxh_b200.utils import tokenizer as tk

QWEN_PATTERN = tk._QWEN_PATTERNS[0]


def _byte_level_alphabet():
    dec = tk._gpt2_byte_decoder()                 # printable stand-in character -> byte
    return {b: ch for ch, b in dec.items()}


def _write_tokenizer(dirname, corpus, n_merges=200):
    """A small byte-level BPE trained here by plain pair counting, written in tokenizer.json format."""
    enc = _byte_level_alphabet()
    words = {}
    import regex
    for piece in regex.findall(QWEN_PATTERN, corpus):
        w = tuple(enc[b] for b in piece.encode("utf-8"))
        words[w] = words.get(w, 0) + 1
    vocab = {enc[b]: b for b in range(256)}
    merges = []
    for _ in range(n_merges):
        pairs = {}
        for w, c in words.items():
            for a, b in zip(w, w[1:]):
                pairs[(a, b)] = pairs.get((a, b), 0) + c
        if not pairs:
            break
        (a, b), c = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))
        if c < 2:
            break
        merges.append(f"{a} {b}")
        vocab[a + b] = len(vocab)
        new = {}
        for w, c in words.items():
            out, i = [], 0
            while i < len(w):
                if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(w[i])
                    i += 1
            new[tuple(out)] = new.get(tuple(out), 0) + c
        words = new
    n = len(vocab)
    added = [{"id": n, "content": "<|endoftext|>", "single_word": False, "lstrip": False, "rstrip": False,
              "normalized": False, "special": True},
             {"id": n + 1, "content": "<|im_start|>", "single_word": False, "lstrip": False, "rstrip": False,
              "normalized": False, "special": True},
             {"id": n + 2, "content": "<|im_end|>", "single_word": False, "lstrip": False, "rstrip": False,
              "normalized": False, "special": True}]
    tj = {"version": "1.0", "truncation": None, "padding": None, "added_tokens": added, "normalizer": None,
          "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
              {"type": "Split", "pattern": {"Regex": QWEN_PATTERN}, "behavior": "Isolated", "invert": False},
              {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": False, "use_regex": False}]},
          "post_processor": None,
          "decoder": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": False, "use_regex": False},
          "model": {"type": "BPE", "dropout": None, "unk_token": None, "continuing_subword_prefix": "",
                    "end_of_word_suffix": "", "fuse_unk": False, "byte_fallback": False, "vocab": vocab, "merges": merges}}
    with open(os.path.join(dirname, "tokenizer.json"), "w", encoding="utf-8") as f:
        json.dump(tj, f, ensure_ascii=False)
    with open(os.path.join(dirname, "tokenizer_config.json"), "w") as f:
        json.dump({"eos_token": "<|im_end|>", "chat_template":
                   "{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{% endfor %}"
                   "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}"}, f)
    return n


CORPUS = ("The quick brown fox jumps over the lazy dog. the the the and and then there were 12345 numbers, "
          "it's what we'd expect; isn't it?  Tabs\tand\nnewlines\r\n too.   Trailing spaces   \n"
          "Unicode: naïve café 東京タワー 你好世界 Привет мир 🙂🙂 é x²  ") * 3


@pytest.fixture(scope="module")
def tok_dir(tmp_path_factory):
    d = tmp_path_factory.mktemp("tok")
    n = _write_tokenizer(str(d), CORPUS)
    return str(d), n


TEXTS = ["", " ", "hello", "Hello, world!", "the the  the   the", "it's isn't we'd THEY'LL I'M",
         "numbers 1 22 333 4444 55555", "tabs\t\tand\n\nnew\r\nlines \n ", "  leading and trailing  ",
         "naïve café — “quotes” …", "東京タワーは高い。你好，世界！", "Привет, мир! Ünïcödé", "🙂 emoji 🙂🙂 👨‍👩‍👧",
         "é combining, x² superscript, ½ fraction", "a" * 300, "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n",
         "special in the middle <|endoftext|> of text", " non-breaking spaces　here"]


def test_native_bpe_matches_hf_tokenizers(tok_dir):
    d, n = tok_dir
    native = tk._native_from_tokenizer_json(os.path.join(d, "tokenizer.json"))
    assert native is not None, "the pre-tokenizer pattern must be recognised"
    hf = tk.HFTokenizer(os.path.join(d, "tokenizer.json"))
    assert native.vocab_size == hf.vocab_size == n + 3
    rng = np.random.default_rng(0)
    alphabet = list("abcdefghijklmnopqrstuvwxyz THEQUICK0123456789.,;'!?\n\t-é東京界🙂") + ["'s", "'ll", "  ", "\r\n"]
    texts = TEXTS + ["".join(rng.choice(alphabet, int(rng.integers(1, 80)))) for _ in range(300)]
    for t in texts:
        a, b = native.encode(t), hf.encode(t)
        assert a == b, repr(t)
        assert native.decode(a, skip_special_tokens=False) == t
    ids = native.encode("<|im_start|>x<|im_end|>")
    assert ids[0] == n + 1 and ids[-1] == n + 2
    assert native.decode(ids) == "x" and native.decode(ids, skip_special_tokens=False) == "<|im_start|>x<|im_end|>"
    assert native.token_to_id("<|endoftext|>") == n and native.id_to_token(n + 2) == "<|im_end|>"


def test_load_tokenizer_reads_config_and_template(tok_dir):
    d, n = tok_dir
    t = tk.load_tokenizer(d)
    assert isinstance(t, tk.NativeBpeTokenizer) and t.eos_token_id == n + 2
    from xllm_wxh_b200.api.chat_template import JinjaChatTemplate
    tpl = JinjaChatTemplate(t.chat_template, t)
    text = tpl.apply([{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}])
    assert text == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    assert tpl.apply([{"role": "user", "content": "hi"}], add_generation_prompt=False).endswith("<|im_end|>\n")
    assert t.encode(text).count(n + 1) == 3
    # no directory: prompts are token ids
    ident = tk.load_tokenizer(None, vocab_size=100, eos_token_id=7)
    assert ident.encode("3 4 5") == [3, 4, 5] and ident.decode([3, 4]).split() == ["3", "4"]


def test_chat_template_tools_kwargs_and_errors():
    from xllm_wxh_b200.api.chat_template import JinjaChatTemplate
    tpl = JinjaChatTemplate("{% if tools %}TOOLS {{ tools | tojson }}\n{% endif %}"
                            "{% for m in messages %}{{ m.role }}:{{ m.content }};{% endfor %}"
                            "{% if enable_thinking is defined and not enable_thinking %}<think></think>{% endif %}"
                            "{% if messages | length == 0 %}{{ raise_exception('no messages') }}{% endif %}")
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object"}}}]
    out = tpl.apply([{"role": "user", "content": "é"}], tools=tools, kwargs={"enable_thinking": False})
    assert out.startswith('TOOLS [{"type": "function"') and "user:é;" in out and out.endswith("<think></think>")
    with pytest.raises(Exception):
        tpl.apply([])


def test_incremental_decoder_never_splits_a_character(tok_dir):
    d, _ = tok_dir
    t = tk.load_tokenizer(d)
    text = "naïve 東京タワー 🙂🙂 done"
    ids = t.encode(text)
    dec = tk.IncrementalDecoder(t)
    pieces = [dec.add([i]) for i in ids] + [dec.flush()]
    assert "".join(pieces) == text
    assert all("�" not in p for p in pieces)       # a character is released only when all its bytes arrived
    dec = tk.IncrementalDecoder(t)
    assert dec.add(ids[:5]) + dec.add(ids[5:]) + dec.flush() == text


def test_incremental_decoder_text_tokenizers_decode_a_short_window_only():
    """A tokenizer that only gives text (here: one token per UTF-8 byte, unfinished characters decode to U+FFFD, as with
    byte-fallback vocabularies): the pieces join to the text, no piece carries a replacement character, and every call
    decodes a handful of tokens however long the output has grown."""
    class ByteTok(tk.Tokenizer):
        def __init__(self):
            self.longest = 0
        def encode(self, text, add_special_tokens=True):
            return list(text.encode("utf-8"))
        def decode(self, ids, skip_special_tokens=True):
            self.longest = max(self.longest, len(ids))
            return bytes(ids).decode("utf-8", "replace")
        def token_to_id(self, tok):
            return -1
        def id_to_token(self, i):
            return chr(i)
        @property
        def vocab_size(self):
            return 256
    t = ByteTok()
    text = "naïve 東京タワー 🙂🙂 done " * 40
    ids = t.encode(text)
    dec = tk.IncrementalDecoder(t)
    pieces = [dec.add([i]) for i in ids] + [dec.flush()]
    assert "".join(pieces) == text and all("\ufffd" not in p for p in pieces)
    assert t.longest <= 8, t.longest                      # never the whole list
    dec = tk.IncrementalDecoder(t)
    assert dec.add(ids[:7]) + dec.add(ids[7:300]) + dec.add(ids[300:]) + dec.flush() == text
    # an output that ends inside a character: the held bytes come out of flush() as they are
    cut = t.encode("ab東")[:-1]
    dec = tk.IncrementalDecoder(t)
    assert "".join(dec.add([i]) for i in cut) == "ab" and dec.flush() == bytes(cut[2:]).decode("utf-8", "replace")
    # the preset tokenizer (ids as text)
    ident = tk.load_tokenizer(None, vocab_size=100, eos_token_id=7)
    dec = tk.IncrementalDecoder(ident)
    assert "".join(dec.add([i]) for i in (3, 44, 5)) + dec.flush() == ident.decode([3, 44, 5])


# ------------------------------------------------------------------ safetensors / checkpoint
def test_safetensors_reader_and_checkpoint_loader(tmp_path):
    from xllm_wxh_b200.utils.safetensors_io import CheckpointReader, save_safetensors
    g = torch.Generator().manual_seed(0)
    a = {"model.embed_tokens.weight": torch.randn(16, 8, generator=g).to(torch.bfloat16),
         "model.layers.0.w": torch.randn(4, 8, generator=g), "scalar": torch.tensor(3.5),
         "ints": torch.arange(6, dtype=torch.int64).reshape(2, 3), "empty": torch.zeros(0, 4),
         "f8": torch.randn(8, 8, generator=g).to(torch.float8_e4m3fn), "half": torch.randn(3, generator=g).half()}
    b = {"model.layers.1.w": torch.randn(4, 8, generator=g), "flags": torch.tensor([True, False])}
    save_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), a, metadata={"format": "pt"})
    save_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), b)
    f = _core.SafeTensorsFile(str(tmp_path / "model-00001-of-00002.safetensors"))
    assert sorted(f.keys()) == sorted(a) and f.metadata == {"format": "pt"}
    info = f.info("model.embed_tokens.weight")
    assert info.dtype == "BF16" and info.shape == [16, 8] and info.end - info.begin == 16 * 8 * 2
    assert bytes(f.view("ints")) == a["ints"].numpy().tobytes()
    assert f.has("scalar") and not f.has("nope")
    with pytest.raises(Exception):
        f.info("nope")
    ck = CheckpointReader(str(tmp_path))
    assert sorted(ck.keys()) == sorted(list(a) + list(b))
    for name, t in {**a, **b}.items():
        got = ck.get(name)
        assert got.dtype == t.dtype and got.shape == t.shape
        assert torch.equal(got.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else got,
                           t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t), name
    assert ck.get_or_none("missing") is None
    assert [k for k, _ in ck.items("model.layers.")] == ["model.layers.0.w", "model.layers.1.w"]


@pytest.mark.parametrize("damage", ["short", "header_len", "json", "offsets"])
def test_safetensors_rejects_damaged_files(tmp_path, damage):
    p = tmp_path / "x.safetensors"
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}).encode()
    body = struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8
    if damage == "short":
        body = body[:5]
    elif damage == "header_len":
        body = struct.pack("<Q", 1 << 40) + body[8:]
    elif damage == "json":
        body = struct.pack("<Q", len(hdr)) + b"{" * len(hdr) + b"\0" * 8
    else:
        hdr2 = json.dumps({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 64]}}).encode()
        body = struct.pack("<Q", len(hdr2)) + hdr2 + b"\0" * 8
    p.write_bytes(body)
    with pytest.raises(Exception):
        _core.SafeTensorsFile(str(p))


def test_model_round_trips_through_a_checkpoint_directory(tmp_path):
    """Weights saved in the HF layout load back into the same logits (hf_model_loader_test.cpp's role)."""
    from xllm_wxh_b200.models.args import preset
    from xllm_wxh_b200.models.qwen import QwenForCausalLM
    from xllm_wxh_b200.utils.safetensors_io import save_safetensors
    args = preset("tiny-qwen2")
    m = QwenForCausalLM(args, device="cpu").init_random(seed=3)
    sd = m.state_dict()
    assert "model.layers.0.self_attn.q_proj.weight" in sd and "model.layers.0.mlp.gate_proj.weight" in sd
    save_safetensors(str(tmp_path / "model.safetensors"), sd)
    with open(tmp_path / "config.json", "w") as f:
        json.dump({
            "model_type": "qwen2", "hidden_size": args.hidden_size, "num_hidden_layers": args.n_layers,
            "num_attention_heads": args.n_heads, "num_key_value_heads": args.n_kv_heads,
            "intermediate_size": args.intermediate_size, "vocab_size": args.vocab_size, "rms_norm_eps": args.rms_norm_eps,
            "rope_theta": args.rope_theta, "max_position_embeddings": args.max_position_embeddings,
            "tie_word_embeddings": args.tie_word_embeddings, "head_dim": args.head_dim, "torch_dtype": "float32"}, f)
    from xllm_wxh_b200.models.args import load_model_args
    args2 = load_model_args(str(tmp_path))
    assert (args2.hidden_size, args2.n_layers, args2.n_heads, args2.n_kv_heads, args2.head_dim, args2.attention_bias) == \
           (args.hidden_size, args.n_layers, args.n_heads, args.n_kv_heads, args.head_dim, args.attention_bias)
    from xllm_wxh_b200.utils.safetensors_io import CheckpointReader
    args2.dtype = "float32"
    m2 = QwenForCausalLM(args2, device="cpu").load_weights(CheckpointReader(str(tmp_path)))
    sd2 = m2.state_dict()
    assert set(sd2) == set(sd)
    for k in sd:
        assert torch.equal(sd[k].float(), sd2[k].float()), k


# ------------------------------------------------------------------ suffix-tree drafter
def test_suffix_cache_speculates_repeats():
    c = _core.SuffixCache(max_depth=16)
    c.append(1, [5, 6, 7, 8, 9, 5, 6, 7])
    assert c.speculate(1, [5, 6, 7], 3) == [8, 9, 5]            # what followed "5 6 7" last time
    assert c.speculate(1, [6, 7], 2) == [8, 9]
    assert c.speculate(1, [1, 2], 3) == []                       # unseen context
    assert c.speculate(1, [7], 3, 2) == []                       # match shorter than min_match
    c.append(2, [5, 6, 7, 1, 1])
    assert c.speculate(2, [5, 6, 7], 2) in ([1, 1], [8, 9])      # global tree: either continuation is a seen one
    n = c.num_nodes
    c.evict(1)
    assert c.num_nodes <= n and c.speculate(1, [5, 6, 7], 3) in ([], [1, 1])


def test_suffix_cache_scored_speculation_follows_the_reference_rule():
    """A match of m tokens proposes at most m * factor + offset tokens; a token is proposed while the product of the
    branch frequencies on the way to it is at least min_token_prob; the proposal with the largest sum of those products
    wins.  First cases: the vectors of the reference's suffix_decoding_cache_test.cpp (AddResponseAndSpeculate,
    GlobalCacheSpeculateAcrossRequests)."""
    c = _core.SuffixCache(max_depth=32)
    c.append(1, [1, 2, 3, 4, 5, 6, 7])
    d = c.speculate_scored([2, 3, 4], 4, 2.0, 0.0, 0.01)
    assert d[:1] == [5] and d == [5, 6, 7]
    g = _core.SuffixCache(max_depth=32)
    g.append(1, [10, 20, 30, 40, 50, 60])
    g.append(2, [1, 2, 10, 20, 30, 40])
    assert g.speculate_scored([20, 30, 40], 3, 2.0, 0.0, 0.01)[:1] == [50]
    # the length cap: a one-token match with factor 1 proposes one token, offset adds to it
    t = _core.SuffixCache(max_depth=32)
    t.append(1, [9, 1, 2, 3, 4, 8, 1, 2, 3, 4])
    assert t.speculate_scored([7, 4], 4, 1.0, 0.0, 0.01) == [8]              # only "4" matches: 1 token allowed
    assert t.speculate_scored([7, 4], 4, 1.0, 2.0, 0.01) == [8, 1, 2]        # 1 * 1 + 2
    assert t.speculate_scored([1, 2, 3], 4, 1.0, 0.0, 0.01) == [4, 8, 1]     # three tokens matched: three allowed
    assert t.speculate_scored([5, 5], 4, 2.0, 0.0, 0.01) == []               # unseen context
    # the probability floor: after "1 2" comes 3 three times and 7 once
    p = _core.SuffixCache(max_depth=32)
    p.append(1, [1, 2, 3, 0, 1, 2, 3, 0, 1, 2, 3, 0, 1, 2, 7])
    assert p.speculate_scored([1, 2], 3, 2.0, 0.0, 0.5) == [3, 0, 1]         # 3/4, then certain continuations
    assert p.speculate_scored([1, 2], 3, 2.0, 0.0, 0.8) == []                # 0.75 is below the floor
    assert p.speculate_scored([0, 1, 2], 2, 2.0, 0.0, 0.7) == [3, 0]         # the shorter matches (3/4) carry it
    assert p.speculate_scored([0, 1, 2], 2, 2.0, 0.0, 0.9) == []


# ------------------------------------------------------------------ request parameters / rate limiter
def test_request_params_verify_and_mapping():
    from xllm_wxh_b200.api.openai_service import params_from_body
    from xllm_wxh_b200.framework.params import RequestParams
    assert RequestParams().verify().ok
    for bad in (dict(n=0), dict(n=2, best_of=1), dict(temperature=2.5), dict(top_p=0.0), dict(top_p=1.5),
                dict(frequency_penalty=3.0), dict(presence_penalty=-2.5), dict(repetition_penalty=0.0),
                dict(max_tokens=0), dict(top_logprobs=21), dict(streaming=True, n=1, best_of=2)):
        st = RequestParams(**bad).verify()
        assert not st.ok, bad
    p = params_from_body({"max_tokens": 7, "temperature": 0.5, "top_p": 0.8, "top_k": 5, "n": 2, "best_of": 3, "seed": 9,
                          "stop": ["\n\n"], "stop_token_ids": [3], "ignore_eos": True, "priority": 1, "offline": True,
                          "ttft_slo_ms": 200, "tpot_slo_ms": 30, "ttft_priority_weight": 3, "repetition_penalty": 1.1,
                          "frequency_penalty": 0.2, "presence_penalty": 0.1, "logprobs": 2}, chat=False)
    assert (p.max_tokens, p.n, p.best_of, p.seed, p.priority, p.offline) == (7, 2, 3, 9, 1, True)
    assert (p.ttft_slo_ms, p.tpot_slo_ms, p.ttft_priority_weight, p.tpot_priority_weight) == (200.0, 30.0, 3, 1)
    sp, st = p.to_core(eos_token_id=2, extra_stop_ids=[4], stop_sequences=[[8, 9]])
    assert sp.temperature == pytest.approx(0.5) and sp.top_k == 5 and sp.seed == 9 and sp.logprobs
    assert sp.repetition_penalty == pytest.approx(1.1) and sp.frequency_penalty == pytest.approx(0.2)
    assert st.max_tokens == 7 and st.eos_token_id == 2 and st.ignore_eos and st.stop_token_ids == [3, 4]
    assert st.stop_sequences == [[8, 9]]
    c = params_from_body({"messages": [], "logprobs": True, "top_logprobs": 4, "max_completion_tokens": 11}, chat=True)
    assert c.logprobs and c.top_logprobs == 4 and c.max_tokens == 11


def test_rate_limiter_counts_concurrent_requests():
    from xllm_wxh_b200.api.openai_service import RateLimiter
    r = RateLimiter(2)
    assert r.acquire() and r.acquire() and not r.acquire()
    r.release()
    assert r.acquire() and not r.acquire()
    unlimited = RateLimiter(0)
    assert all(unlimited.acquire() for _ in range(100))
    r = RateLimiter(8)
    got = []
    def worker():
        ok = r.acquire()
        got.append(ok)
    ts = [threading.Thread(target=worker) for _ in range(32)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert sum(got) == 8


# ------------------------------------------------------------------ shared-memory step channel
def test_shm_channel_broadcasts_in_order_to_every_reader():
    name = f"/xl_test_{os.getpid()}_bc"
    w = _core.ShmChannel(name, 1 << 12, 2, True)
    r = _core.ShmChannel(name, 1 << 12, 2, False)
    try:
        msgs = [bytes([i]) * (i * 37 + 1) for i in range(1, 9)]
        out = {0: [], 1: []}
        def reader(k):
            for _ in msgs:
                out[k].append(r.read(k, 5.0))
        ts = [threading.Thread(target=reader, args=(k,)) for k in (0, 1)]
        [t.start() for t in ts]
        for m in msgs:
            assert w.write(m, 5.0) == 0              # a slot is reused only after both readers took the message
        [t.join() for t in ts]
        assert out[0] == msgs and out[1] == msgs
        assert r.read(0, 0.05) is None               # nothing pending: bounded wait, then None
        assert w.write(b"x" * (1 << 13), 0.05) != 0  # larger than the channel
    finally:
        w.close()
        _core.ShmChannel.unlink(name)


def test_fp8_checkpoints_of_a_dense_model_load_dequantised(tmp_path):
    """A Qwen checkpoint whose projection weights are fp8 with per-tensor, per-channel or 128 x 128 block scales (and
    static input scales, which a bf16 compute path ignores) loads into the same model up to the quantisation error."""
    from xllm_wxh_b200.models.args import ModelArgs
    from xllm_wxh_b200.models.qwen import QwenForCausalLM
    from xllm_wxh_b200.ops import reference as ref
    from xllm_wxh_b200.utils.safetensors_io import CheckpointReader, DequantizingReader, save_safetensors
    args = ModelArgs(model_type="qwen3", dtype="float32", vocab_size=512, hidden_size=256, n_layers=2, n_heads=4, n_kv_heads=2,
                     head_dim=64, intermediate_size=512, qk_norm=True, max_position_embeddings=512)
    m = QwenForCausalLM(args, device="cpu").init_random(seed=4, std=0.05)
    sd = m.state_dict()
    q = {}
    modes = ["tensor", "channel", "block"]
    n_q = 0
    for k, v in sd.items():
        if v.dim() == 2 and k.endswith("_proj.weight") and v.shape[0] % 128 == 0 and v.shape[1] % 128 == 0:
            mode = modes[n_q % 3]
            n_q += 1
            if mode == "block":
                q[k], q[k.replace(".weight", ".weight_scale_inv")] = ref.quant_weight_128x128(v)
            else:
                amax = v.abs().amax(dim=None if mode == "tensor" else 1, keepdim=mode == "channel").clamp_min(1e-8)
                scale = (amax / 448.0).float()
                q[k] = (v / scale).to(torch.float8_e4m3fn)
                q[k.replace(".weight", ".weight_scale")] = scale.reshape(-1) if mode == "channel" else scale.reshape(1)
                q[k.replace(".weight", ".input_scale")] = torch.tensor([0.02])
        else:
            q[k] = v
    assert n_q >= 6
    save_safetensors(str(tmp_path / "model.safetensors"), q)
    ck = CheckpointReader(str(tmp_path))
    assert ck.get("model.layers.0.self_attn.q_proj.weight").dtype == torch.float8_e4m3fn
    dq = DequantizingReader(ck)
    assert dq.get("model.layers.0.self_attn.q_proj.weight").dtype == torch.bfloat16
    m2 = QwenForCausalLM(args, device="cpu").load_weights(ck)
    sd2 = m2.state_dict()
    for k, v in sd.items():
        err = (sd2[k].float() - v.float()).abs().max().item()
        assert err <= 0.08 * v.abs().max().item() + 1e-6, (k, err)
    bad = dict(q)
    del bad["model.layers.0.self_attn.q_proj.weight_scale"]
    (tmp_path / "bad").mkdir()
    save_safetensors(str(tmp_path / "bad" / "model.safetensors"), bad)
    with pytest.raises(ValueError):
        QwenForCausalLM(args, device="cpu").load_weights(CheckpointReader(str(tmp_path / "bad")))
