"""The C interface (libxllm.so, csrc/capi/xllm_c_api.h) driven through ctypes from this process, and from a plain C program
that embeds the interpreter."""
import ctypes
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "xllm_wxh_b200", "libxllm.so")


class Opts(ctypes.Structure):
    _fields_ = [("enable_prefix_cache", ctypes.c_bool), ("enable_chunked_prefill", ctypes.c_bool),
                ("enable_schedule_overlap", ctypes.c_bool), ("enable_graph", ctypes.c_bool), ("block_size", ctypes.c_int32),
                ("max_tokens_per_batch", ctypes.c_int32), ("max_seqs_per_batch", ctypes.c_int32),
                ("max_tokens_per_chunk_for_prefill", ctypes.c_int32), ("num_kv_blocks", ctypes.c_int32),
                ("max_memory_utilization", ctypes.c_double), ("dp_size", ctypes.c_int32), ("ep_size", ctypes.c_int32),
                ("num_speculative_tokens", ctypes.c_int32), ("draft_model", ctypes.c_char_p), ("dtype", ctypes.c_char_p)]


class Params(ctypes.Structure):
    _fields_ = [("max_tokens", ctypes.c_int32), ("n", ctypes.c_int32), ("temperature", ctypes.c_float), ("top_p", ctypes.c_float),
                ("top_k", ctypes.c_int32), ("repetition_penalty", ctypes.c_float), ("frequency_penalty", ctypes.c_float),
                ("presence_penalty", ctypes.c_float), ("ignore_eos", ctypes.c_bool), ("logprobs", ctypes.c_bool),
                ("top_logprobs", ctypes.c_int32), ("seed", ctypes.c_int64)]


class Usage(ctypes.Structure):
    _fields_ = [("prompt_tokens", ctypes.c_int32), ("completion_tokens", ctypes.c_int32), ("total_tokens", ctypes.c_int32)]


class Choice(ctypes.Structure):
    _fields_ = [("index", ctypes.c_int32), ("text", ctypes.c_char_p), ("token_ids", ctypes.POINTER(ctypes.c_int32)),
                ("num_token_ids", ctypes.c_size_t), ("token_logprobs", ctypes.POINTER(ctypes.c_float)),
                ("finish_reason", ctypes.c_char_p)]


class Response(ctypes.Structure):
    _fields_ = [("status_code", ctypes.c_int), ("error", ctypes.c_char_p), ("id", ctypes.c_char_p),
                ("choices", ctypes.POINTER(Choice)), ("num_choices", ctypes.c_size_t), ("usage", Usage)]


@pytest.mark.skipif(not os.path.exists(LIB), reason="libxllm.so not built")
def test_c_api_completions_through_ctypes():
    from oracle import greedy_generate
    from xllm_wxh_b200.models.args import preset
    from xllm_wxh_b200.models.qwen import QwenForCausalLM
    L = ctypes.PyDLL(LIB)            # PyDLL keeps the GIL handling consistent when called from Python
    L.xllm_llm_create.restype = ctypes.c_void_p
    L.xllm_llm_completions.restype = ctypes.POINTER(Response)
    L.xllm_llm_initialize.restype = ctypes.c_bool
    L.xllm_llm_last_error.restype = ctypes.c_char_p
    h = ctypes.c_void_p(L.xllm_llm_create())
    p = Params()
    L.xllm_llm_request_params_default(ctypes.byref(p))
    assert p.max_tokens == 5120 and p.temperature == 0.0 and p.top_k == -1
    # not initialised yet
    r = L.xllm_llm_completions(h, b"m", b"1 2 3", 0, ctypes.byref(p))
    assert r.contents.status_code == 1 and r.contents.error
    L.xllm_llm_free_response(r)
    o = Opts()
    L.xllm_llm_init_options_default(ctypes.byref(o))
    assert o.block_size == 128 and o.enable_prefix_cache
    o.block_size, o.num_kv_blocks, o.dtype, o.max_tokens_per_batch = 16, 128, b"float32", 512
    assert L.xllm_llm_initialize(h, b"preset:tiny-qwen2", b"cpu", ctypes.byref(o)), L.xllm_llm_last_error(h)
    p.max_tokens, p.ignore_eos, p.logprobs = 6, True, True
    r = L.xllm_llm_completions(h, b"tiny", b"5 6 7 8 9", 60000, ctypes.byref(p))
    resp = r.contents
    assert resp.status_code == 0 and resp.num_choices == 1, resp.error
    ch = resp.choices[0]
    ids = [ch.token_ids[i] for i in range(ch.num_token_ids)]
    args = preset("tiny-qwen2")
    sd = QwenForCausalLM(args, device="cpu").init_random(seed=0).state_dict()       # the engine's default seed
    assert ids == greedy_generate(sd, args, [5, 6, 7, 8, 9], 6)
    assert ch.finish_reason == b"length" and ch.text.decode().split() == [str(i) for i in ids]
    assert resp.usage.prompt_tokens == 5 and resp.usage.completion_tokens == 6 and resp.usage.total_tokens == 11
    assert all(ch.token_logprobs[i] <= 1e-4 for i in range(6))
    L.xllm_llm_free_response(r)
    L.xllm_llm_destroy(h)


C_PROGRAM = r'''
#include <stdio.h>
#include <string.h>
#include "xllm_c_api.h"
int main(void) {
  XLLM_LLM_Handler* h = xllm_llm_create();
  XLLM_InitLLMOptions o;
  xllm_llm_init_options_default(&o);
  o.block_size = 16; o.num_kv_blocks = 128; o.dtype = "float32"; o.max_tokens_per_batch = 512;
  if (!xllm_llm_initialize(h, "preset:tiny-qwen2", "cpu", &o)) { printf("init failed: %s\n", xllm_llm_last_error(h)); return 1; }
  XLLM_RequestParams p;
  xllm_llm_request_params_default(&p);
  p.max_tokens = 4; p.ignore_eos = true;
  XLLM_Response* r = xllm_llm_completions(h, "tiny", "1 2 3", 60000, &p);
  if (r->status_code != XLLM_OK) { printf("error: %s\n", r->error); return 2; }
  printf("tokens=%zu text=%s finish=%s\n", r->choices[0].num_token_ids, r->choices[0].text, r->choices[0].finish_reason);
  xllm_llm_free_response(r);
  xllm_llm_destroy(h);
  return 0;
}
'''


@pytest.mark.skipif(not os.path.exists(LIB), reason="libxllm.so not built")
def test_c_api_from_a_c_program(tmp_path):
    src = tmp_path / "main.c"
    src.write_text(C_PROGRAM)
    exe = str(tmp_path / "capi_demo")
    inc = os.path.join(ROOT, "xllm_wxh_b200", "csrc", "capi")
    libdir = os.path.join(ROOT, "xllm_wxh_b200")
    cc = subprocess.run(["gcc", str(src), "-I", inc, "-L", libdir, "-lxllm", f"-Wl,-rpath,{libdir}", "-o", exe],
                        stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert cc.returncode == 0, cc.stdout
    site = [p for p in sys.path if p.endswith("site-packages")]
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT] + site), PYTHONHOME=sys.base_prefix)
    p = subprocess.run([exe], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert p.returncode == 0 and "tokens=4" in p.stdout and "finish=length" in p.stdout, p.stdout[-3000:]


CPP_PROGRAM = r'''
#include <cstdio>
#include "xllm_llm.hpp"
int main() {
  xllm::LLM llm;
  XLLM_InitLLMOptions o = xllm::DefaultInitOptions();
  o.block_size = 16; o.num_kv_blocks = 128; o.dtype = "float32"; o.max_tokens_per_batch = 512;
  xllm::Response early = llm.Completions("tiny", "1 2 3", 1000);
  if (early.ok()) { std::printf("a request before Initialize must fail\n"); return 3; }
  if (!llm.Initialize("preset:tiny-qwen2", "cpu", o)) { std::printf("init failed: %s\n", llm.LastError().c_str()); return 1; }
  XLLM_RequestParams p = xllm::DefaultRequestParams();
  p.max_tokens = 4; p.ignore_eos = true; p.logprobs = true;
  xllm::Response r = llm.Completions("tiny", "1 2 3", 60000, p);
  if (!r.ok()) { std::printf("error: %s\n", r.error.c_str()); return 2; }
  std::printf("tokens=%zu logprobs=%zu finish=%s prompt_tokens=%d\n", r.choices[0].token_ids.size(), r.choices[0].token_logprobs.size(),
              r.choices[0].finish_reason.c_str(), r.usage.prompt_tokens);
  xllm::Response c = llm.ChatCompletions("tiny", {{"system", "7 8"}, {"user", "1 2 3"}}, 60000, p);
  if (!c.ok()) { std::printf("chat error: %s\n", c.error.c_str()); return 4; }
  std::printf("chat_tokens=%zu\n", c.choices[0].token_ids.size());
  return 0;
}
'''


@pytest.mark.skipif(not os.path.exists(LIB), reason="libxllm.so not built")
def test_cpp_class_api_from_a_cpp_program(tmp_path):
    """`xllm::LLM` (csrc/capi/xllm_llm.hpp): Initialize / Completions / ChatCompletions from a C++ program."""
    src = tmp_path / "main.cpp"
    src.write_text(CPP_PROGRAM)
    exe = str(tmp_path / "cppapi_demo")
    inc = os.path.join(ROOT, "xllm_wxh_b200", "csrc", "capi")
    libdir = os.path.join(ROOT, "xllm_wxh_b200")
    cc = subprocess.run(["g++", "-std=c++17", str(src), "-I", inc, "-L", libdir, "-lxllm", f"-Wl,-rpath,{libdir}", "-o", exe],
                        stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert cc.returncode == 0, cc.stdout
    site = [p for p in sys.path if p.endswith("site-packages")]
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT] + site), PYTHONHOME=sys.base_prefix)
    p = subprocess.run([exe], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert p.returncode == 0 and "tokens=4 logprobs=4 finish=length prompt_tokens=3" in p.stdout and "chat_tokens=4" in p.stdout, \
        p.stdout[-3000:]
