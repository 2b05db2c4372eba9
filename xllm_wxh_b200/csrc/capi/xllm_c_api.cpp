// libxllm.so: the C interface declared in xllm_c_api.h, implemented over the package's Python API through the CPython
// C API.  A host program without an interpreter gets one embedded (initialised at the first xllm_llm_create); inside a
// Python process (ctypes, tests) the running interpreter is used.  Every entry point takes the GIL for its duration.
#include "xllm_c_api.h"

#include <Python.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

struct XLLM_LLM_Handler {
  PyObject* llm = nullptr;          // xllm_wxh_b200.LLM
  PyObject* mod = nullptr;          // the package
  std::mutex mu;
  std::string error;
  bool owns_interpreter = false;
};

namespace {

struct Gil {
  PyGILState_STATE st;
  Gil() : st(PyGILState_Ensure()) {}
  ~Gil() { PyGILState_Release(st); }
};

char* dup_str(const std::string& s) {
  char* p = static_cast<char*>(std::malloc(s.size() + 1));
  std::memcpy(p, s.c_str(), s.size() + 1);
  return p;
}

std::string py_error() {
  std::string msg = "python error";
  PyObject *t = nullptr, *v = nullptr, *tb = nullptr;
  PyErr_Fetch(&t, &v, &tb);
  PyErr_NormalizeException(&t, &v, &tb);
  if (v) {
    PyObject* s = PyObject_Str(v);
    if (s) {
      const char* c = PyUnicode_AsUTF8(s);
      if (c) msg = c;
      Py_DECREF(s);
    }
  }
  Py_XDECREF(t); Py_XDECREF(v); Py_XDECREF(tb);
  return msg;
}

XLLM_Response* make_error(XLLM_StatusCode code, const std::string& msg) {
  XLLM_Response* r = static_cast<XLLM_Response*>(std::calloc(1, sizeof(XLLM_Response)));
  r->status_code = code;
  r->error = dup_str(msg);
  return r;
}

std::string attr_str(PyObject* o, const char* name) {
  std::string out;
  PyObject* a = PyObject_GetAttrString(o, name);
  if (a && a != Py_None) {
    PyObject* s = PyObject_Str(a);
    if (s) {
      const char* c = PyUnicode_AsUTF8(s);
      if (c) out = c;
      Py_DECREF(s);
    }
  }
  if (!a) PyErr_Clear();
  Py_XDECREF(a);
  return out;
}

long attr_long(PyObject* o, const char* name, long dflt = 0) {
  PyObject* a = PyObject_GetAttrString(o, name);
  long v = dflt;
  if (a && PyLong_Check(a)) v = PyLong_AsLong(a);
  if (!a) PyErr_Clear();
  Py_XDECREF(a);
  return v;
}

// RequestOutput -> XLLM_Response
XLLM_Response* to_response(PyObject* out) {
  XLLM_Response* r = static_cast<XLLM_Response*>(std::calloc(1, sizeof(XLLM_Response)));
  r->id = dup_str(attr_str(out, "request_id"));
  PyObject* status = PyObject_GetAttrString(out, "status");
  if (status && status != Py_None) {
    PyObject* ok = PyObject_GetAttrString(status, "ok");
    const bool good = ok && PyObject_IsTrue(ok);
    Py_XDECREF(ok);
    if (!good) {
      r->status_code = XLLM_INTERNAL_ERROR;
      r->error = dup_str(attr_str(status, "message"));
    }
  }
  if (!status) PyErr_Clear();
  Py_XDECREF(status);
  PyObject* usage = PyObject_GetAttrString(out, "usage");
  if (usage && usage != Py_None) {
    r->usage.prompt_tokens = int32_t(attr_long(usage, "num_prompt_tokens"));
    r->usage.completion_tokens = int32_t(attr_long(usage, "num_generated_tokens"));
    r->usage.total_tokens = r->usage.prompt_tokens + r->usage.completion_tokens;
  }
  if (!usage) PyErr_Clear();
  Py_XDECREF(usage);
  PyObject* outs = PyObject_GetAttrString(out, "outputs");
  if (outs && PyList_Check(outs)) {
    const Py_ssize_t n = PyList_Size(outs);
    r->num_choices = size_t(n);
    r->choices = static_cast<XLLM_Choice*>(std::calloc(size_t(n) ? size_t(n) : 1, sizeof(XLLM_Choice)));
    for (Py_ssize_t i = 0; i < n; ++i) {
      PyObject* so = PyList_GetItem(outs, i);      // borrowed
      XLLM_Choice& c = r->choices[i];
      c.index = int32_t(attr_long(so, "index", long(i)));
      c.text = dup_str(attr_str(so, "text"));
      c.finish_reason = dup_str(attr_str(so, "finish_reason"));
      PyObject* ids = PyObject_GetAttrString(so, "token_ids");
      if (ids && PyList_Check(ids)) {
        c.num_token_ids = size_t(PyList_Size(ids));
        c.token_ids = static_cast<int32_t*>(std::malloc(sizeof(int32_t) * (c.num_token_ids ? c.num_token_ids : 1)));
        for (size_t j = 0; j < c.num_token_ids; ++j) c.token_ids[j] = int32_t(PyLong_AsLong(PyList_GetItem(ids, Py_ssize_t(j))));
      }
      if (!ids) PyErr_Clear();
      Py_XDECREF(ids);
      PyObject* lps = PyObject_GetAttrString(so, "logprobs");
      if (lps && PyList_Check(lps) && size_t(PyList_Size(lps)) == c.num_token_ids && c.num_token_ids) {
        c.token_logprobs = static_cast<float*>(std::malloc(sizeof(float) * c.num_token_ids));
        for (size_t j = 0; j < c.num_token_ids; ++j) {
          PyObject* lp = PyObject_GetAttrString(PyList_GetItem(lps, Py_ssize_t(j)), "logprob");
          c.token_logprobs[j] = lp ? float(PyFloat_AsDouble(lp)) : 0.f;
          Py_XDECREF(lp);
        }
      }
      if (!lps) PyErr_Clear();
      Py_XDECREF(lps);
    }
  }
  if (!outs) PyErr_Clear();
  Py_XDECREF(outs);
  return r;
}

PyObject* make_sampling_params(XLLM_LLM_Handler* h, const XLLM_RequestParams* p) {
  XLLM_RequestParams d;
  xllm_llm_request_params_default(&d);
  if (p) d = *p;
  PyObject* cls = PyObject_GetAttrString(h->mod, "SamplingParams");
  if (!cls) return nullptr;
  PyObject* kw = Py_BuildValue("{s:i,s:i,s:f,s:f,s:i,s:f,s:f,s:f,s:O,s:O,s:i}", "max_tokens", int(d.max_tokens), "n", int(d.n),
                               "temperature", d.temperature, "top_p", d.top_p, "top_k", int(d.top_k), "repetition_penalty",
                               d.repetition_penalty, "frequency_penalty", d.frequency_penalty, "presence_penalty",
                               d.presence_penalty, "ignore_eos", d.ignore_eos ? Py_True : Py_False, "logprobs",
                               d.logprobs ? Py_True : Py_False, "top_logprobs", int(d.top_logprobs));
  if (kw && d.seed >= 0) {
    PyObject* s = PyLong_FromLongLong(d.seed);
    PyDict_SetItemString(kw, "seed", s);
    Py_DECREF(s);
  }
  PyObject* args = PyTuple_New(0);
  PyObject* sp = kw ? PyObject_Call(cls, args, kw) : nullptr;
  Py_DECREF(args);
  Py_XDECREF(kw);
  Py_DECREF(cls);
  return sp;
}

XLLM_Response* run_generate(XLLM_LLM_Handler* h, PyObject* prompt, uint32_t timeout_ms, const XLLM_RequestParams* params) {
  PyObject* sp = make_sampling_params(h, params);
  if (!sp) return make_error(XLLM_INVALID_ARGUMENT, py_error());
  if (timeout_ms > 0) {
    PyObject* t = PyFloat_FromDouble(timeout_ms / 1e3);
    PyObject_SetAttrString(h->llm, "generate_timeout_s", t);
    Py_DECREF(t);
  }
  PyObject* outs = PyObject_CallMethod(h->llm, "generate", "OO", prompt, sp);
  Py_DECREF(sp);
  if (!outs) return make_error(XLLM_INTERNAL_ERROR, py_error());
  XLLM_Response* r = nullptr;
  if (PyList_Check(outs) && PyList_Size(outs) >= 1) r = to_response(PyList_GetItem(outs, 0));
  else r = make_error(XLLM_INTERNAL_ERROR, "generate returned no output");
  Py_DECREF(outs);
  return r;
}

}  // namespace

extern "C" {

XLLM_LLM_Handler* xllm_llm_create(void) {
  XLLM_LLM_Handler* h = new XLLM_LLM_Handler();
  if (!Py_IsInitialized()) {
    Py_InitializeEx(0);
    h->owns_interpreter = true;
    PyEval_SaveThread();               // release the GIL taken by the initialisation; entry points re-acquire it
  }
  return h;
}

void xllm_llm_destroy(XLLM_LLM_Handler* h) {
  if (!h) return;
  {
    Gil g;
    if (h->llm) {
      PyObject* r = PyObject_CallMethod(h->llm, "finish", nullptr);
      if (!r) PyErr_Clear();
      Py_XDECREF(r);
    }
    Py_XDECREF(h->llm);
    Py_XDECREF(h->mod);
  }
  delete h;       // an embedded interpreter stays alive for the process: CUDA contexts and extension modules outlive handlers
}

void xllm_llm_init_options_default(XLLM_InitLLMOptions* o) {
  if (!o) return;
  std::memset(o, 0, sizeof(*o));
  o->enable_prefix_cache = true;
  o->enable_chunked_prefill = true;
  o->enable_schedule_overlap = false;
  o->enable_graph = true;
  o->block_size = 128;
  o->max_tokens_per_batch = 20480;
  o->max_seqs_per_batch = 256;
  o->max_tokens_per_chunk_for_prefill = -1;
  o->num_kv_blocks = 0;
  o->max_memory_utilization = 0.9;
  o->dp_size = 1;
  o->ep_size = 1;
  o->num_speculative_tokens = 0;
  o->draft_model = nullptr;
  o->dtype = nullptr;
}

bool xllm_llm_initialize(XLLM_LLM_Handler* h, const char* model_path, const char* devices, const XLLM_InitLLMOptions* options) {
  if (!h || !model_path) return false;
  std::lock_guard<std::mutex> lk(h->mu);
  Gil g;
  XLLM_InitLLMOptions o;
  xllm_llm_init_options_default(&o);
  if (options) o = *options;
  if (!h->mod) h->mod = PyImport_ImportModule("xllm_wxh_b200");
  if (!h->mod) { h->error = py_error(); return false; }
  PyObject* cls = PyObject_GetAttrString(h->mod, "LLM");
  if (!cls) { h->error = py_error(); return false; }
  PyObject* kw = Py_BuildValue("{s:s,s:s,s:O,s:O,s:O,s:O,s:i,s:i,s:i,s:i,s:d,s:i,s:i,s:i}", "model", model_path, "devices",
                               devices ? devices : "auto", "disable_prefix_cache", o.enable_prefix_cache ? Py_False : Py_True,
                               "disable_chunked_prefill", o.enable_chunked_prefill ? Py_False : Py_True,
                               "enable_schedule_overlap", o.enable_schedule_overlap ? Py_True : Py_False, "enable_graph",
                               o.enable_graph ? Py_True : Py_False, "block_size", int(o.block_size), "max_tokens_per_batch",
                               int(o.max_tokens_per_batch), "max_seqs_per_batch", int(o.max_seqs_per_batch),
                               "max_tokens_per_chunk_for_prefill", int(o.max_tokens_per_chunk_for_prefill),
                               "max_memory_utilization", o.max_memory_utilization, "dp_size", int(o.dp_size), "ep_size",
                               int(o.ep_size), "num_speculative_tokens", int(o.num_speculative_tokens));
  if (kw && o.num_kv_blocks > 0) {
    PyObject* v = PyLong_FromLong(o.num_kv_blocks);
    PyDict_SetItemString(kw, "num_kv_blocks", v);
    Py_DECREF(v);
  }
  if (kw && o.draft_model) {
    PyObject* v = PyUnicode_FromString(o.draft_model);
    PyDict_SetItemString(kw, "draft_model", v);
    Py_DECREF(v);
  }
  if (kw && o.dtype) {
    PyObject* v = PyUnicode_FromString(o.dtype);
    PyDict_SetItemString(kw, "dtype", v);
    Py_DECREF(v);
  }
  PyObject* args = PyTuple_New(0);
  PyObject* llm = kw ? PyObject_Call(cls, args, kw) : nullptr;
  Py_DECREF(args);
  Py_XDECREF(kw);
  Py_DECREF(cls);
  if (!llm) { h->error = py_error(); return false; }
  Py_XDECREF(h->llm);
  h->llm = llm;
  h->error.clear();
  return true;
}

void xllm_llm_request_params_default(XLLM_RequestParams* p) {
  if (!p) return;
  p->max_tokens = 5120;
  p->n = 1;
  p->temperature = 0.0f;
  p->top_p = 1.0f;
  p->top_k = -1;
  p->repetition_penalty = 1.0f;
  p->frequency_penalty = 0.0f;
  p->presence_penalty = 0.0f;
  p->ignore_eos = false;
  p->logprobs = false;
  p->top_logprobs = 0;
  p->seed = -1;
}

XLLM_Response* xllm_llm_completions(XLLM_LLM_Handler* h, const char* /*model_id*/, const char* prompt, uint32_t timeout_ms,
                                    const XLLM_RequestParams* params) {
  if (!h || !h->llm) return make_error(XLLM_NOT_INITIALIZED, "handler is not initialised");
  if (!prompt) return make_error(XLLM_INVALID_ARGUMENT, "prompt is NULL");
  std::lock_guard<std::mutex> lk(h->mu);
  Gil g;
  PyObject* p = PyUnicode_FromString(prompt);
  if (!p) return make_error(XLLM_INVALID_ARGUMENT, py_error());
  XLLM_Response* r = run_generate(h, p, timeout_ms, params);
  Py_DECREF(p);
  return r;
}

XLLM_Response* xllm_llm_chat_completions(XLLM_LLM_Handler* h, const char* /*model_id*/, const XLLM_ChatMessage* messages,
                                         size_t num_messages, uint32_t timeout_ms, const XLLM_RequestParams* params) {
  if (!h || !h->llm) return make_error(XLLM_NOT_INITIALIZED, "handler is not initialised");
  if (!messages || num_messages == 0) return make_error(XLLM_INVALID_ARGUMENT, "no messages");
  std::lock_guard<std::mutex> lk(h->mu);
  Gil g;
  // a list of {"role", "content"} dictionaries goes through the chat template of the model
  PyObject* msgs = PyList_New(Py_ssize_t(num_messages));
  for (size_t i = 0; i < num_messages; ++i)
    PyList_SetItem(msgs, Py_ssize_t(i), Py_BuildValue("{s:s,s:s}", "role", messages[i].role ? messages[i].role : "user", "content",
                                                      messages[i].content ? messages[i].content : ""));
  PyObject* wrapped = PyList_New(1);      // generate() takes a list of prompts; one prompt = one list of messages
  PyList_SetItem(wrapped, 0, msgs);
  XLLM_Response* r = run_generate(h, wrapped, timeout_ms, params);
  Py_DECREF(wrapped);
  return r;
}

void xllm_llm_free_response(XLLM_Response* r) {
  if (!r) return;
  for (size_t i = 0; i < r->num_choices; ++i) {
    std::free(r->choices[i].text);
    std::free(r->choices[i].token_ids);
    std::free(r->choices[i].token_logprobs);
    std::free(r->choices[i].finish_reason);
  }
  std::free(r->choices);
  std::free(r->error);
  std::free(r->id);
  std::free(r);
}

const char* xllm_llm_last_error(XLLM_LLM_Handler* h) { return h ? h->error.c_str() : ""; }

}  // extern "C"
