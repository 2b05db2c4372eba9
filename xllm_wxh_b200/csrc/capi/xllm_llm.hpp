// C++ face of the serving engine: class xllm::LLM with Initialize / Completions / ChatCompletions, the call sequence of
// the reference's C++ API (xllm/cc_api/llm.h:33-96: construct, Initialize once, then any number of Completions /
// ChatCompletions).  Header-only over the C interface of libxllm.so (xllm_c_api.h): link with -lxllm.  Results are
// plain C++ values (strings and vectors); the C response they were copied from is freed before the call returns.
#ifndef XLLM_LLM_HPP_
#define XLLM_LLM_HPP_

#include <cstdint>
#include <string>
#include <vector>

#include "xllm_c_api.h"

namespace xllm {

struct ChatMessage {
  std::string role;      // "system" | "user" | "assistant"
  std::string content;
};

struct Choice {
  int32_t index = 0;
  std::string text;
  std::vector<int32_t> token_ids;
  std::vector<float> token_logprobs;     // empty unless log-probabilities were requested
  std::string finish_reason;
};

struct Response {
  XLLM_StatusCode status_code = XLLM_NOT_INITIALIZED;
  std::string error;                     // empty when status_code == XLLM_OK
  std::string id;
  std::vector<Choice> choices;
  XLLM_Usage usage{0, 0, 0};
  bool ok() const { return status_code == XLLM_OK; }
};

// Option and request structures are the C ones; these return them filled with the library's defaults.
inline XLLM_InitLLMOptions DefaultInitOptions() {
  XLLM_InitLLMOptions o;
  xllm_llm_init_options_default(&o);
  return o;
}
inline XLLM_RequestParams DefaultRequestParams() {
  XLLM_RequestParams p;
  xllm_llm_request_params_default(&p);
  return p;
}

class LLM {
 public:
  LLM() : handler_(xllm_llm_create()) {}
  ~LLM() {
    if (handler_ != nullptr) xllm_llm_destroy(handler_);
  }
  LLM(const LLM&) = delete;
  LLM& operator=(const LLM&) = delete;
  LLM(LLM&&) = delete;
  LLM& operator=(LLM&&) = delete;

  // Load the model and start the engine.  `model_path`: a Hugging Face model directory or "preset:<name>"; `devices`:
  // "cuda:0", "cuda:0,cuda:1", "cpu".  Call once, before the first request.
  bool Initialize(const std::string& model_path, const std::string& devices, const XLLM_InitLLMOptions& options = DefaultInitOptions()) {
    return handler_ != nullptr && xllm_llm_initialize(handler_, model_path.c_str(), devices.c_str(), &options);
  }

  Response Completions(const std::string& model_id, const std::string& prompt, uint32_t timeout_ms,
                       const XLLM_RequestParams& params = DefaultRequestParams()) {
    if (handler_ == nullptr) return Response{};
    return Take(xllm_llm_completions(handler_, model_id.c_str(), prompt.c_str(), timeout_ms, &params));
  }

  Response ChatCompletions(const std::string& model_id, const std::vector<ChatMessage>& messages, uint32_t timeout_ms,
                           const XLLM_RequestParams& params = DefaultRequestParams()) {
    if (handler_ == nullptr) return Response{};
    std::vector<XLLM_ChatMessage> raw;
    raw.reserve(messages.size());
    for (const ChatMessage& m : messages) raw.push_back(XLLM_ChatMessage{m.role.c_str(), m.content.c_str()});
    return Take(xllm_llm_chat_completions(handler_, model_id.c_str(), raw.data(), raw.size(), timeout_ms, &params));
  }

  std::string LastError() const { return handler_ != nullptr ? std::string(xllm_llm_last_error(handler_)) : std::string("no handler"); }

 private:
  static Response Take(XLLM_Response* r) {
    Response out;
    if (r == nullptr) {
      out.status_code = XLLM_INTERNAL_ERROR;
      out.error = "no response";
      return out;
    }
    out.status_code = r->status_code;
    if (r->error != nullptr) out.error = r->error;
    if (r->id != nullptr) out.id = r->id;
    out.usage = r->usage;
    out.choices.resize(r->num_choices);
    for (size_t i = 0; i < r->num_choices; ++i) {
      const XLLM_Choice& c = r->choices[i];
      Choice& d = out.choices[i];
      d.index = c.index;
      if (c.text != nullptr) d.text = c.text;
      if (c.token_ids != nullptr) d.token_ids.assign(c.token_ids, c.token_ids + c.num_token_ids);
      if (c.token_logprobs != nullptr) d.token_logprobs.assign(c.token_logprobs, c.token_logprobs + c.num_token_ids);
      if (c.finish_reason != nullptr) d.finish_reason = c.finish_reason;
    }
    xllm_llm_free_response(r);
    return out;
  }

  XLLM_LLM_Handler* handler_ = nullptr;
};

}  // namespace xllm
#endif  // XLLM_LLM_HPP_
