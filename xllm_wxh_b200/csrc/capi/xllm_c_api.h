/* C interface of the serving engine (libxllm.so): create an engine, run completions / chat completions, free the results.
 *
 * Same entry-point names and call sequence as the reference's C API (xllm/c_api/llm.h:37-221: create -> initialize ->
 * completions / chat_completions -> free_response -> destroy); the option and response structures are this library's own
 * (plain C, no C++ types).  The engine itself is the Python / C++ / CUDA runtime of this package: the library embeds a
 * CPython interpreter when the host program has none, or attaches to the running one.
 *
 * Thread safety: calls on one handler are serialised inside the library.  All returned pointers stay valid until
 * xllm_llm_free_response() / xllm_llm_destroy(). */
#ifndef XLLM_C_API_H_
#define XLLM_C_API_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XLLM_CAPI_EXPORT __attribute__((visibility("default")))

typedef struct XLLM_LLM_Handler XLLM_LLM_Handler;

typedef enum XLLM_StatusCode {
  XLLM_OK = 0,
  XLLM_NOT_INITIALIZED = 1,
  XLLM_INVALID_ARGUMENT = 2,
  XLLM_INTERNAL_ERROR = 3,
  XLLM_TIMEOUT = 4
} XLLM_StatusCode;

typedef struct XLLM_InitLLMOptions {
  bool enable_prefix_cache;
  bool enable_chunked_prefill;
  bool enable_schedule_overlap;
  bool enable_graph;
  int32_t block_size;
  int32_t max_tokens_per_batch;
  int32_t max_seqs_per_batch;
  int32_t max_tokens_per_chunk_for_prefill;
  int32_t num_kv_blocks;            /* 0: sized from free device memory */
  double max_memory_utilization;
  int32_t dp_size;
  int32_t ep_size;
  int32_t num_speculative_tokens;
  const char* draft_model;          /* may be NULL */
  const char* dtype;                /* "auto" | "bfloat16" | "float32" ...; may be NULL */
} XLLM_InitLLMOptions;

typedef struct XLLM_RequestParams {
  int32_t max_tokens;
  int32_t n;
  float temperature;
  float top_p;
  int32_t top_k;
  float repetition_penalty;
  float frequency_penalty;
  float presence_penalty;
  bool ignore_eos;
  bool logprobs;
  int32_t top_logprobs;
  int64_t seed;                     /* < 0: none */
} XLLM_RequestParams;

typedef struct XLLM_ChatMessage {
  const char* role;
  const char* content;
} XLLM_ChatMessage;

typedef struct XLLM_Usage {
  int32_t prompt_tokens;
  int32_t completion_tokens;
  int32_t total_tokens;
} XLLM_Usage;

typedef struct XLLM_Choice {
  int32_t index;
  char* text;
  int32_t* token_ids;
  size_t num_token_ids;
  float* token_logprobs;            /* NULL unless logprobs were requested */
  char* finish_reason;
} XLLM_Choice;

typedef struct XLLM_Response {
  XLLM_StatusCode status_code;
  char* error;                      /* NULL when status_code == XLLM_OK */
  char* id;
  XLLM_Choice* choices;
  size_t num_choices;
  XLLM_Usage usage;
} XLLM_Response;

XLLM_CAPI_EXPORT XLLM_LLM_Handler* xllm_llm_create(void);
XLLM_CAPI_EXPORT void xllm_llm_destroy(XLLM_LLM_Handler* handler);
XLLM_CAPI_EXPORT void xllm_llm_init_options_default(XLLM_InitLLMOptions* options);
/* `model_path`: a HF model directory or "preset:<name>"; `devices`: "cuda:0", "cuda:0,cuda:1", "cpu" ... */
XLLM_CAPI_EXPORT bool xllm_llm_initialize(XLLM_LLM_Handler* handler, const char* model_path, const char* devices,
                                          const XLLM_InitLLMOptions* options);
XLLM_CAPI_EXPORT void xllm_llm_request_params_default(XLLM_RequestParams* params);
XLLM_CAPI_EXPORT XLLM_Response* xllm_llm_completions(XLLM_LLM_Handler* handler, const char* model_id, const char* prompt,
                                                     uint32_t timeout_ms, const XLLM_RequestParams* params);
XLLM_CAPI_EXPORT XLLM_Response* xllm_llm_chat_completions(XLLM_LLM_Handler* handler, const char* model_id,
                                                          const XLLM_ChatMessage* messages, size_t num_messages,
                                                          uint32_t timeout_ms, const XLLM_RequestParams* params);
XLLM_CAPI_EXPORT void xllm_llm_free_response(XLLM_Response* resp);
/* Last error of the handler (empty string when none); valid until the next call on the handler. */
XLLM_CAPI_EXPORT const char* xllm_llm_last_error(XLLM_LLM_Handler* handler);

#ifdef __cplusplus
}
#endif
#endif /* XLLM_C_API_H_ */
