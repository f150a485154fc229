/*
 * vllm_cpp_b200 stable C interface.
 *
 * Handle based, never throws, never exits: every entry point returns a vllm_status and leaves
 * a message for vllm_last_error() (per thread) when it fails. Strings handed to the caller
 * are released with vllm_string_free / vllm_completion_free; strings handed in are copied.
 * The 19 symbols, the struct layouts (field order, widths, the int32 flags) and the defaults
 * are those of the reference project's include/vllm.h at ABI version 5, so a program compiled
 * against that header loads this library unchanged. What the multi-GPU engine needs on top
 * (tensor-parallel size, expert parallelism, device) comes through vllm_engine_load_ex and its
 * size-prefixed vllm_engine_options, or through the environment (VLLM_TENSOR_PARALLEL_SIZE,
 * VLLM_ENABLE_EXPERT_PARALLEL, VLLM_DEVICE) for callers that only know vllm_engine_load.
 *
 * The engine behind the handle runs in an embedded Python interpreter (one per process);
 * calls may come from any thread.
 */
#ifndef VLLM_CPP_B200_VLLM_H
#define VLLM_CPP_B200_VLLM_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define VLLM_API __declspec(dllexport)
#else
#define VLLM_API __attribute__((visibility("default")))
#endif

#define VLLM_ABI_VERSION 5

typedef enum vllm_status {
  VLLM_OK = 0,
  VLLM_ERR_INVALID_ARGUMENT = 1,
  VLLM_ERR_MODEL_LOAD = 2,
  VLLM_ERR_RUNTIME = 3,
  VLLM_ERR_UNKNOWN = 4
} vllm_status;

typedef struct vllm_engine vllm_engine;    /* opaque */
typedef struct vllm_request vllm_request;  /* opaque */

typedef struct vllm_model_params {
  const char* model_path;             /* model directory or .gguf file (required) */
  const char* tokenizer_config_path;  /* NULL: look beside the model */
  int32_t block_size;                 /* <= 0: 32 */
  int32_t num_blocks;                 /* <= 0: 256 */
  int32_t max_model_len;              /* <= 0: from the model config */
  int32_t max_num_seqs;               /* <= 0: 8 */
  const char* tool_parser;            /* NULL or "": detect from the chat template, else hermes */
  const char* reasoning_parser;       /* NULL: detect; "none": off */
} vllm_model_params;

/* Options beyond vllm_model_params. struct_size = sizeof(vllm_engine_options) as the caller
 * compiled it: the library reads no field that lies beyond it, so the struct can grow. */
typedef struct vllm_engine_options {
  size_t struct_size;
  int32_t tensor_parallel_size;       /* <= 0: 1 */
  int32_t enable_expert_parallel;     /* 0 / 1 */
  const char* device;                 /* NULL: "cuda" */
} vllm_engine_options;

typedef struct vllm_sampling_params {
  float temperature;
  float top_p;
  int32_t top_k;                      /* 0: off */
  float min_p;
  int32_t max_tokens;
  uint64_t seed;
  int32_t has_seed;                   /* 0: unseeded */
  float presence_penalty;
  float frequency_penalty;
  float repetition_penalty;           /* must be > 0: a zeroed struct is invalid */
  int32_t min_tokens;
  int32_t ignore_eos;                 /* 0 / 1 */
  const char* const* stop;
  int32_t n_stop;
  /* at most one structured-output constraint */
  const char* structured_json;
  const char* structured_regex;
  const char* const* structured_choice;
  int32_t n_structured_choice;
  const char* structured_grammar;
  int32_t structured_json_object;     /* 0 / 1 */
} vllm_sampling_params;

typedef struct vllm_completion {
  char* text;                 /* caller frees with vllm_completion_free */
  const char* finish_reason;  /* static string: "stop", "length", "abort" */
  int32_t prompt_tokens;
  int32_t completion_tokens;
} vllm_completion;

/* delta: UTF-8 text produced since the last call ("" allowed); finished: last call.
 * Return false to stop the generation (the call still returns VLLM_OK). */
typedef bool (*vllm_token_callback)(const char* delta, bool finished, void* user);

VLLM_API vllm_model_params vllm_model_params_default(void);
VLLM_API vllm_sampling_params vllm_sampling_params_default(void);

VLLM_API vllm_status vllm_engine_load(const vllm_model_params* params, vllm_engine** out);
/* Not in the reference: vllm_engine_load plus options (NULL options = vllm_engine_load). */
VLLM_API vllm_status vllm_engine_load_ex(const vllm_model_params* params,
                                         const vllm_engine_options* options, vllm_engine** out);
VLLM_API void vllm_engine_free(vllm_engine* engine);   /* NULL is a no-op */

VLLM_API vllm_status vllm_complete(vllm_engine* engine, const char* prompt,
                                   const vllm_sampling_params* params, vllm_completion* out);
VLLM_API vllm_status vllm_complete_stream(vllm_engine* engine, const char* prompt,
                                          const vllm_sampling_params* params,
                                          vllm_token_callback cb, void* user);

/* Non-blocking requests: deltas arrive on a thread the library owns. */
VLLM_API vllm_status vllm_request_submit(vllm_engine* engine, const char* prompt,
                                         const vllm_sampling_params* params,
                                         vllm_token_callback cb, void* user, vllm_request** out);
VLLM_API vllm_status vllm_request_cancel(vllm_request* request); /* idempotent */
VLLM_API vllm_status vllm_request_wait(vllm_request* request);   /* blocks until finished */
VLLM_API bool vllm_request_done(const vllm_request* request);
VLLM_API const char* vllm_request_error(const vllm_request* request);   /* NULL: none */
VLLM_API void vllm_request_free(vllm_request* request);          /* joins the delivery thread */

/* OpenAI chat-completions request JSON in, response JSON out (chat template, tools,
 * tool_choice and the tool / reasoning parsers are applied by the engine). */
VLLM_API vllm_status vllm_chat(vllm_engine* engine, const char* request_json, char** out_json);
/* Same with one chat.completion.chunk JSON per callback. */
VLLM_API vllm_status vllm_chat_stream(vllm_engine* engine, const char* request_json,
                                      vllm_token_callback cb, void* user);

VLLM_API void vllm_string_free(char* s);
VLLM_API void vllm_completion_free(vllm_completion* c);

VLLM_API const char* vllm_last_error(void);   /* thread-local; "" when none */
VLLM_API const char* vllm_version(void);
VLLM_API int32_t vllm_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif
