// The native engine: tokenizer + detokenizer, scheduler, engine core, native model runner —
// assembled and driven from C++, so a process that serves through the C interface holds no
// interpreter. Surface of an LLMEngine: add_request / abort / step / has_unfinished.
//
// Reference: LoadedEngine (src/vllm/entrypoints/model_loader.cpp:273-366, :434-504) and
// LLMEngine (src/vllm/v1/engine/llm_engine.cpp:22-83).
#pragma once
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <vector>

#include "core/engine_core.h"
#include "runtime/native_runner.h"
#include "structured/manager.h"
#include "tokenizer/tokenizer.h"

namespace b200::rt {

struct EngineOptions {
  std::string model_path;
  std::string tokenizer_path;       // empty: beside the model
  std::string device = "cuda";
  int block_size = 32;
  int num_blocks = 0;               // 0: from gpu_memory_utilization (CPU: from max_num_seqs)
  int max_model_len = 0;            // 0: from the model config
  int max_num_seqs = 8;
  int max_num_batched_tokens = 0;   // 0: 2048
  double gpu_memory_utilization = 0.90;
  bool enable_prefix_caching = true;
};

struct RequestDelta {
  std::string request_id;
  std::vector<int32_t> new_token_ids;
  std::string delta_text;           // text that became final with this step
  bool finished = false;
  std::string finish_reason;        // "stop" | "length" | "abort" when finished
  int prompt_tokens = 0, completion_tokens = 0;
};

class NativeLLM {
 public:
  static std::unique_ptr<NativeLLM> load(const EngineOptions& opt);   // throws std::runtime_error
  ~NativeLLM();
  // Tokenises `prompt` (or takes `prompt_ids`), validates the parameters, queues the request.
  std::string add_request(const std::string& prompt, SamplingParams params, const std::string& request_id = "");
  std::string add_request_ids(std::vector<int32_t> prompt_ids, SamplingParams params,
                              const std::string& request_id = "");
  void abort(const std::string& request_id);
  bool has_unfinished() const;
  // One engine step: the requests that produced tokens, with the text those tokens finalised.
  std::vector<RequestDelta> step();
  const tok::Tokenizer* tokenizer() const { return tokenizer_.get(); }
  const DenseConfig& config() const { return cfg_; }
  int max_model_len() const { return max_model_len_; }
  NativeRunner& runner() { return *runner_; }

 private:
  NativeLLM() = default;
  struct Live {
    std::vector<int32_t> prompt_ids;
    std::unique_ptr<tok::IncrementalDetokenizer> detok;
    int completion_tokens = 0;
  };
  DenseConfig cfg_;
  std::unique_ptr<tok::Tokenizer> tokenizer_;
  std::unique_ptr<so::StructuredOutputManager> structured_;
  std::unique_ptr<NativeRunner> runner_;
  std::unique_ptr<Executor> executor_;
  std::unique_ptr<EngineCore> core_;
  std::map<std::string, Live> live_;
  int max_model_len_ = 0;
  uint64_t counter_ = 0;
};

}  // namespace b200::rt
