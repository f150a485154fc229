// Model runner of the native runtime: SchedulerOutput -> packed step buffer (InputBatch::prepare,
// one pinned-host -> device copy) -> DenseModel::forward -> sampler pipeline -> sampled ids.
// The same ModelRunnerBase the engine core drives; no interpreter in the loop.
//
// Reference: src/vllm/v1/worker/gpu/runner.cpp:669-880 (execute_model), :1051 (sample_tokens),
// src/vllm/v1/sample/sampler.cpp (pipeline order).
#pragma once
#include <map>
#include <memory>
#include <optional>

#include "core/engine_core.h"
#include "runtime/dense_model.h"
#include "worker/input_batch.h"

namespace b200::rt {

class NativeRunner : public ModelRunnerBase {
 public:
  NativeRunner(std::unique_ptr<DenseModel> model, int block_size, int num_blocks, int max_num_seqs,
               int max_num_batched_tokens, int max_model_len);
  void execute_model(const SchedulerOutput& so) override;
  ModelRunnerOutput sample_tokens(const GrammarOutput* grammar) override;
  KVCacheConfig kv_cache_config() const override;
  void set_eos(const std::string& req_id, int eos) { eos_[req_id] = eos; }
  void forget(const std::string& req_id) { eos_.erase(req_id); }
  DenseModel& model() { return *model_; }
  int64_t h2d_bytes = 0, d2h_bytes = 0;

 private:
  template <class T> T* dev(size_t off) const { return reinterpret_cast<T*>(dev_base_ + off); }
  template <class T> T* host(size_t off) const { return reinterpret_cast<T*>(host_buf_.as<uint8_t>() + off); }
  void sample_host(const float* logits, const GrammarOutput* grammar, std::vector<int64_t>& ids);
  void sample_device(float* logits, const GrammarOutput* grammar, std::vector<int64_t>& ids);
  void check_kernel_status();
  std::unique_ptr<DenseModel> model_;
  Device dev_;
  int block_size_, num_blocks_, max_num_seqs_, max_tokens_, max_model_len_, max_blocks_;
  StepLayout layout_;
  InputBatch batch_;
  Buffer host_buf_, dev_buf_, sampled_dev_, sampled_host_, scratch_dev_, probs_dev_, status_host_;
  uint8_t* dev_base_ = nullptr;
  std::optional<StepInfo> info_;
  float* logits_ = nullptr;
  std::map<std::string, int32_t> eos_;
};

}  // namespace b200::rt
