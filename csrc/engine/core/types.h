// Value types shared by the host engine: sampling parameters, the request state machine,
// scheduler input/output records and model-runner results.
//
// Behavioural parity targets in the reference: include/vllm/sampling_params.h:116-183,
// include/vllm/v1/request.h, include/vllm/v1/engine/types.h, include/vllm/v1/core/sched/output.h.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <optional>
#include <set>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace b200 {

constexpr double kSamplingEps = 1e-5;

enum class OutputKind : int { kCumulative = 0, kDelta = 1, kFinalOnly = 2 };
enum class SamplingType : int { kGreedy = 0, kRandom = 1, kRandomSeed = 2 };

struct StructuredOutputsParams {
  std::optional<std::string> json;
  std::optional<std::string> regex;
  std::optional<std::vector<std::string>> choice;
  std::optional<std::string> grammar;
  bool json_object = false;
  std::optional<std::string> structural_tag;  // lazy (triggered) grammar description, JSON
  bool any() const {
    return json || regex || choice || grammar || json_object || structural_tag;
  }
  int count() const {
    return (json ? 1 : 0) + (regex ? 1 : 0) + (choice ? 1 : 0) + (grammar ? 1 : 0) +
           (json_object ? 1 : 0) + (structural_tag ? 1 : 0);
  }
};

struct SamplingParams {
  int n = 1;
  double presence_penalty = 0.0;
  double frequency_penalty = 0.0;
  double repetition_penalty = 1.0;
  double temperature = 1.0;
  double top_p = 1.0;
  int top_k = 0;
  double min_p = 0.0;
  std::optional<uint64_t> seed;
  std::vector<std::string> stop;
  std::vector<int32_t> stop_token_ids;
  bool ignore_eos = false;
  std::optional<int> max_tokens = 16;
  int min_tokens = 0;
  std::optional<int> logprobs;
  std::optional<int> prompt_logprobs;
  bool detokenize = true;
  bool skip_special_tokens = true;
  bool spaces_between_special_tokens = true;
  bool include_stop_str_in_output = false;
  OutputKind output_kind = OutputKind::kCumulative;
  std::map<int32_t, float> logit_bias;
  std::vector<int32_t> allowed_token_ids;
  std::vector<std::vector<int32_t>> bad_words_token_ids;
  std::optional<StructuredOutputsParams> structured_outputs;

  SamplingType type() const {
    if (temperature < kSamplingEps) return SamplingType::kGreedy;
    return seed ? SamplingType::kRandomSeed : SamplingType::kRandom;
  }
  // Throws std::invalid_argument on an out-of-range field (same rules as vLLM).
  void verify() const;
  // Normalises: top_k -1 -> 0, greedy resets top_p/top_k/min_p, stop ids de-duplicated.
  void post_init();
  bool has_penalties() const {
    return presence_penalty != 0.0 || frequency_penalty != 0.0 || repetition_penalty != 1.0;
  }
};

enum class RequestStatus : int {
  kWaiting = 0,
  kWaitingForFsm,
  kWaitingForRemoteKvs,
  kRunning,
  kPreempted,
  // everything after kPreempted is finished
  kFinishedStopped,
  kFinishedLengthCapped,
  kFinishedAborted,
  kFinishedIgnored,
};
inline bool is_finished(RequestStatus s) { return (int)s > (int)RequestStatus::kPreempted; }

enum class FinishReason : int { kStop = 0, kLength = 1, kAbort = 2 };
inline const char* finish_reason_str(FinishReason r) {
  switch (r) {
    case FinishReason::kStop: return "stop";
    case FinishReason::kLength: return "length";
    default: return "abort";
  }
}
inline std::optional<FinishReason> finish_reason_of(RequestStatus s) {
  switch (s) {
    case RequestStatus::kFinishedStopped: return FinishReason::kStop;
    case RequestStatus::kFinishedLengthCapped: return FinishReason::kLength;
    case RequestStatus::kFinishedIgnored: return FinishReason::kLength;
    case RequestStatus::kFinishedAborted: return FinishReason::kAbort;
    default: return std::nullopt;
  }
}

using BlockHash = std::string;  // 32 raw bytes

// What the front end hands to the engine core.
struct EngineCoreRequest {
  std::string request_id;
  std::vector<int32_t> prompt_token_ids;
  SamplingParams sampling_params;
  std::optional<int32_t> eos_token_id;
  double arrival_time = 0.0;
  int priority = 0;
  std::optional<std::string> cache_salt;
};

// Stop reason: either a token id or a stop string.
struct StopReason {
  bool is_token = false;
  int32_t token = 0;
  std::string text;
};

struct Request {
  std::string request_id;
  std::vector<int32_t> prompt_token_ids;
  SamplingParams sampling_params;
  std::optional<int32_t> eos_token_id;
  double arrival_time = 0.0;
  int priority = 0;
  std::optional<std::string> cache_salt;

  RequestStatus status = RequestStatus::kWaiting;
  std::optional<StopReason> stop_reason;
  std::vector<int32_t> output_token_ids;
  std::vector<int32_t> all_token_ids;      // prompt + output
  std::vector<int32_t> spec_token_ids;     // draft tokens scheduled for verification
  int num_computed_tokens = 0;
  int num_cached_tokens = -1;              // prefix-cache hit length at first schedule
  int num_output_placeholders = 0;         // async scheduling: tokens in flight
  int num_preemptions = 0;
  int max_tokens = 16;
  bool use_structured_output = false;
  void* structured_state = nullptr;        // owned by the structured-output manager
  std::vector<BlockHash> block_hashes;     // chained hashes of the full blocks seen so far
  int num_nans_in_logits = 0;

  explicit Request(const EngineCoreRequest& r);
  int num_prompt_tokens() const { return (int)prompt_token_ids.size(); }
  int num_tokens() const { return (int)all_token_ids.size(); }
  int num_tokens_with_spec() const { return num_tokens() + (int)spec_token_ids.size(); }
  int num_output_tokens() const { return (int)output_token_ids.size(); }
  void append_output_token(int32_t t) {
    output_token_ids.push_back(t);
    all_token_ids.push_back(t);
  }
  bool finished() const { return is_finished(status); }
};
using RequestPtr = std::shared_ptr<Request>;

// ---------------------------------------------------------------------------------------
// Scheduler -> worker
// ---------------------------------------------------------------------------------------
struct NewRequestData {
  std::string req_id;
  std::vector<int32_t> prompt_token_ids;     // all tokens known so far (resumed requests
                                             // carry prompt + generated tokens)
  SamplingParams sampling_params;
  std::vector<std::vector<int32_t>> block_ids;  // per KV-cache group
  int num_computed_tokens = 0;
  int num_prompt_tokens = 0;
};

struct CachedRequestData {
  std::vector<std::string> req_ids;
  std::vector<uint8_t> resumed_from_preemption;
  std::vector<std::vector<int32_t>> new_token_ids;               // tokens sampled since last step
  std::vector<std::vector<std::vector<int32_t>>> new_block_ids;  // per request, per group
  std::vector<int> num_computed_tokens;
  std::vector<int> num_output_tokens;
  size_t size() const { return req_ids.size(); }
};

struct SchedulerOutput {
  std::vector<NewRequestData> scheduled_new_reqs;
  CachedRequestData scheduled_cached_reqs;
  std::vector<std::pair<std::string, int>> num_scheduled_tokens;  // in schedule order
  int total_num_scheduled_tokens = 0;
  std::map<std::string, std::vector<int32_t>> scheduled_spec_decode_tokens;
  std::vector<int> num_common_prefix_blocks;
  std::set<std::string> finished_req_ids;
  std::vector<std::string> structured_output_request_ids;
  std::vector<std::string> preempted_req_ids;
  std::shared_ptr<void> kv_connector_metadata;
  int tokens_for(const std::string& id) const {
    for (auto& p : num_scheduled_tokens)
      if (p.first == id) return p.second;
    return 0;
  }
};

struct GrammarOutput {
  std::vector<std::string> structured_output_request_ids;
  std::vector<int32_t> bitmask;  // [n, ceil(vocab/32)] row-major; bit set = token allowed
  int words_per_row = 0;
};

// ---------------------------------------------------------------------------------------
// Worker -> scheduler
// ---------------------------------------------------------------------------------------
struct LogprobsRow {
  std::vector<int32_t> token_ids;  // sampled token first, then top-k
  std::vector<float> logprobs;
  std::vector<int32_t> ranks;
};

struct ModelRunnerOutput {
  std::vector<std::string> req_ids;
  std::vector<std::vector<int32_t>> sampled_token_ids;  // per request; empty while prefilling
  std::vector<std::vector<LogprobsRow>> logprobs;       // optional, per request per token
  std::vector<int> num_nans_in_logits;
  std::set<std::string> finished_sending, finished_recving;
  // Speculative decoding on models with recurrent state: a rejected draft has advanced the state
  // past the tokens that were kept, so the runner restores the state it saved before the step and
  // asks for the kept tokens of the step (this many) to be computed again with the next one.
  std::map<std::string, int> num_recompute;
  bool empty() const { return req_ids.empty(); }
};

struct DraftTokenIds {
  std::vector<std::string> req_ids;
  std::vector<std::vector<int32_t>> draft_token_ids;
};

struct EngineCoreOutput {
  std::string request_id;
  std::vector<int32_t> new_token_ids;
  std::vector<LogprobsRow> new_logprobs;
  std::optional<FinishReason> finish_reason;
  std::optional<StopReason> stop_reason;
  int num_cached_tokens = 0;
  bool finished() const { return finish_reason.has_value(); }
};

struct SchedulerStats {
  int num_running_reqs = 0;
  int num_waiting_reqs = 0;
  double kv_cache_usage = 0.0;
  int64_t prefix_cache_queries = 0;
  int64_t prefix_cache_hits = 0;
  int num_preempted = 0;
  int step_scheduled_tokens = 0;
};

struct EngineCoreOutputs {
  std::vector<EngineCoreOutput> outputs;
  std::optional<SchedulerStats> scheduler_stats;
  std::set<std::string> finished_requests;
  bool engine_dead = false;
  std::string error;
};

struct SchedulerConfig {
  int max_num_batched_tokens = 2048;
  int max_num_seqs = 8;
  int max_model_len = 8192;
  bool enable_chunked_prefill = true;
  int long_prefill_token_threshold = 0;
  int max_num_partial_prefills = 1;
  std::string policy = "fcfs";  // fcfs | priority
  bool async_scheduling = false;
  int num_lookahead_tokens = 0;  // speculative decoding
  bool enable_prefix_caching = true;
  double watermark = 0.0;
  bool log_stats = true;
};

}  // namespace b200
