#include "core/types.h"

#include <algorithm>
#include <cmath>

namespace b200 {

void SamplingParams::verify() const {
  auto bad = [](const std::string& m) { throw std::invalid_argument(m); };
  if (n < 1) bad("n must be at least 1, got " + std::to_string(n));
  if (!(presence_penalty >= -2.0 && presence_penalty <= 2.0)) bad("presence_penalty must be in [-2, 2]");
  if (!(frequency_penalty >= -2.0 && frequency_penalty <= 2.0)) bad("frequency_penalty must be in [-2, 2]");
  if (!(repetition_penalty > 0.0 && repetition_penalty <= 2.0)) bad("repetition_penalty must be in (0, 2]");
  if (temperature < 0.0) bad("temperature must be non-negative");
  if (!(top_p > 0.0 && top_p <= 1.0)) bad("top_p must be in (0, 1]");
  if (top_k < -1) bad("top_k must be -1 (disable), 0 (disable) or at least 1");
  if (!(min_p >= 0.0 && min_p <= 1.0)) bad("min_p must be in [0, 1]");
  if (max_tokens && *max_tokens < 1) bad("max_tokens must be at least 1");
  if (min_tokens < 0) bad("min_tokens must be greater than or equal to 0");
  if (max_tokens && min_tokens > *max_tokens) bad("min_tokens must be less than or equal to max_tokens");
  if (logprobs && *logprobs < 0) bad("logprobs must be non-negative");
  if (prompt_logprobs && *prompt_logprobs < 0) bad("prompt_logprobs must be non-negative");
  for (auto& s : stop)
    if (s.empty()) bad("stop cannot contain an empty string");
  if (!stop.empty() && !detokenize) bad("stop strings are only supported when detokenize is True");
  if (structured_outputs && structured_outputs->count() > 1)
    bad("You can only use one kind of structured outputs constraint");
}

void SamplingParams::post_init() {
  if (top_k == -1) top_k = 0;
  if (temperature > 0.0 && temperature < 1e-2) temperature = 1e-2;
  if (temperature < kSamplingEps) {
    // greedy: the filters are irrelevant
    top_p = 1.0;
    top_k = 0;
    min_p = 0.0;
  }
  std::sort(stop_token_ids.begin(), stop_token_ids.end());
  stop_token_ids.erase(std::unique(stop_token_ids.begin(), stop_token_ids.end()), stop_token_ids.end());
  if (!stop.empty() && !include_stop_str_in_output) {
    // hold back enough characters to strip a stop string once matched (used by the detokenizer)
  }
}

Request::Request(const EngineCoreRequest& r)
    : request_id(r.request_id), prompt_token_ids(r.prompt_token_ids),
      sampling_params(r.sampling_params), eos_token_id(r.eos_token_id),
      arrival_time(r.arrival_time), priority(r.priority), cache_salt(r.cache_salt) {
  all_token_ids = prompt_token_ids;
  max_tokens = sampling_params.max_tokens ? *sampling_params.max_tokens : (1 << 30);
  use_structured_output = sampling_params.structured_outputs && sampling_params.structured_outputs->any();
  if (use_structured_output) status = RequestStatus::kWaitingForFsm;
}

}  // namespace b200
