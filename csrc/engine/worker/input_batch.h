// Worker-side persistent batch state and per-step input preparation.
//
// The worker keeps, for every live request, its token ids, block ids per KV group and
// sampling state (InputBatch). Each step `prepare()` turns a SchedulerOutput into flat
// arrays written into ONE caller-provided (pinned) host buffer with a fixed layout, so a
// step costs a single host->device copy: token ids, positions, slot mapping, query start
// offsets, sequence lengths, block tables, logits row indices, the list of 128-row prefill
// tiles, and the per-request sampling scalars. Requests are ordered decode-first.
//
// Behavioural parity: src/vllm/v1/worker/gpu/input_batch.cpp, block_table.cpp,
// prepare_inputs.cpp:20-91, v1/attention/backends/utils.cpp (split_decodes_and_prefills,
// reorder_batch_to_split_decodes_and_prefills), gdn_attn.cpp (state slot bookkeeping).
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "core/types.h"

namespace b200 {

struct CachedRequestState {
  std::string req_id;
  std::vector<int32_t> token_ids;  // prompt + generated so far (as known to the worker)
  int num_prompt_tokens = 0;
  int num_computed_tokens = 0;
  std::vector<std::vector<int32_t>> block_ids;  // per KV group
  SamplingParams sampling_params;
  int state_slot = -1;   // recurrent-state slot (GDN / Mamba), stable for the request's life
  uint64_t sample_step = 0;
  int batch_row = -1;    // row in the last prepared batch (for device-resident sampled ids)
};

// Byte offsets of each array inside the packed step buffer.
struct StepLayout {
  int max_tokens = 0, max_reqs = 0, max_blocks = 0, num_groups = 1, max_tiles = 0;
  int max_logits = 0;         // max_reqs * (1 + max draft tokens per request)
  size_t input_ids = 0;       // int64 [max_tokens]
  size_t positions = 0;       // int64 [max_tokens]
  size_t slot_mapping = 0;    // int64 [num_groups][max_tokens]
  size_t query_start = 0;     // int32 [max_reqs + 1]
  size_t seq_lens = 0;        // int32 [max_reqs]
  size_t block_table = 0;     // int32 [num_groups][max_reqs][max_blocks]
  size_t logits_indices = 0;  // int32 [max_logits]
  size_t tile_req = 0;        // int32 [max_tiles]   (request index relative to first prefill)
  size_t tile_q0 = 0;         // int32 [max_tiles]
  size_t prefill_q_start = 0; // int32 [max_reqs + 1] (token offsets relative to first prefill token)
  size_t state_slots = 0;     // int32 [max_reqs]
  size_t temperature = 0;     // f32 [max_reqs]
  size_t top_p = 0;           // f32 [max_reqs]
  size_t min_p = 0;           // f32 [max_reqs]
  size_t top_k = 0;           // int32 [max_reqs]
  size_t seeds = 0;           // u64 [max_reqs]
  size_t steps = 0;           // u64 [max_reqs]
  size_t rep_pen = 0, freq_pen = 0, pres_pen = 0;  // f32 [max_reqs]
  size_t splice_dst = 0;      // int32 [max_reqs] async: position in input_ids to overwrite
  size_t splice_src = 0;      // int32 [max_reqs] async: row of the previous batch's sampled ids
  size_t sample_rows = 0;     // int32 [max_reqs] batch row of each logits row (rows that sample)
  size_t total_bytes = 0;
  // max_spec: draft tokens a request may verify per step (each adds a logits row).
  static StepLayout make(int max_tokens, int max_reqs, int max_blocks, int num_groups,
                         int max_spec = 0);
};

struct StepInfo {
  int num_reqs = 0, num_tokens = 0;
  int num_decodes = 0, num_decode_tokens = 0;
  int num_prefills = 0, num_prefill_tokens = 0;
  int num_tiles = 0;
  int max_query_len = 0, max_seq_len = 0;
  int num_logits = 0;
  int num_splice = 0;
  bool all_greedy = true, any_penalties = false, any_top_k_top_p = false, any_min_p = false;
  bool any_logprobs = false;
  // a sampling row has a logit bias, an allow / ban list or a min_tokens ban still in force
  bool any_logit_edits = false;
  std::vector<std::string> req_ids;        // batch order
  std::vector<int> num_scheduled;          // per request
  std::vector<uint8_t> produces_token;     // request finishes its known tokens this step
  std::vector<int> max_logprobs;           // per request (-1 = none)
  std::vector<int> num_draft;              // per request: draft tokens verified this step
  std::vector<int> logits_row0;            // per request: its first logits row (-1 = none)
};

class InputBatch {
 public:
  InputBatch(int max_num_reqs, int max_model_len, int max_num_tokens,
             const std::vector<int>& block_sizes);
  // Applies finished / preempted / new / cached request updates.
  void update_states(const SchedulerOutput& so);
  // Fills the packed buffer for this step. `async_mode`: token ids of requests whose last
  // sampled token is still on the device are left as 0 and listed in splice_dst/src.
  StepInfo prepare(const SchedulerOutput& so, const StepLayout& layout, uint8_t* buf,
                   bool async_mode = false);
  // Sync mode: record sampled tokens (the scheduler also sends them back as new_token_ids).
  void append_sampled(const std::string& req_id, const std::vector<int32_t>& toks);
  const CachedRequestState* get(const std::string& id) const;
  // Prompt-lookup drafting (reference: include/vllm/v1/spec_decode/ngram_proposer.h): the longest
  // suffix of between min_n and max_n tokens that occurred earlier in the request (latest
  // occurrence first); returns up to k tokens that followed it. Empty if none.
  std::vector<int32_t> propose_ngram(const std::string& id, int min_n, int max_n, int k) const;
  // True if the request samples greedily with nothing that edits its logits (the case drafts are
  // verified by plain argmax comparison).
  bool plain_greedy(const std::string& id) const;
  size_t num_requests() const { return reqs_.size(); }
  int max_num_reqs() const { return max_num_reqs_; }
  // Penalty triples (row, token, output count) for the rows of the last prepared batch.
  void build_penalty_entries(const StepInfo& info, std::vector<int32_t>& rows,
                             std::vector<int32_t>& toks, std::vector<int32_t>& out_cnt) const;
  // Sparse logit edits: logit_bias (mode 0) and banned tokens (min_tokens stop ids,
  // bad words, mode 1) for the rows of the last prepared batch.
  void build_logit_edits(const StepInfo& info, std::vector<int32_t>& bias_rows,
                         std::vector<int32_t>& bias_toks, std::vector<float>& bias_vals,
                         std::vector<int32_t>& ban_rows, std::vector<int32_t>& ban_toks,
                         const std::map<std::string, int32_t>& eos_of) const;

 private:
  int alloc_state_slot();
  int max_num_reqs_, max_model_len_, max_num_tokens_;
  std::vector<int> block_sizes_;
  std::unordered_map<std::string, CachedRequestState> reqs_;
  std::vector<int> free_state_slots_;
  std::unordered_map<std::string, int> last_rows_;  // req id -> row in the previous batch
};

}  // namespace b200
