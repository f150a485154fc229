// Unified token-budget scheduler (vLLM V1 semantics): no prefill/decode phases, every step
// hands each running request as many tokens as the budget allows, admits waiting requests
// (prefix-cache lookup, chunked prefill) and preempts from the tail (or the lowest priority)
// when the KV pool runs out.
//
// Behavioural parity: src/vllm/v1/core/sched/scheduler.cpp:130-504 (schedule), :546-719
// (update_from_output), :115-128 (preempt), sched/utils.cpp (check_stop),
// sched/async_scheduler.cpp, sched/request_queue.cpp.
#pragma once
#include <deque>
#include <functional>
#include <list>
#include <memory>
#include <optional>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "core/kv_cache.h"
#include "core/types.h"

namespace b200 {

// ------------------------------------------------------------------------ request queue
class RequestQueue {
 public:
  explicit RequestQueue(bool priority) : priority_(priority) {}
  void add(const RequestPtr& r);
  RequestPtr pop();                       // throws when empty
  RequestPtr peek() const;
  void prepend(const RequestPtr& r);      // FCFS: front; priority: same as add
  void prepend_all(const std::vector<RequestPtr>& rs);  // keeps the given order at the front
  bool remove(const RequestPtr& r);
  size_t size() const { return q_.size(); }
  bool empty() const { return q_.empty(); }
  std::vector<RequestPtr> snapshot() const { return {q_.begin(), q_.end()}; }

 private:
  static bool before(const RequestPtr& a, const RequestPtr& b) {
    if (a->priority != b->priority) return a->priority < b->priority;
    return a->arrival_time < b->arrival_time;
  }
  bool priority_;
  std::deque<RequestPtr> q_;  // priority mode: kept sorted (stable)
};

// ------------------------------------------------------------- structured-output hook
class StructuredOutputHook {
 public:
  virtual ~StructuredOutputHook() = default;
  // Compile the grammar of a request. Returns false if it is not ready yet (async compile).
  virtual bool grammar_ready(Request& req) = 0;
  // Feed sampled tokens to the request's matcher; returns false if a token was rejected.
  virtual bool accept_tokens(Request& req, const std::vector<int32_t>& tokens) = 0;
  virtual void rollback(Request& req, int num_tokens) = 0;
  // Fill one bitmask row per structured request scheduled this step.
  virtual GrammarOutput grammar_bitmask(const std::vector<RequestPtr>& reqs,
                                        const std::map<std::string, std::vector<int32_t>>& spec) = 0;
  virtual void release(Request& req) = 0;
  virtual bool is_terminated(Request& req) { return false; }
};

// ----------------------------------------------------------------- external KV connector
class KVConnectorHook {
 public:
  virtual ~KVConnectorHook() = default;
  // Tokens beyond `num_computed_tokens` available from the external store.
  // nullopt = "not known yet, retry later"; second = load is asynchronous.
  virtual std::optional<std::pair<int, bool>> get_num_new_matched_tokens(
      const Request& req, int num_computed_tokens) = 0;
  virtual void update_state_after_alloc(const Request& req,
                                        const std::vector<std::vector<int32_t>>& block_ids,
                                        int num_external_tokens) = 0;
  virtual std::shared_ptr<void> build_connector_meta(const SchedulerOutput& out) = 0;
  // Returns true if the blocks must stay alive until an asynchronous save finishes.
  virtual bool request_finished(const Request& req,
                                const std::vector<std::vector<int32_t>>& block_ids) = 0;
};

// ------------------------------------------------------------------------------ scheduler
class Scheduler {
 public:
  Scheduler(const SchedulerConfig& cfg, const KVCacheConfig& kv_cfg,
            StructuredOutputHook* so = nullptr, KVConnectorHook* connector = nullptr);
  virtual ~Scheduler() = default;

  void add_request(const RequestPtr& req);
  virtual SchedulerOutput schedule();
  // Returns one EngineCoreOutputs (single client).
  virtual EngineCoreOutputs update_from_output(const SchedulerOutput& so,
                                               const ModelRunnerOutput& mro);
  void finish_requests(const std::vector<std::string>& ids, RequestStatus status);
  void update_draft_token_ids(const DraftTokenIds& drafts);
  GrammarOutput get_grammar_bitmask(const SchedulerOutput& so);

  int get_num_unfinished_requests() const { return (int)(waiting_.size() + running_.size()); }
  bool has_unfinished_requests() const { return get_num_unfinished_requests() > 0; }
  bool has_finished_requests() const { return !finished_req_ids_.empty(); }
  bool has_requests() const { return has_unfinished_requests() || has_finished_requests(); }
  int num_running() const { return (int)running_.size(); }
  int num_waiting() const { return (int)waiting_.size(); }
  int num_delayed_free() const { return (int)delayed_free_.size(); }
  bool reset_prefix_cache() { return kv_->reset_prefix_cache(); }
  SchedulerStats make_stats();
  KVCacheManager& kv_cache_manager() { return *kv_; }
  const SchedulerConfig& config() const { return cfg_; }
  RequestPtr get_request(const std::string& id) const;
  std::vector<std::string> all_request_ids() const {
    std::vector<std::string> ids;
    for (auto& kv : requests_) ids.push_back(kv.first);
    return ids;
  }
  const std::vector<RequestPtr>& running() const { return running_; }
  int64_t prefix_cache_queries() const { return pc_queries_; }
  int64_t prefix_cache_hits() const { return pc_hits_; }

 protected:
  virtual void update_after_schedule(const SchedulerOutput& so);
  // Async scheduling: called for each request that produced tokens this step.
  virtual void update_request_with_output(Request& req, std::vector<int32_t>& new_tokens, bool& stopped);
  void preempt_request(const RequestPtr& req);
  void free_request(const RequestPtr& req);
  bool check_stop(Request& req);
  bool promote_after_remote_kv(Request& req);

  SchedulerConfig cfg_;
  KVCacheConfig kv_cfg_;
  std::unique_ptr<KVCacheManager> kv_;
  StructuredOutputHook* so_;
  KVConnectorHook* connector_;
  std::unordered_map<std::string, RequestPtr> requests_;
  RequestQueue waiting_;
  std::vector<RequestPtr> running_;
  std::set<std::string> finished_req_ids_;
  // external KV connector: loads the runner has reported complete but the waiting loop has not
  // consumed yet, and finished requests whose blocks the connector is still sending
  std::set<std::string> finished_recving_;
  std::unordered_map<std::string, RequestPtr> delayed_free_;
  int num_preempted_since_stats_ = 0;
  int last_step_tokens_ = 0;
  int64_t pc_queries_ = 0, pc_hits_ = 0;
};

// Schedules step N+1 before the tokens of step N are known: every request with a sampled
// token in flight carries an output placeholder that is counted in its length.
class AsyncScheduler : public Scheduler {
 public:
  using Scheduler::Scheduler;

 protected:
  void update_after_schedule(const SchedulerOutput& so) override;
  void update_request_with_output(Request& req, std::vector<int32_t>& new_tokens,
                                  bool& stopped) override;
};

}  // namespace b200
