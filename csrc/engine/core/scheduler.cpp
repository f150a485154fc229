#include "core/scheduler.h"

#include <algorithm>
#include <cassert>

namespace b200 {

// ------------------------------------------------------------------------ RequestQueue
void RequestQueue::add(const RequestPtr& r) {
  if (!priority_) {
    q_.push_back(r);
    return;
  }
  auto it = std::upper_bound(q_.begin(), q_.end(), r, before);
  q_.insert(it, r);
}
RequestPtr RequestQueue::pop() {
  if (q_.empty()) throw std::out_of_range("pop from an empty request queue");
  RequestPtr r = q_.front();
  q_.pop_front();
  return r;
}
RequestPtr RequestQueue::peek() const {
  if (q_.empty()) throw std::out_of_range("peek into an empty request queue");
  return q_.front();
}
void RequestQueue::prepend(const RequestPtr& r) {
  if (priority_) add(r);
  else q_.push_front(r);
}
void RequestQueue::prepend_all(const std::vector<RequestPtr>& rs) {
  if (priority_) {
    for (auto& r : rs) add(r);
  } else {
    for (auto it = rs.rbegin(); it != rs.rend(); ++it) q_.push_front(*it);
  }
}
bool RequestQueue::remove(const RequestPtr& r) {
  auto it = std::find(q_.begin(), q_.end(), r);
  if (it == q_.end()) return false;
  q_.erase(it);
  return true;
}

// --------------------------------------------------------------------------- Scheduler
Scheduler::Scheduler(const SchedulerConfig& cfg, const KVCacheConfig& kv_cfg,
                     StructuredOutputHook* so, KVConnectorHook* connector)
    : cfg_(cfg), kv_cfg_(kv_cfg),
      kv_(std::make_unique<KVCacheManager>(kv_cfg, cfg.max_model_len, cfg.enable_prefix_caching,
                                           cfg.log_stats)),
      so_(so), connector_(connector), waiting_(cfg.policy == "priority") {
  if (cfg.policy != "fcfs" && cfg.policy != "priority")
    throw std::invalid_argument("Unknown scheduling policy: " + cfg.policy);
}

RequestPtr Scheduler::get_request(const std::string& id) const {
  auto it = requests_.find(id);
  return it == requests_.end() ? nullptr : it->second;
}

void Scheduler::add_request(const RequestPtr& req) {
  if (requests_.count(req->request_id))
    throw std::invalid_argument("duplicate request id " + req->request_id);
  requests_[req->request_id] = req;
  waiting_.add(req);
}

void Scheduler::preempt_request(const RequestPtr& req) {
  kv_->free(*req);
  req->status = RequestStatus::kPreempted;
  req->num_computed_tokens = 0;
  req->num_output_placeholders = 0;
  req->spec_token_ids.clear();
  req->num_preemptions += 1;
  ++num_preempted_since_stats_;
  waiting_.prepend(req);
}

SchedulerOutput Scheduler::schedule() {
  SchedulerOutput out;
  std::vector<RequestPtr> new_reqs, resumed_reqs, running_reqs, preempted;
  std::unordered_map<std::string, KVCacheBlocks> new_blocks_of;
  std::unordered_map<std::string, int> sched_tokens;
  int budget = cfg_.max_num_batched_tokens;
  kv_->new_step_starts();

  auto unschedule = [&](const RequestPtr& r) {
    auto it = std::find(running_reqs.begin(), running_reqs.end(), r);
    if (it == running_reqs.end()) return;
    running_reqs.erase(it);
    budget += sched_tokens[r->request_id];
    sched_tokens.erase(r->request_id);
    new_blocks_of.erase(r->request_id);
    out.scheduled_spec_decode_tokens.erase(r->request_id);
    out.num_scheduled_tokens.erase(
        std::remove_if(out.num_scheduled_tokens.begin(), out.num_scheduled_tokens.end(),
                       [&](auto& p) { return p.first == r->request_id; }),
        out.num_scheduled_tokens.end());
  };

  // ------------------------------ running requests first ------------------------------
  size_t idx = 0;
  while (idx < running_.size() && budget > 0) {
    RequestPtr req = running_[idx];
    if (req->num_output_placeholders > 0 &&
        req->num_computed_tokens + 2 - req->num_output_placeholders >=
            req->num_prompt_tokens() + req->max_tokens) {
      // Async scheduling: the token that ends this request is already in flight.
      ++idx;
      continue;
    }
    int num_new = req->num_tokens_with_spec() + req->num_output_placeholders - req->num_computed_tokens;
    if (cfg_.long_prefill_token_threshold > 0 && num_new > cfg_.long_prefill_token_threshold)
      num_new = cfg_.long_prefill_token_threshold;
    num_new = std::min(num_new, budget);
    num_new = std::min(num_new, cfg_.max_model_len - 1 - req->num_computed_tokens);
    if (num_new <= 0) {
      ++idx;
      continue;
    }
    std::optional<KVCacheBlocks> nb;
    bool can_schedule = true;
    while (true) {
      nb = kv_->allocate_slots(*req, num_new, 0, nullptr, cfg_.num_lookahead_tokens);
      if (nb) break;
      // Out of KV blocks: preempt the lowest-priority (or most recent) running request.
      RequestPtr victim;
      if (cfg_.policy == "priority") {
        victim = *std::max_element(running_.begin(), running_.end(),
                                   [](const RequestPtr& a, const RequestPtr& b) {
                                     if (a->priority != b->priority) return a->priority < b->priority;
                                     return a->arrival_time < b->arrival_time;
                                   });
        running_.erase(std::find(running_.begin(), running_.end(), victim));
        unschedule(victim);
      } else {
        victim = running_.back();
        running_.pop_back();
      }
      preempt_request(victim);
      preempted.push_back(victim);
      if (victim == req) {
        can_schedule = false;
        break;
      }
    }
    if (!can_schedule) break;
    // The request may have moved if an earlier-indexed victim was removed (priority policy).
    auto pos = std::find(running_.begin(), running_.end(), req);
    idx = (size_t)(pos - running_.begin()) + 1;
    running_reqs.push_back(req);
    new_blocks_of[req->request_id] = *nb;
    sched_tokens[req->request_id] = num_new;
    out.num_scheduled_tokens.emplace_back(req->request_id, num_new);
    budget -= num_new;
    if (!req->spec_token_ids.empty()) {
      int n_spec = num_new + req->num_computed_tokens - req->num_tokens() - req->num_output_placeholders;
      if (n_spec > 0) {
        if ((int)req->spec_token_ids.size() > n_spec) req->spec_token_ids.resize(n_spec);
        out.scheduled_spec_decode_tokens[req->request_id] = req->spec_token_ids;
      }
    }
  }

  // ------------------------------ then waiting requests -------------------------------
  std::vector<RequestPtr> skipped;
  if (preempted.empty()) {
    while (!waiting_.empty() && budget > 0) {
      if ((int)running_.size() >= cfg_.max_num_seqs) break;
      RequestPtr req = waiting_.peek();
      if (req->status == RequestStatus::kWaitingForFsm) {
        if (so_ && !so_->grammar_ready(*req)) {
          waiting_.pop();
          skipped.push_back(req);
          continue;
        }
        req->status = RequestStatus::kWaiting;
      }
      if (req->status == RequestStatus::kWaitingForRemoteKvs) {
        // promoted once the runner has reported the transfer complete (update_from_output)
        if (!promote_after_remote_kv(*req)) {
          waiting_.pop();
          skipped.push_back(req);
          continue;
        }
        req->status = RequestStatus::kWaiting;
      }
      int num_local = 0, num_external = 0;
      bool load_async = false;
      KVCacheBlocks computed = kv_->empty_blocks();
      int num_computed;
      if (req->num_computed_tokens == 0) {
        auto hit = kv_->get_computed_blocks(*req);
        computed = hit.first;
        num_local = hit.second;
        if (connector_) {
          auto ext = connector_->get_num_new_matched_tokens(*req, num_local);
          if (!ext) {  // the store cannot answer yet: try again next step
            waiting_.pop();
            skipped.push_back(req);
            continue;
          }
          num_external = ext->first;
          load_async = ext->second;
        }
        num_computed = num_local + num_external;
      } else {
        num_computed = req->num_computed_tokens;
      }
      int num_new;
      if (load_async) {
        num_new = 0;
      } else {
        num_new = req->num_tokens() - num_computed;
        if (cfg_.long_prefill_token_threshold > 0 && num_new > cfg_.long_prefill_token_threshold)
          num_new = cfg_.long_prefill_token_threshold;
        if (!cfg_.enable_chunked_prefill && num_new > budget) break;
        num_new = std::min(num_new, budget);
        assert(num_new > 0);
      }
      auto nb = kv_->allocate_slots(*req, num_new + num_external, num_local, &computed,
                                    cfg_.num_lookahead_tokens, load_async);
      if (!nb) break;  // cannot fit: stop admitting
      if (connector_)
        connector_->update_state_after_alloc(*req, kv_->get_block_ids(req->request_id), num_external);
      waiting_.pop();
      if (load_async) {
        req->status = RequestStatus::kWaitingForRemoteKvs;
        skipped.push_back(req);
        continue;
      }
      running_.push_back(req);
      if (req->status == RequestStatus::kPreempted) resumed_reqs.push_back(req);
      else new_reqs.push_back(req);
      new_blocks_of[req->request_id] = kv_->get_blocks(req->request_id);
      sched_tokens[req->request_id] = num_new;
      out.num_scheduled_tokens.emplace_back(req->request_id, num_new);
      budget -= num_new;
      req->status = RequestStatus::kRunning;
      req->num_computed_tokens = num_computed;
      if (req->num_cached_tokens < 0) req->num_cached_tokens = num_computed;
    }
  }
  if (!skipped.empty()) waiting_.prepend_all(skipped);

  // ------------------------------ assemble the output ---------------------------------
  out.total_num_scheduled_tokens = cfg_.max_num_batched_tokens - budget;
  assert(out.total_num_scheduled_tokens <= cfg_.max_num_batched_tokens);
  if (!running_.empty())
    out.num_common_prefix_blocks = kv_->get_num_common_prefix_blocks(*running_[0], (int)running_.size());
  else
    out.num_common_prefix_blocks.assign(kv_->num_groups(), 0);

  auto as_new = [&](const RequestPtr& r) {
    NewRequestData d;
    d.req_id = r->request_id;
    d.prompt_token_ids = r->all_token_ids;  // resumed requests carry their generated tokens too
    d.sampling_params = r->sampling_params;
    d.block_ids = new_blocks_of[r->request_id].block_ids();
    d.num_computed_tokens = r->num_computed_tokens;
    d.num_prompt_tokens = r->num_prompt_tokens();
    return d;
  };
  for (auto& r : new_reqs) out.scheduled_new_reqs.push_back(as_new(r));
  for (auto& r : resumed_reqs) out.scheduled_new_reqs.push_back(as_new(r));
  for (auto& r : running_reqs) {
    auto& c = out.scheduled_cached_reqs;
    c.req_ids.push_back(r->request_id);
    c.resumed_from_preemption.push_back(0);
    // tokens the worker has not seen yet: everything sampled after what it has computed
    int n_sched = sched_tokens[r->request_id];
    int lo = r->num_computed_tokens;
    int hi = std::min(r->num_tokens(), lo + n_sched);
    std::vector<int32_t> toks;
    if (lo < hi && lo >= r->num_prompt_tokens())
      toks.assign(r->all_token_ids.begin() + lo, r->all_token_ids.begin() + hi);
    c.new_token_ids.push_back(std::move(toks));
    c.new_block_ids.push_back(new_blocks_of[r->request_id].block_ids());
    c.num_computed_tokens.push_back(r->num_computed_tokens);
    c.num_output_tokens.push_back(r->num_output_tokens());
  }
  for (auto& r : preempted) out.preempted_req_ids.push_back(r->request_id);
  for (auto& p : out.num_scheduled_tokens) {
    auto r = requests_[p.first];
    if (r->use_structured_output) out.structured_output_request_ids.push_back(p.first);
  }
  out.finished_req_ids = finished_req_ids_;
  if (connector_) out.kv_connector_metadata = connector_->build_connector_meta(out);
  last_step_tokens_ = out.total_num_scheduled_tokens;
  update_after_schedule(out);
  return out;
}

void Scheduler::update_after_schedule(const SchedulerOutput& so) {
  for (auto& p : so.num_scheduled_tokens) requests_[p.first]->num_computed_tokens += p.second;
  finished_req_ids_.clear();
}

GrammarOutput Scheduler::get_grammar_bitmask(const SchedulerOutput& so) {
  GrammarOutput g;
  if (!so_ || so.structured_output_request_ids.empty()) return g;
  std::vector<RequestPtr> reqs;
  for (auto& id : so.structured_output_request_ids) {
    auto r = get_request(id);
    // Only requests that will sample this step need a mask row.
    if (r && r->num_computed_tokens >= r->num_tokens() + r->num_output_placeholders - (cfg_.async_scheduling ? 1 : 0))
      reqs.push_back(r);
  }
  if (reqs.empty()) return g;
  return so_->grammar_bitmask(reqs, so.scheduled_spec_decode_tokens);
}

bool Scheduler::check_stop(Request& req) {
  const SamplingParams& sp = req.sampling_params;
  if (req.num_output_tokens() < sp.min_tokens) return false;
  int32_t last = req.output_token_ids.back();
  if (!sp.ignore_eos && req.eos_token_id && last == *req.eos_token_id) {
    req.status = RequestStatus::kFinishedStopped;
    return true;
  }
  if (std::binary_search(sp.stop_token_ids.begin(), sp.stop_token_ids.end(), last)) {
    req.status = RequestStatus::kFinishedStopped;
    req.stop_reason = StopReason{true, last, ""};
    return true;
  }
  if (req.num_tokens() >= cfg_.max_model_len || req.num_output_tokens() >= req.max_tokens) {
    req.status = RequestStatus::kFinishedLengthCapped;
    return true;
  }
  return false;
}

void Scheduler::update_request_with_output(Request& req, std::vector<int32_t>& new_tokens,
                                           bool& stopped) {
  stopped = false;
  for (size_t i = 0; i < new_tokens.size(); ++i) {
    req.append_output_token(new_tokens[i]);
    if (check_stop(req)) {
      new_tokens.resize(i + 1);
      stopped = true;
      break;
    }
  }
}

EngineCoreOutputs Scheduler::update_from_output(const SchedulerOutput& so,
                                                const ModelRunnerOutput& mro) {
  EngineCoreOutputs outs;
  std::unordered_map<std::string, size_t> index;
  for (size_t i = 0; i < mro.req_ids.size(); ++i) index[mro.req_ids[i]] = i;
  std::unordered_set<Request*> stopped_set;

  for (auto& p : so.num_scheduled_tokens) {
    auto rit = requests_.find(p.first);
    if (rit == requests_.end()) continue;  // finished or aborted while the step ran
    RequestPtr req = rit->second;
    auto iit = index.find(p.first);
    std::vector<int32_t> generated;
    if (iit != index.end() && iit->second < mro.sampled_token_ids.size())
      generated = mro.sampled_token_ids[iit->second];

    auto sit = so.scheduled_spec_decode_tokens.find(p.first);
    if (sit != so.scheduled_spec_decode_tokens.end() && !generated.empty()) {
      int num_draft = (int)sit->second.size();
      int num_accepted = (int)generated.size() - 1;
      int num_rejected = num_draft - num_accepted;
      if (num_rejected > 0) {
        req->num_computed_tokens -= num_rejected;
        if (req->num_output_placeholders > 0) req->num_output_placeholders -= num_rejected;
        if (so_ && req->use_structured_output) so_->rollback(*req, 0);
      }
    }
    {
      auto rc = mro.num_recompute.find(p.first);
      if (rc != mro.num_recompute.end() && rc->second > 0) {
        // kept tokens whose recurrent state was rolled back: they run again with the next step
        req->num_computed_tokens -= std::min(rc->second, req->num_computed_tokens);
      }
    }
    bool stopped = false;
    if (!generated.empty()) update_request_with_output(*req, generated, stopped);

    if (!generated.empty() && so_ && req->use_structured_output) {
      if (!so_->accept_tokens(*req, generated)) {
        // the grammar rejected a sampled token: terminate rather than emit invalid output
        if (!stopped) {
          req->status = RequestStatus::kFinishedStopped;
          stopped = true;
        }
      } else if (!stopped && so_->is_terminated(*req) && false) {
      }
    }
    if (iit != index.end() && iit->second < mro.num_nans_in_logits.size())
      req->num_nans_in_logits = mro.num_nans_in_logits[iit->second];

    if (!generated.empty() || stopped) {
      EngineCoreOutput o;
      o.request_id = req->request_id;
      o.new_token_ids = generated;
      if (iit != index.end() && iit->second < mro.logprobs.size()) o.new_logprobs = mro.logprobs[iit->second];
      o.finish_reason = finish_reason_of(req->status);
      o.stop_reason = req->stop_reason;
      o.num_cached_tokens = std::max(req->num_cached_tokens, 0);
      outs.outputs.push_back(std::move(o));
    }
    if (stopped) {
      stopped_set.insert(req.get());
      free_request(req);
    }
  }
  if (!stopped_set.empty()) {
    running_.erase(std::remove_if(running_.begin(), running_.end(),
                                  [&](const RequestPtr& r) { return stopped_set.count(r.get()) > 0; }),
                   running_.end());
  }
  // external KV transfers the runner saw complete during this step
  for (auto& id : mro.finished_recving)
    if (requests_.count(id)) finished_recving_.insert(id);
  for (auto& id : mro.finished_sending) {
    auto it = delayed_free_.find(id);
    if (it == delayed_free_.end()) continue;
    kv_->free(*it->second);
    delayed_free_.erase(it);
  }
  auto st = kv_->take_prefix_cache_stats();
  pc_queries_ += st.queries;
  pc_hits_ += st.hits;
  if (cfg_.log_stats) outs.scheduler_stats = make_stats();
  outs.finished_requests = finished_req_ids_;
  return outs;
}

void Scheduler::free_request(const RequestPtr& req) {
  bool delay = false;
  if (connector_) delay = connector_->request_finished(*req, kv_->get_block_ids(req->request_id));
  if (so_ && req->use_structured_output) so_->release(*req);
  finished_req_ids_.insert(req->request_id);
  finished_recving_.erase(req->request_id);
  if (delay) delayed_free_[req->request_id] = req;   // blocks stay until finished_sending names it
  else kv_->free(*req);
  requests_.erase(req->request_id);
}

// A request whose prefix is being loaded by the connector holds its blocks but computes
// nothing. When the runner reports the load complete, the loaded blocks become ordinary
// computed (and cacheable) blocks and the request goes back to plain waiting. The last prompt
// token is always left to compute, so that the request produces logits.
bool Scheduler::promote_after_remote_kv(Request& req) {
  auto it = finished_recving_.find(req.request_id);
  if (it == finished_recving_.end()) return false;
  const auto ids = kv_->get_block_ids(req.request_id);
  int n = ids.empty() ? 0 : (int)ids[0].size() * kv_->block_size();
  n = std::min(n, req.num_tokens());
  if (n == req.num_tokens()) n -= 1;
  if (n > 0) kv_->cache_blocks(req, n);
  req.num_computed_tokens = std::max(n, 0);
  if (req.num_cached_tokens < 0) req.num_cached_tokens = req.num_computed_tokens;
  finished_recving_.erase(it);
  return true;
}

void Scheduler::finish_requests(const std::vector<std::string>& ids, RequestStatus status) {
  assert(is_finished(status));
  for (auto& id : ids) {
    auto it = requests_.find(id);
    if (it == requests_.end()) continue;  // already finished
    RequestPtr req = it->second;
    if (req->status == RequestStatus::kRunning) {
      running_.erase(std::remove(running_.begin(), running_.end(), req), running_.end());
    } else {
      waiting_.remove(req);
    }
    req->status = status;
    free_request(req);
  }
}

void Scheduler::update_draft_token_ids(const DraftTokenIds& drafts) {
  for (size_t i = 0; i < drafts.req_ids.size(); ++i) {
    auto r = get_request(drafts.req_ids[i]);
    if (!r || r->finished()) continue;
    // A request that is still prefilling (chunked) cannot verify drafts yet.
    if (r->num_computed_tokens < r->num_tokens() - 1) { r->spec_token_ids.clear(); continue; }
    r->spec_token_ids = drafts.draft_token_ids[i];
  }
}

SchedulerStats Scheduler::make_stats() {
  SchedulerStats s;
  s.num_running_reqs = (int)running_.size();
  s.num_waiting_reqs = (int)waiting_.size();
  s.kv_cache_usage = kv_->usage();
  s.prefix_cache_queries = pc_queries_;
  s.prefix_cache_hits = pc_hits_;
  s.num_preempted = num_preempted_since_stats_;
  s.step_scheduled_tokens = last_step_tokens_;
  num_preempted_since_stats_ = 0;
  return s;
}

// ----------------------------------------------------------------------- AsyncScheduler
void AsyncScheduler::update_after_schedule(const SchedulerOutput& so) {
  Scheduler::update_after_schedule(so);
  for (auto& p : so.num_scheduled_tokens) {
    Request& r = *requests_[p.first];
    // This step computes the request's last known token: a new token will come out of it.
    if (r.num_computed_tokens == r.num_tokens() + r.num_output_placeholders)
      r.num_output_placeholders += 1;
  }
}

void AsyncScheduler::update_request_with_output(Request& req, std::vector<int32_t>& new_tokens,
                                                bool& stopped) {
  RequestStatus before = req.status;
  size_t n_in = new_tokens.size();
  Scheduler::update_request_with_output(req, new_tokens, stopped);
  req.num_output_placeholders -= (int)n_in;
  if (req.num_output_placeholders < 0) req.num_output_placeholders = 0;
  if (before == RequestStatus::kRunning && !stopped)
    kv_->cache_blocks(req, req.num_computed_tokens - req.num_output_placeholders);
}

}  // namespace b200
