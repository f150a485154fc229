#include "core/engine_core.h"

#include <chrono>

namespace b200 {

static inline double now_ms() {
  return std::chrono::duration<double, std::milli>(
             std::chrono::steady_clock::now().time_since_epoch()).count();
}

EngineCore::EngineCore(std::unique_ptr<Scheduler> scheduler, Executor* executor)
    : scheduler_(std::move(scheduler)), executor_(executor),
      batch_queue_size_(executor->max_concurrent_batches()) {}

void EngineCore::add_request(const EngineCoreRequest& r) {
  SamplingParams sp = r.sampling_params;
  sp.verify();
  EngineCoreRequest rr = r;
  rr.sampling_params.post_init();
  if (rr.prompt_token_ids.empty()) throw std::invalid_argument("prompt must contain at least one token");
  scheduler_->add_request(std::make_shared<Request>(rr));
}

void EngineCore::abort_requests(const std::vector<std::string>& ids) {
  scheduler_->finish_requests(ids, RequestStatus::kFinishedAborted);
}

void EngineCore::post_step(bool model_executed) {
  if (!model_executed) return;
  auto drafts = executor_->take_draft_token_ids();
  if (drafts) scheduler_->update_draft_token_ids(*drafts);
}

std::pair<EngineCoreOutputs, bool> EngineCore::step() {
  ++num_steps;
  if (!scheduler_->has_requests()) return {EngineCoreOutputs{}, false};
  double t0 = now_ms();
  SchedulerOutput so = scheduler_->schedule();
  double t1 = now_ms();
  bool executed = so.total_num_scheduled_tokens > 0;
  ModelRunnerOutput mro;
  // The runner sees every scheduler output, also an empty one: that is how it learns about
  // finished and preempted requests and releases their state.
  executor_->execute_model(so);
  if (executed) {
    GrammarOutput g = scheduler_->get_grammar_bitmask(so);
    mro = executor_->sample_tokens(g.structured_output_request_ids.empty() ? nullptr : &g);
    ++num_executed_steps;
  }
  double t2 = now_ms();
  EngineCoreOutputs outs = scheduler_->update_from_output(so, mro);
  post_step(executed);
  double t3 = now_ms();
  last_schedule_ms = t1 - t0;
  last_execute_ms = t2 - t1;
  last_update_ms = t3 - t2;
  return {std::move(outs), executed};
}

std::pair<EngineCoreOutputs, bool> EngineCore::step_with_batch_queue() {
  ++num_steps;
  bool executed = false;
  // Fill the queue first: launching the next batch has priority over collecting results.
  if ((int)batch_queue_.size() < batch_queue_size_ && scheduler_->has_requests()) {
    double t0 = now_ms();
    SchedulerOutput so = scheduler_->schedule();
    last_schedule_ms = now_ms() - t0;
    executor_->execute_model(so);  // also for an empty schedule (state release)
    if (so.total_num_scheduled_tokens > 0) {
      // Structured requests need the tokens of the previous step to advance their grammar
      // before a mask can be built, so their sampling cannot be deferred behind the queue.
      bool has_structured = !so.structured_output_request_ids.empty();
      if (has_structured) {
        while (!batch_queue_.empty()) {
          InFlight f = std::move(batch_queue_.front());
          batch_queue_.pop_front();
          ModelRunnerOutput m = f.get();
          // results of drained batches are folded in below through a recursive-free path
          EngineCoreOutputs o = scheduler_->update_from_output(f.so, m);
          pending_.push_back(std::move(o));
        }
        GrammarOutput g = scheduler_->get_grammar_bitmask(so);
        ModelRunnerOutput m = executor_->sample_tokens(g.structured_output_request_ids.empty() ? nullptr : &g);
        batch_queue_.push_back(InFlight{so, [m]() { return m; }});
      } else {
        batch_queue_.push_back(InFlight{so, executor_->sample_tokens_async(nullptr)});
      }
      executed = true;
      ++num_executed_steps;
      if (!pending_.empty()) {
        EngineCoreOutputs o = std::move(pending_.front());
        pending_.pop_front();
        return {std::move(o), true};
      }
      // Queue not yet full and more work can be scheduled: come back without blocking.
      if ((int)batch_queue_.size() < batch_queue_size_ && scheduler_->has_unfinished_requests() &&
          !has_structured)
        return {EngineCoreOutputs{}, true};
    } else if (batch_queue_.empty()) {
      // Nothing to run: still report finished/aborted ids.
      EngineCoreOutputs o = scheduler_->update_from_output(so, ModelRunnerOutput{});
      return {std::move(o), false};
    }
  }
  if (!pending_.empty()) {
    EngineCoreOutputs o = std::move(pending_.front());
    pending_.pop_front();
    return {std::move(o), executed};
  }
  if (batch_queue_.empty()) return {EngineCoreOutputs{}, executed};
  InFlight f = std::move(batch_queue_.front());
  batch_queue_.pop_front();
  double t0 = now_ms();
  ModelRunnerOutput mro = f.get();  // the only host wait: a copy-stream event
  last_execute_ms = now_ms() - t0;
  t0 = now_ms();
  EngineCoreOutputs outs = scheduler_->update_from_output(f.so, mro);
  post_step(true);
  last_update_ms = now_ms() - t0;
  return {std::move(outs), executed};
}

// ---------------------------------------------------------------------- EngineCoreProc
EngineCoreProc::EngineCoreProc(EngineCore* core, bool use_batch_queue)
    : core_(core), use_batch_queue_(use_batch_queue) {}

EngineCoreProc::~EngineCoreProc() { shutdown(true); }

void EngineCoreProc::start() {
  if (running_.exchange(true)) return;
  thread_ = std::thread([this] { run_busy_loop(); });
}

void EngineCoreProc::shutdown(bool abort) {
  if (!running_.load() && !thread_.joinable()) return;
  drain_.store(!abort);
  shutdown_requested_.store(true);
  CoreInput in;
  in.type = CoreRequestType::kShutdown;
  input_.put(in);
  if (thread_.joinable()) thread_.join();
  running_.store(false);
}

void EngineCoreProc::handle(const CoreInput& in) {
  switch (in.type) {
    case CoreRequestType::kAdd:
      if (shutdown_requested_.load()) {
        // Too late: answer with a terminal abort so the waiter is released.
        EngineCoreOutputs o;
        EngineCoreOutput e;
        e.request_id = in.request->request_id;
        e.finish_reason = FinishReason::kAbort;
        o.outputs.push_back(e);
        output_.put(std::move(o));
      } else {
        try {
          core_->add_request(*in.request);
        } catch (const std::invalid_argument& ex) {
          EngineCoreOutputs o;
          EngineCoreOutput e;
          e.request_id = in.request->request_id;
          e.finish_reason = FinishReason::kAbort;
          o.outputs.push_back(e);
          o.error = ex.what();
          output_.put(std::move(o));
        }
      }
      break;
    case CoreRequestType::kAbort: core_->abort_requests(in.abort_ids); break;
    case CoreRequestType::kExecutorFailed: throw std::runtime_error("Executor failed.");
    default: break;
  }
}

bool EngineCoreProc::process_input_queue() {
  // Block while there is nothing to do; then drain whatever has arrived.
  if (!core_->has_work() && !shutdown_requested_.load()) {
    CoreInput in = input_.get();
    handle(in);
  }
  while (auto in = input_.get_nowait()) handle(*in);
  return true;
}

void EngineCoreProc::run_busy_loop() {
  try {
    while (true) {
      process_input_queue();
      if (shutdown_requested_.load()) {
        if (!drain_.load() || !core_->has_unfinished()) {
          // abort whatever is left so that every waiter sees a terminal output
          EngineCoreOutputs o;
          std::vector<std::string> all = core_->scheduler().all_request_ids();
          core_->abort_requests(all);
          for (auto& id : all) {
            EngineCoreOutput e;
            e.request_id = id;
            e.finish_reason = FinishReason::kAbort;
            o.outputs.push_back(e);
          }
          if (!o.outputs.empty()) output_.put(std::move(o));
          break;
        }
      }
      if (!core_->has_work()) continue;
      auto [outs, executed] = use_batch_queue_ ? core_->step_with_batch_queue() : core_->step();
      (void)executed;
      if (!outs.outputs.empty() || !outs.finished_requests.empty() || outs.scheduler_stats)
        output_.put(std::move(outs));
    }
  } catch (const std::exception& ex) {
    dead_.store(true);
    EngineCoreOutputs o;
    o.engine_dead = true;
    o.error = ex.what();
    output_.put(std::move(o));
  }
  running_.store(false);
}

// ------------------------------------------------------------------------ InprocClient
void InprocClient::add_request_async(const EngineCoreRequest& r) {
  if (proc_.dead()) throw EngineDeadError();
  CoreInput in;
  in.type = CoreRequestType::kAdd;
  in.request = r;
  proc_.input().put(std::move(in));
}
void InprocClient::abort_requests_async(const std::vector<std::string>& ids) {
  if (ids.empty() || proc_.dead()) return;
  CoreInput in;
  in.type = CoreRequestType::kAbort;
  in.abort_ids = ids;
  proc_.input().put(std::move(in));
}
EngineCoreOutputs InprocClient::get_output() {
  EngineCoreOutputs o = proc_.output().get();
  if (o.engine_dead) throw EngineDeadError(o.error.empty() ? "engine core died" : o.error);
  return o;
}
std::optional<EngineCoreOutputs> InprocClient::get_output_for(double seconds) {
  auto o = proc_.output().get_for(seconds);
  if (o && o->engine_dead) throw EngineDeadError(o->error.empty() ? "engine core died" : o->error);
  return o;
}

}  // namespace b200
