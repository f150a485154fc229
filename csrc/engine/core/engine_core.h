// Engine core: the schedule -> execute -> sample -> update step loop, its depth-2
// batch-queue variant for asynchronous scheduling, and the busy-loop process wrapper with
// blocking input/output queues.
//
// Behavioural parity: src/vllm/v1/engine/core.cpp:44-118 (step), :135-245
// (step_with_batch_queue), core_proc.cpp:30-146, core_client.cpp (InprocClient),
// include/vllm/v1/executor/executor.h:48-85, worker/gpu/model_runner_base.h.
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <future>
#include <mutex>
#include <thread>

#include "core/scheduler.h"

namespace b200 {

// What a worker must implement. execute_model runs the forward pass for the scheduled
// tokens and keeps the logits; sample_tokens consumes them (after the grammar bitmask is
// known) and returns the sampled ids.
class ModelRunnerBase {
 public:
  virtual ~ModelRunnerBase() = default;
  virtual void execute_model(const SchedulerOutput& so) = 0;
  virtual ModelRunnerOutput sample_tokens(const GrammarOutput* grammar) = 0;
  // Asynchronous variant: returns a handle whose get() blocks only on the device->host copy
  // of the sampled ids. The default wraps the synchronous call.
  virtual std::function<ModelRunnerOutput()> sample_tokens_async(const GrammarOutput* grammar) {
    ModelRunnerOutput o = sample_tokens(grammar);
    return [o]() { return o; };
  }
  virtual std::optional<DraftTokenIds> take_draft_token_ids() { return std::nullopt; }
  virtual bool supports_async() const { return false; }
  virtual KVCacheConfig kv_cache_config() const { return {}; }
};

// Single-process executor: forwards to one runner. (Multi-GPU ranks are separate processes
// that run the same schedule in lockstep; see the parallel package.)
class Executor {
 public:
  explicit Executor(ModelRunnerBase* runner, int max_concurrent_batches = 1)
      : runner_(runner), max_concurrent_batches_(max_concurrent_batches) {}
  void execute_model(const SchedulerOutput& so) { runner_->execute_model(so); }
  ModelRunnerOutput sample_tokens(const GrammarOutput* g) { return runner_->sample_tokens(g); }
  std::function<ModelRunnerOutput()> sample_tokens_async(const GrammarOutput* g) {
    return runner_->sample_tokens_async(g);
  }
  std::optional<DraftTokenIds> take_draft_token_ids() { return runner_->take_draft_token_ids(); }
  int max_concurrent_batches() const { return max_concurrent_batches_; }
  ModelRunnerBase* runner() { return runner_; }

 private:
  ModelRunnerBase* runner_;
  int max_concurrent_batches_;
};

class EngineCore {
 public:
  EngineCore(std::unique_ptr<Scheduler> scheduler, Executor* executor);
  void add_request(const EngineCoreRequest& req);
  void abort_requests(const std::vector<std::string>& ids);
  // One step; returns (outputs, model_executed).
  std::pair<EngineCoreOutputs, bool> step();
  // Depth-N overlap: schedules and launches the next batch before blocking on the oldest.
  std::pair<EngineCoreOutputs, bool> step_with_batch_queue();
  bool has_work() const { return scheduler_->has_requests() || !batch_queue_.empty(); }
  bool has_unfinished() const { return scheduler_->has_unfinished_requests(); }
  Scheduler& scheduler() { return *scheduler_; }
  Executor& executor() { return *executor_; }
  int batch_queue_size() const { return batch_queue_size_; }
  bool reset_prefix_cache() { return scheduler_->reset_prefix_cache(); }
  // Step counters for tests / observability.
  int64_t num_steps = 0, num_executed_steps = 0;
  double last_schedule_ms = 0, last_execute_ms = 0, last_update_ms = 0;

 private:
  void post_step(bool model_executed);
  std::unique_ptr<Scheduler> scheduler_;
  Executor* executor_;
  int batch_queue_size_;
  struct InFlight {
    SchedulerOutput so;
    std::function<ModelRunnerOutput()> get;
  };
  std::deque<InFlight> batch_queue_;
  std::deque<EngineCoreOutputs> pending_;
};

// ------------------------------------------------------------------------ blocking queue
template <class T>
class BlockingQueue {
 public:
  void put(T v) {
    {
      std::lock_guard<std::mutex> l(mu_);
      q_.push_back(std::move(v));
    }
    cv_.notify_one();
  }
  T get() {
    std::unique_lock<std::mutex> l(mu_);
    cv_.wait(l, [&] { return !q_.empty(); });
    T v = std::move(q_.front());
    q_.pop_front();
    return v;
  }
  std::optional<T> get_nowait() {
    std::lock_guard<std::mutex> l(mu_);
    if (q_.empty()) return std::nullopt;
    T v = std::move(q_.front());
    q_.pop_front();
    return v;
  }
  std::optional<T> get_for(double seconds) {
    std::unique_lock<std::mutex> l(mu_);
    if (!cv_.wait_for(l, std::chrono::duration<double>(seconds), [&] { return !q_.empty(); }))
      return std::nullopt;
    T v = std::move(q_.front());
    q_.pop_front();
    return v;
  }
  bool empty() const {
    std::lock_guard<std::mutex> l(mu_);
    return q_.empty();
  }

 private:
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::deque<T> q_;
};

enum class CoreRequestType : int { kAdd, kAbort, kWakeup, kExecutorFailed, kShutdown };
struct CoreInput {
  CoreRequestType type = CoreRequestType::kWakeup;
  std::optional<EngineCoreRequest> request;
  std::vector<std::string> abort_ids;
};

class EngineDeadError : public std::runtime_error {
 public:
  explicit EngineDeadError(const std::string& m = "EngineCore encountered an issue. See the log for the root cause.")
      : std::runtime_error(m) {}
};

// Busy loop on its own thread: while running: drain input queue (blocking when idle), step,
// push outputs. A runner exception turns into an `engine_dead` output for every waiter.
class EngineCoreProc {
 public:
  EngineCoreProc(EngineCore* core, bool use_batch_queue);
  ~EngineCoreProc();
  void start();
  // abort = true: running requests finish as aborted; false: drain them first.
  void shutdown(bool abort = true);
  BlockingQueue<CoreInput>& input() { return input_; }
  BlockingQueue<EngineCoreOutputs>& output() { return output_; }
  bool dead() const { return dead_.load(); }
  bool running() const { return running_.load(); }

 private:
  void run_busy_loop();
  bool process_input_queue();
  void handle(const CoreInput& in);
  EngineCore* core_;
  bool use_batch_queue_;
  BlockingQueue<CoreInput> input_;
  BlockingQueue<EngineCoreOutputs> output_;
  std::thread thread_;
  std::atomic<bool> running_{false}, dead_{false}, shutdown_requested_{false}, drain_{false};
};

// In-process client: owns the engine thread.
class InprocClient {
 public:
  InprocClient(EngineCore* core, bool use_batch_queue) : proc_(core, use_batch_queue) { proc_.start(); }
  ~InprocClient() { proc_.shutdown(true); }
  void add_request_async(const EngineCoreRequest& r);
  void abort_requests_async(const std::vector<std::string>& ids);
  // Blocks; throws EngineDeadError once the engine thread died.
  EngineCoreOutputs get_output();
  std::optional<EngineCoreOutputs> get_output_for(double seconds);
  bool engine_dead() const { return proc_.dead(); }
  void shutdown(bool abort = true) { proc_.shutdown(abort); }
  EngineCoreProc& proc() { return proc_; }

 private:
  EngineCoreProc proc_;
};

}  // namespace b200
