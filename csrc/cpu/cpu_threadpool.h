// Persistent worker pool for the CPU backend. Work is always split by OUTPUT index (rows of a
// GEMM, tokens of a norm, (request, head) pairs of attention), every output element is computed
// by exactly one thread with a fixed summation order, so results are bit-identical for any
// thread count. Workers spin briefly between ops and then park on a condition variable. The pool
// runs one job at a time; a caller that finds it busy computes its whole range itself (same
// result, since the partition never changes what one output element sums).
// Reference: src/vt/cpu/cpu_threadpool.{h,cpp}.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace b200cpu {

class ThreadPool {
 public:
  explicit ThreadPool(int num_threads);
  ~ThreadPool();
  int size() const { return (int)workers_.size() + 1; }
  // Calls fn(begin, end) on contiguous chunks of [0, n); the caller runs one chunk itself.
  // `grain`: smallest chunk worth a thread.
  void parallel_for(int64_t n, int64_t grain, const std::function<void(int64_t, int64_t)>& fn);
  static ThreadPool& instance();
  static void set_num_threads(int n);

 private:
  void worker_loop(int id);
  std::vector<std::thread> workers_;
  std::mutex mu_;
  std::mutex job_mu_;       // held by the caller whose job the workers are running
  std::condition_variable cv_;
  std::atomic<uint64_t> epoch_{0};
  std::atomic<int> pending_{0};
  std::atomic<bool> stop_{false};
  // current job
  const std::function<void(int64_t, int64_t)>* fn_ = nullptr;
  int64_t n_ = 0, chunk_ = 0;
  int parts_ = 0;
};

}  // namespace b200cpu
