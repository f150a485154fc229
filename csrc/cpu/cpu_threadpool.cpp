#include "cpu_threadpool.h"

#include <algorithm>
#include <cstdlib>
#include <memory>

namespace b200cpu {

static std::unique_ptr<ThreadPool> g_pool;
static std::mutex g_pool_mu;
static int g_threads = 0;

ThreadPool& ThreadPool::instance() {
  std::lock_guard<std::mutex> lock(g_pool_mu);
  if (!g_pool) {
    int n = g_threads;
    if (n <= 0) {
      const char* e = std::getenv("B200_CPU_THREADS");
      n = e ? std::atoi(e) : (int)std::thread::hardware_concurrency();
    }
    if (n < 1) n = 1;
    g_pool.reset(new ThreadPool(n));
  }
  return *g_pool;
}

void ThreadPool::set_num_threads(int n) {
  std::lock_guard<std::mutex> lock(g_pool_mu);
  g_threads = n;
  g_pool.reset();
}

ThreadPool::ThreadPool(int num_threads) {
  for (int i = 1; i < num_threads; ++i) workers_.emplace_back([this, i] { worker_loop(i); });
}

ThreadPool::~ThreadPool() {
  {
    std::lock_guard<std::mutex> lock(mu_);
    stop_.store(true);
    epoch_.fetch_add(1);
  }
  cv_.notify_all();
  for (auto& t : workers_) t.join();
}

void ThreadPool::worker_loop(int id) {
  uint64_t seen = 0;
  while (true) {
    // spin for about a millisecond (the ops of one forward pass follow each other within tens of
    // microseconds; waking a parked thread costs more than the small ops themselves), then park
    uint64_t e = epoch_.load(std::memory_order_acquire);
    for (int spin = 0; e == seen && spin < 30000; ++spin) {
#if defined(__x86_64__)
      __builtin_ia32_pause();
#endif
      e = epoch_.load(std::memory_order_acquire);
    }
    if (e == seen) {
      std::unique_lock<std::mutex> lock(mu_);
      cv_.wait(lock, [&] { return epoch_.load(std::memory_order_acquire) != seen; });
      e = epoch_.load(std::memory_order_acquire);
    }
    seen = e;
    if (stop_.load()) return;
    if (id < parts_) {
      const int64_t b = (int64_t)id * chunk_, en = std::min(n_, b + chunk_);
      if (b < en) (*fn_)(b, en);
    }
    pending_.fetch_sub(1, std::memory_order_acq_rel);
  }
}

void ThreadPool::parallel_for(int64_t n, int64_t grain, const std::function<void(int64_t, int64_t)>& fn) {
  if (n <= 0) return;
  const int threads = size();
  int parts = (int)std::min<int64_t>(threads, std::max<int64_t>(1, n / std::max<int64_t>(1, grain)));
  if (parts <= 1 || workers_.empty()) {
    fn(0, n);
    return;
  }
  // One job at a time: a second caller (another host thread driving its own model, or a call made
  // from inside a job) runs its range inline instead of waiting for the pool.
  std::unique_lock<std::mutex> job(job_mu_, std::try_to_lock);
  if (!job.owns_lock()) {
    fn(0, n);
    return;
  }
  {
    std::lock_guard<std::mutex> lock(mu_);
    fn_ = &fn;
    n_ = n;
    parts_ = parts;
    chunk_ = (n + parts - 1) / parts;
    pending_.store((int)workers_.size(), std::memory_order_release);
    epoch_.fetch_add(1, std::memory_order_acq_rel);
  }
  cv_.notify_all();
  fn(0, std::min(n, chunk_));                      // part 0 on the calling thread
  while (pending_.load(std::memory_order_acquire) != 0) {
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  }
}

}  // namespace b200cpu
