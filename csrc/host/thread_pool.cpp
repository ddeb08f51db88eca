#include "host/thread_pool.h"

#include <algorithm>
#include <atomic>
#include <cstdlib>

namespace recml {

ThreadPool::ThreadPool(int threads) {
  threads = std::max(1, threads);
  for (int i = 0; i < threads; ++i) workers_.emplace_back([this] { loop(); });
}

ThreadPool::~ThreadPool() {
  {
    std::lock_guard<std::mutex> lock(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  for (auto& t : workers_) t.join();
}

void ThreadPool::submit(std::function<void()> fn) {
  {
    std::lock_guard<std::mutex> lock(mu_);
    tasks_.push(std::move(fn));
    ++pending_;
  }
  cv_.notify_one();
}

void ThreadPool::wait() {
  std::unique_lock<std::mutex> lock(mu_);
  done_cv_.wait(lock, [this] { return pending_ == 0; });
}

void ThreadPool::loop() {
  for (;;) {
    std::function<void()> fn;
    {
      std::unique_lock<std::mutex> lock(mu_);
      cv_.wait(lock, [this] { return stop_ || !tasks_.empty(); });
      if (stop_ && tasks_.empty()) return;
      fn = std::move(tasks_.front());
      tasks_.pop();
    }
    fn();
    {
      std::lock_guard<std::mutex> lock(mu_);
      if (--pending_ == 0) done_cv_.notify_all();
    }
  }
}

void ThreadPool::parallel_for(long long n, const std::function<void(long long, long long, int)>& fn, long long min_chunk) {
  if (n <= 0) return;
  const int parts = static_cast<int>(std::max<long long>(1, std::min<long long>(size(), n / std::max<long long>(1, min_chunk))));
  if (parts == 1) {
    fn(0, n, 0);
    return;
  }
  // Work is handed out in grains from a shared counter, so uneven items (a long file, a wide feature) do
  // not leave the other workers idle.  A private completion latch, so nested / concurrent parallel_for
  // calls do not wait on each other.
  const long long grain = std::max<long long>(std::max<long long>(1, min_chunk), (n + parts * 8LL - 1) / (parts * 8LL));
  std::atomic<long long> next{0};
  std::mutex mu;
  std::condition_variable cv;
  int left = parts;
  for (int p = 0; p < parts; ++p) {
    submit([&, p] {
      for (;;) {
        const long long b = next.fetch_add(grain);
        if (b >= n) break;
        fn(b, std::min(n, b + grain), p);
      }
      std::lock_guard<std::mutex> lock(mu);
      if (--left == 0) cv.notify_all();
    });
  }
  std::unique_lock<std::mutex> lock(mu);
  cv.wait(lock, [&] { return left == 0; });
}

ThreadPool& ThreadPool::global() {
  static ThreadPool* pool = [] {
    const char* env = std::getenv("RECML_HOST_THREADS");
    int n = env ? std::atoi(env) : static_cast<int>(std::thread::hardware_concurrency());
    return new ThreadPool(std::max(1, std::min(n, 64)));
  }();
  return *pool;
}

}  // namespace recml
