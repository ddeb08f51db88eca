// Fixed-size worker pool shared by the host-side native components (id preprocessing, record
// parsing, checkpoint chunk I/O).  parallel_for hands [0, n) out in contiguous grains from a shared counter.
#pragma once
#include <condition_variable>
#include <functional>
#include <mutex>
#include <queue>
#include <thread>
#include <vector>

namespace recml {

class ThreadPool {
 public:
  explicit ThreadPool(int threads);
  ~ThreadPool();
  void submit(std::function<void()> fn);
  void wait();  // until every submitted task has finished
  int size() const { return static_cast<int>(workers_.size()); }
  // Runs fn(begin, end, worker_slot) over a partition of [0, n); blocks until done.
  void parallel_for(long long n, const std::function<void(long long, long long, int)>& fn, long long min_chunk = 1);
  static ThreadPool& global();

 private:
  void loop();
  std::vector<std::thread> workers_;
  std::queue<std::function<void()>> tasks_;
  std::mutex mu_;
  std::condition_variable cv_, done_cv_;
  int pending_ = 0;
  bool stop_ = false;
};

}  // namespace recml
