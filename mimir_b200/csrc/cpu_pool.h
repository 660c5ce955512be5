// Worker pool shared by the host kernels of the library (quantized products, fused elementwise
// programs): rows or blocks of one job are handed to the workers, the caller takes part.
#pragma once
#include <immintrin.h>
#include <pthread.h>

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <mutex>
#include <new>
#include <thread>
#include <vector>

namespace mimir_cpu {

// Workers spin briefly on the job counter before they sleep, so the back-to-back products of a
// decode step are picked up in well under a microsecond; after some tens of microseconds without work they block
// on a condition variable and cost nothing.
class Pool {
 public:
  explicit Pool(int n) {
    for (int i = 1; i < n; ++i) workers_.emplace_back([this, i] { loop(i); });
  }
  ~Pool() {
    {
      std::lock_guard<std::mutex> lk(m_);
      quit_.store(true);
    }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
  }
  int size() const { return static_cast<int>(workers_.size()) + 1; }
  // While a Hot object lives the workers keep spinning between jobs instead of going to sleep: for a
  // caller that hands over many short jobs with serial work of its own in between (a tree grower), where
  // waking a sleeper would cost more than the job.
  class Hot {
   public:
    explicit Hot(Pool& p) : p_(p) { p_.hot_.fetch_add(1, std::memory_order_relaxed); }
    ~Hot() { p_.hot_.fetch_sub(1, std::memory_order_relaxed); }
    Hot(const Hot&) = delete;
    Hot& operator=(const Hot&) = delete;

   private:
    Pool& p_;
  };
  // runs fn(part, parts) on every thread (the caller is part 0) and returns when all are done
  void run(const std::function<void(int, int)>& fn) {
    const int parts = size();
    if (parts == 1) { fn(0, 1); return; }
    fn_ = &fn;
    pending_.store(parts - 1, std::memory_order_relaxed);
    {
      std::lock_guard<std::mutex> lk(m_);        // pairs with the sleepers' predicate check
      epoch_.fetch_add(1, std::memory_order_release);
    }
    if (sleepers_.load(std::memory_order_acquire) > 0) cv_.notify_all();
    fn(0, parts);
    for (int spins = 0; pending_.load(std::memory_order_acquire) != 0; ++spins) {
      if (spins < 20000) _mm_pause();
      else std::this_thread::yield();
    }
  }

 private:
  void loop(int id) {
    uint64_t seen = 0;
    for (;;) {
      int spins = 0;
      while (epoch_.load(std::memory_order_acquire) == seen && !quit_.load(std::memory_order_relaxed)) {
        if (++spins < 1500 || hot_.load(std::memory_order_relaxed) > 0) { _mm_pause(); continue; }
        std::unique_lock<std::mutex> lk(m_);
        sleepers_.fetch_add(1, std::memory_order_release);
        cv_.wait(lk, [&] { return quit_.load() || epoch_.load(std::memory_order_acquire) != seen; });
        sleepers_.fetch_sub(1, std::memory_order_release);
      }
      if (quit_.load(std::memory_order_relaxed)) return;
      seen = epoch_.load(std::memory_order_acquire);
      (*fn_)(id, size());
      pending_.fetch_sub(1, std::memory_order_release);
    }
  }
  std::vector<std::thread> workers_;
  std::mutex m_;
  std::condition_variable cv_;
  const std::function<void(int, int)>* fn_ = nullptr;
  std::atomic<int> pending_{0};
  std::atomic<int> sleepers_{0};
  std::atomic<int> hot_{0};
  std::atomic<uint64_t> epoch_{0};
  std::atomic<bool> quit_{false};
};



// The pool, created on first use (one thread per hardware thread unless set_threads said otherwise),
// and the lock that serialises jobs.  Defined in cpu_quant.cc.
Pool& pool();
std::mutex& pool_mutex();
int set_threads(int n);

}  // namespace mimir_cpu
