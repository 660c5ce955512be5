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
  // While one of these lives the workers do not go to sleep between jobs: for a native routine that hands the
  // pool many short jobs with short serial steps between them (a tree, a boosting loop), where a sleeping
  // worker would miss most of the jobs.  Only for the length of one native call: the workers spin meanwhile.
  class Awake {
   public:
    explicit Awake(Pool& p) : p_(p) { p_.awake_.fetch_add(1, std::memory_order_relaxed); }
    ~Awake() { p_.awake_.fetch_sub(1, std::memory_order_relaxed); }
    Awake(const Awake&) = delete;
    Awake& operator=(const Awake&) = delete;
   private:
    Pool& p_;
  };
  // Runs fn(part, parts) on the caller and on whichever workers turn up before the caller has finished: for
  // jobs whose pieces are handed out from a shared counter, so that any subset of the threads completes
  // them.  Unlike run() it never waits for a sleeping worker to wake: on a busy or virtual machine that wait
  // can be longer than the whole job.
  void run_shared(const std::function<void(int, int)>& fn) {
    const int parts = size();
    if (parts == 1) { fn(0, 1); return; }
    fn_ = &fn;
    uint64_t mine;
    {
      std::lock_guard<std::mutex> lk(m_);
      mine = next_epoch(true);
    }
    if (sleepers_.load(std::memory_order_acquire) > 0) cv_.notify_all();
    fn(0, parts);
    closed_.store(mine, std::memory_order_seq_cst);
    for (int spins = 0; active_.load(std::memory_order_seq_cst) != 0; ++spins) {
      if (spins < 20000) _mm_pause();
      else std::this_thread::yield();
    }
  }
  // runs fn(part, parts) on every thread (the caller is part 0) and returns when all are done
  void run(const std::function<void(int, int)>& fn) {
    const int parts = size();
    if (parts == 1) { fn(0, 1); return; }
    fn_ = &fn;
    pending_.store(parts - 1, std::memory_order_relaxed);
    {
      std::lock_guard<std::mutex> lk(m_);        // pairs with the sleepers' predicate check
      next_epoch(false);
    }
    if (sleepers_.load(std::memory_order_acquire) > 0) cv_.notify_all();
    fn(0, parts);
    for (int spins = 0; pending_.load(std::memory_order_acquire) != 0; ++spins) {
      if (spins < 20000) _mm_pause();
      else std::this_thread::yield();
    }
  }

 private:
  // The job counter carries the kind of the job in its lowest bit (1: shared), so a worker reads both at once.
  uint64_t next_epoch(bool shared) {
    const uint64_t v = (((epoch_.load(std::memory_order_relaxed) >> 1) + 1) << 1) | (shared ? 1u : 0u);
    epoch_.store(v, std::memory_order_release);
    return v;
  }
  void loop(int id) {
    uint64_t seen = 0;
    for (;;) {
      int spins = 0;
      while (epoch_.load(std::memory_order_acquire) == seen && !quit_.load(std::memory_order_relaxed)) {
        if (++spins < 1500 || awake_.load(std::memory_order_relaxed) > 0) { _mm_pause(); continue; }
        std::unique_lock<std::mutex> lk(m_);
        sleepers_.fetch_add(1, std::memory_order_release);
        cv_.wait(lk, [&] { return quit_.load() || epoch_.load(std::memory_order_acquire) != seen; });
        sleepers_.fetch_sub(1, std::memory_order_release);
      }
      if (quit_.load(std::memory_order_relaxed)) return;
      seen = epoch_.load(std::memory_order_acquire);
      if (seen & 1) {
        // a shared job: join only while it is open.  The caller closes it when the work has run out and then
        // waits for the workers that are inside, so one that wakes late finds it closed and goes back to waiting.
        active_.fetch_add(1, std::memory_order_seq_cst);
        if (closed_.load(std::memory_order_seq_cst) < seen) (*fn_)(id, size());
        active_.fetch_sub(1, std::memory_order_seq_cst);
        continue;
      }
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
  std::atomic<int> active_{0};
  std::atomic<int> awake_{0};
  std::atomic<uint64_t> closed_{0};
  std::atomic<uint64_t> epoch_{0};
  std::atomic<bool> quit_{false};
};



// The pool, created on first use (one thread per hardware thread unless set_threads said otherwise),
// and the lock that serialises jobs.  Defined in cpu_quant.cc.
Pool& pool();
std::mutex& pool_mutex();
int set_threads(int n);

}  // namespace mimir_cpu
