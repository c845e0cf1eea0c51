// A small pool of host threads owned by a context, for the host-side part of result delivery
// (scattering a packed walk result into the caller's row matrix).  run(fn) calls fn(t, T) on every
// thread t of T and returns when all have finished.  Threads are created on first use and live until
// the context is destroyed.
#pragma once
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace skw {

class HostPool {
 public:
  explicit HostPool(int threads) : n_(threads < 1 ? 1 : threads) {
    for (int t = 1; t < n_; ++t) th_.emplace_back([this, t] { loop(t); });
  }
  ~HostPool() {
    {
      std::lock_guard<std::mutex> l(m_);
      stop_ = true;
      ++gen_;
    }
    cv_.notify_all();
    for (auto& t : th_) t.join();
  }
  int size() const { return n_; }
  void run(const std::function<void(int, int)>& fn) {
    {
      std::lock_guard<std::mutex> l(m_);
      job_ = &fn;
      pending_ = n_ - 1;
      ++gen_;
    }
    cv_.notify_all();
    fn(0, n_);  // the calling thread is thread 0
    std::unique_lock<std::mutex> l(m_);
    done_.wait(l, [this] { return pending_ == 0; });
    job_ = nullptr;
  }

 private:
  void loop(int t) {
    unsigned long long seen = 0;
    for (;;) {
      const std::function<void(int, int)>* job;
      {
        std::unique_lock<std::mutex> l(m_);
        cv_.wait(l, [&] { return gen_ != seen; });
        seen = gen_;
        if (stop_) return;
        job = job_;
      }
      (*job)(t, n_);
      {
        std::lock_guard<std::mutex> l(m_);
        if (--pending_ == 0) done_.notify_one();
      }
    }
  }
  int n_;
  std::vector<std::thread> th_;
  std::mutex m_;
  std::condition_variable cv_, done_;
  const std::function<void(int, int)>* job_ = nullptr;
  int pending_ = 0;
  unsigned long long gen_ = 0;
  bool stop_ = false;
};

}  // namespace skw
