// Host-side agreement of the per-GPU threads of the command-line driver before a collective:
// a thread that failed earlier must never leave its peers waiting inside an NCCL kernel, so each
// thread reports its status here and enters the collective only when every thread is present and
// healthy.  A thread that ends, for whatever reason, calls leave() and takes part in no later
// agreement.
#pragma once
#include <condition_variable>
#include <cstdint>
#include <mutex>

struct Rendezvous {
  std::mutex m;
  std::condition_variable cv;
  int ndev = 1, arrived = 0, gone = 0;
  uint64_t gen = 0;
  bool ok = true, outcome = true;
  void release() {  // caller holds m
    outcome = ok && gone == 0;
    arrived = 0;
    ok = true;
    ++gen;
    cv.notify_all();
  }
  bool agree(bool mine) {
    std::unique_lock<std::mutex> l(m);
    ok = ok && mine;
    const uint64_t g = gen;
    if (++arrived + gone >= ndev) {
      release();
      return outcome;
    }
    cv.wait(l, [&] { return gen != g; });
    return outcome;
  }
  void leave() {  // a thread that ends (for whatever reason) takes part in no later agreement
    std::lock_guard<std::mutex> l(m);
    ++gone;
    if (arrived && arrived + gone >= ndev) release();
  }
};
