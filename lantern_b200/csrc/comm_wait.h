// Bounded host-side wait for work that a peer may never let finish (a collective whose partner rank has left).
// Plain host code, no CUDA: the library polls a stream with it (comm.cu), the CPU tests poll flags.
#pragma once
#include <chrono>
#include <cstdint>
#include <thread>

namespace ltb {

enum { WAIT_DONE = 0, WAIT_FAILED = 1, WAIT_TIMEOUT = 2 };

// Polls done() until it is true (WAIT_DONE), failed() is true (WAIT_FAILED: the transport reported an asynchronous error) or
// timeout_ms have passed (WAIT_TIMEOUT; timeout_ms <= 0 waits without limit).  The first polls spin, later ones sleep
// poll_us microseconds so that a long legitimate wait does not burn a core.  done() is checked before failed(), and once
// more after the deadline, so work that finished in time is never reported as lost.
template <class Done, class Failed>
int bounded_wait(Done done, Failed failed, int64_t timeout_ms, int poll_us = 50) {
  const auto t0 = std::chrono::steady_clock::now();
  for (int64_t polls = 0;; ++polls) {
    if (done()) return WAIT_DONE;
    if (failed()) return WAIT_FAILED;
    if (timeout_ms > 0) {
      const auto waited = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
      if (waited >= timeout_ms) return done() ? WAIT_DONE : WAIT_TIMEOUT;
    }
    if (polls > 200) std::this_thread::sleep_for(std::chrono::microseconds(poll_us));
  }
}

}  // namespace ltb
