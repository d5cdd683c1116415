// CPU unit test of the bounded host wait the library uses while a communicator exists (lantern_b200/csrc/comm_wait.h).
// Built and run by tests/test_failure_detection.py.  Prints one line per case; exit code 0 when all hold.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <thread>

#include "../lantern_b200/csrc/comm_wait.h"

using namespace ltb;
using clk = std::chrono::steady_clock;

static long ms_since(clk::time_point t0) { return (long)std::chrono::duration_cast<std::chrono::milliseconds>(clk::now() - t0).count(); }

int main() {
  int bad = 0;
  auto expect = [&](const char* what, bool ok) { std::printf("%s %s\n", ok ? "ok  " : "FAIL", what); if (!ok) ++bad; };

  {  // work that is already finished: done at the first poll, failed() is never consulted
    int asked = 0;
    int r = bounded_wait([] { return true; }, [&] { ++asked; return true; }, 100);
    expect("finished work returns WAIT_DONE without looking at the error state", r == WAIT_DONE && asked == 0);
  }
  {  // work that finishes after a while (another thread sets the flag), well inside the limit
    std::atomic<bool> flag{false};
    std::thread t([&] { std::this_thread::sleep_for(std::chrono::milliseconds(30)); flag = true; });
    auto t0 = clk::now();
    int r = bounded_wait([&] { return flag.load(); }, [] { return false; }, 5000);
    t.join();
    expect("work that finishes in time returns WAIT_DONE", r == WAIT_DONE && ms_since(t0) < 2000);
  }
  {  // the transport reports an error while the work is pending
    std::atomic<int> polls{0};
    auto t0 = clk::now();
    int r = bounded_wait([] { return false; }, [&] { return ++polls > 50; }, 5000);
    expect("an asynchronous error ends the wait at once with WAIT_FAILED", r == WAIT_FAILED && ms_since(t0) < 2000);
  }
  {  // nothing ever happens: the deadline ends the wait
    auto t0 = clk::now();
    int r = bounded_wait([] { return false; }, [] { return false; }, 200);
    const long waited = ms_since(t0);
    expect("a wait on work that never finishes returns WAIT_TIMEOUT at the deadline", r == WAIT_TIMEOUT && waited >= 200 && waited < 2000);
  }
  {  // work that completes exactly as the deadline passes is not reported lost (done() is asked once more)
    const auto t0 = clk::now();
    int r = bounded_wait([&] { return ms_since(t0) >= 100; }, [] { return false; }, 100);
    expect("work finished by the deadline counts as done", r == WAIT_DONE);
  }
  {  // no limit: waits as long as it takes
    std::atomic<bool> flag{false};
    std::thread t([&] { std::this_thread::sleep_for(std::chrono::milliseconds(150)); flag = true; });
    int r = bounded_wait([&] { return flag.load(); }, [] { return false; }, 0);
    t.join();
    expect("timeout 0 waits without limit", r == WAIT_DONE);
  }
  return bad ? 1 : 0;
}
