// Asynchronous operation handle.
//
// Every collective returns a Work. `wait()` orders the caller's execution
// context after the operation (a stream dependency on CUDA, a host block on
// CPU); `wait_blocking()` always blocks the host. Four lifecycle hook lists
// (start, end, wait-pre, wait-post) let recorders follow an operation without
// polling; a hook registered after its state was reached fires at once.
//
// Parity: comms/torchcomms/TorchWork.hpp:31-235, TorchWork.cpp:11-60.
#pragma once

#include <c10/util/intrusive_ptr.h>

#include <atomic>
#include <functional>
#include <future>
#include <mutex>

#include "types.hpp"

namespace b200c {

class B200C_API Work : public c10::intrusive_ptr_target {
 public:
  using Hook = std::function<void()>;

  Work() = default;
  ~Work() override = default;
  Work(const Work&) = delete;
  Work& operator=(const Work&) = delete;

  WorkStatus status() const { return status_.load(std::memory_order_acquire); }
  bool is_completed() const { return status() == WorkStatus::COMPLETED; }

  // Orders the caller after the operation. Never blocks the host on CUDA.
  void wait();
  // Blocks the calling host thread until the operation finished.
  void wait_blocking();

  Millis timeout() const { return timeout_; }
  void set_timeout(Millis t) { timeout_ = t; }

  void on_start(Hook h);
  void on_end(Hook h);
  void on_wait_pre(Hook h);
  void on_wait_post(Hook h);

  // Public so that tests and Python-implemented backends can drive the state
  // machine; transitions into INPROGRESS fire start hooks, transitions into a
  // terminal state fire end hooks exactly once.
  void set_status(WorkStatus s);

  // Error text for ERROR / TIMEDOUT states.
  std::string error() const;
  void set_error(std::string msg);

 protected:
  virtual void do_wait() = 0;
  virtual void do_wait_blocking() { do_wait(); }

 private:
  void fire(std::vector<Hook>& hooks);

  std::atomic<WorkStatus> status_{WorkStatus::NOT_STARTED};
  Millis timeout_{kDefaultTimeout};
  mutable std::mutex mu_;
  bool started_ = false;
  bool ended_ = false;
  std::vector<Hook> start_hooks_, end_hooks_, wait_pre_hooks_, wait_post_hooks_;
  std::string error_;
};

using WorkPtr = c10::intrusive_ptr<Work>;

// A handle for an operation that already finished on the host.
class B200C_API CompletedWork final : public Work {
 public:
  CompletedWork() { set_status(WorkStatus::COMPLETED); }

 protected:
  void do_wait() override {}
};

// Runs a callable on a helper thread; used by CPU backends for async_op=True.
class B200C_API ThreadWork final : public Work {
 public:
  explicit ThreadWork(std::function<void()> fn, Millis timeout);
  ~ThreadWork() override;

 protected:
  void do_wait() override;

 private:
  std::future<void> fut_;
};

} // namespace b200c
