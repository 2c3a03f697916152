// Hook plumbing: what an observer sees before and after each operation.
//
// One record type describes every operation; which fields are meaningful
// depends on `op` (the Python layer presents per-operation typed views such
// as AllReducePreHookArgs built from this record).
//
// Parity: comms/torchcomms/TorchCommHooks.hpp:28-491 (per-op typed args in
// std::variant, PreHook/PostHook/AbortHook/GraphReplayHook signatures) and
// comms/torchcomms/RemovableHandle.hpp:9-41.
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <mutex>

#include "work.hpp"

namespace b200c {

struct OpRecord {
  OpName op = OpName::barrier;
  std::vector<at::Tensor> inputs;   // tensors read by the operation
  std::vector<at::Tensor> outputs;  // tensors written by the operation
  bool in_place = false;            // inputs[0] is also the output
  int root = -1;                    // root (rooted collectives) or peer (p2p)
  bool async_op = false;
  std::optional<RedOpType> red_op;
  std::vector<int64_t> in_splits, out_splits;
  std::vector<P2POp> p2p_ops;       // batch_op_issue
  std::vector<int> ranks;           // split
  std::string name;                 // split
  c10::weak_intrusive_ptr<Work> work{c10::intrusive_ptr<Work>()}; // post hooks only
};

using PreHook = std::function<void(OpName, size_t /*op_id*/, const OpRecord&)>;
using PostHook = std::function<void(size_t /*op_id*/, const OpRecord&)>;
using AbortHook = std::function<void()>;
// (graph_id, replay_id, stream handle, collective index inside the graph,
//  'S' when the collective started or 'E' when it ended)
using GraphReplayHook =
    std::function<void(uint64_t, uint64_t, uintptr_t, size_t, char)>;

// Unregisters a hook when `remove()` is called; safe to call repeatedly.
class RemovableHandle {
 public:
  RemovableHandle() = default;
  explicit RemovableHandle(std::function<void()> remover)
      : remover_(std::make_shared<std::function<void()>>(std::move(remover))) {}
  void remove() {
    if (remover_ && *remover_) {
      auto fn = std::move(*remover_);
      *remover_ = nullptr;
      fn();
    }
  }

 private:
  std::shared_ptr<std::function<void()>> remover_;
};

// Ordered table of callbacks keyed by a registration id.
template <typename Fn>
class HookTable : public std::enable_shared_from_this<HookTable<Fn>> {
 public:
  RemovableHandle add(Fn fn) {
    std::lock_guard<std::mutex> g(mu_);
    const uint64_t id = next_++;
    fns_.emplace(id, std::move(fn));
    std::weak_ptr<HookTable<Fn>> weak = this->shared_from_this();
    return RemovableHandle([weak, id]() {
      if (auto self = weak.lock()) {
        std::lock_guard<std::mutex> g2(self->mu_);
        self->fns_.erase(id);
      }
    });
  }
  std::vector<Fn> snapshot() const {
    std::lock_guard<std::mutex> g(mu_);
    std::vector<Fn> out;
    out.reserve(fns_.size());
    for (auto& kv : fns_) {
      out.push_back(kv.second);
    }
    return out;
  }
  bool empty() const {
    std::lock_guard<std::mutex> g(mu_);
    return fns_.empty();
  }

 private:
  mutable std::mutex mu_;
  uint64_t next_ = 0;
  std::map<uint64_t, Fn> fns_;
};

} // namespace b200c
