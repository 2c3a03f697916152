// Basic value types shared by every layer of the communicator core.
//
// Parity: the reference keeps these in comms/torchcomms/TorchCommTypes.hpp
// (ReduceOp, timeouts, InitHandle) and comms/torchcomms/TorchCommHooks.hpp:28-52
// (the operation-name enum).
#pragma once

// The extension is built with hidden visibility; what an out-of-tree backend
// library derives from or calls is exported explicitly.
#define B200C_API __attribute__((visibility("default")))

#include <ATen/ATen.h>
#include <chrono>
#include <cstdint>
#include <optional>
#include <string>
#include <string_view>
#include <unordered_map>
#include <variant>
#include <vector>

namespace b200c {

using Millis = std::chrono::milliseconds;
using Hints = std::unordered_map<std::string, std::string>;
using InitHandle = std::string;

// 600 s matches the reference's default collective timeout; 0 disables the
// watchdog deadline for an operation.
constexpr Millis kDefaultTimeout{600 * 1000};
constexpr Millis kNoTimeout{0};

enum class RedOpType : uint8_t {
  SUM = 0,
  PRODUCT,
  MIN,
  MAX,
  BAND,
  BOR,
  BXOR,
  PREMUL_SUM,
  AVG,
};

const char* red_op_name(RedOpType t);

// A reduction operator. PREMUL_SUM carries its factor either as a host double
// or as a one-element tensor living on the communicator's device.
class B200C_API ReduceOp {
 public:
  using Factor = std::variant<double, at::Tensor>;

  /*implicit*/ ReduceOp(RedOpType t = RedOpType::SUM) : type_(t) {}
  static ReduceOp premul_sum(Factor f) {
    ReduceOp op(RedOpType::PREMUL_SUM);
    op.factor_ = std::move(f);
    return op;
  }

  RedOpType type() const { return type_; }
  const std::optional<Factor>& factor() const { return factor_; }
  bool has_tensor_factor() const {
    return factor_ && std::holds_alternative<at::Tensor>(*factor_);
  }
  // Host value of the factor (synchronises if the factor is a device tensor).
  double factor_as_double() const;
  bool operator==(const ReduceOp& o) const { return type_ == o.type_; }
  bool operator==(RedOpType t) const { return type_ == t; }

 private:
  RedOpType type_;
  std::optional<Factor> factor_;
};

enum class WorkStatus : uint8_t {
  NOT_STARTED = 0,
  INPROGRESS,
  COMPLETED,
  TIMEDOUT,
  ERROR,
};

const char* work_status_name(WorkStatus s);

// Operation names as seen by hooks, the flight recorder and the text log.
enum class OpName : uint8_t {
  send = 0,
  recv,
  broadcast,
  all_reduce,
  reduce,
  all_gather,
  all_gather_v,
  all_gather_single,
  reduce_scatter,
  reduce_scatter_v,
  reduce_scatter_single,
  all_to_all_single,
  all_to_all_v_single,
  all_to_all,
  barrier,
  scatter,
  gather,
  gather_single,
  split,
  new_window,
  batch_op_issue,
  finalize,
  kCount,
};

std::string_view op_name(OpName op);

enum class P2PKind : uint8_t { SEND = 0, RECV = 1 };

struct P2POp {
  P2PKind kind;
  at::Tensor tensor;
  int peer;
};

// Window access classes: UNIFIED means load/store reachable (NVLink peer or
// self), SEPARATE means a network hop would be needed.
enum class WinAccessType : uint8_t { UNIFIED = 0, SEPARATE = 1 };

struct WindowAttr {
  WinAccessType access_type = WinAccessType::UNIFIED;
};

} // namespace b200c
