// Status / StatusCode, with the reference's names and meaning
// (runtime/include/brt/core/common/status.h:29-162).
#pragma once

#include <memory>
#include <ostream>
#include <string>

namespace brt {
namespace common {

enum StatusCategory { NONE = 0, SYSTEM = 1, BRT = 2 };

enum StatusCode {
  OK = 0,
  FAIL = 1,
  INVALID_ARGUMENT = 2,
  NO_SUCHFILE = 3,
  NO_MODEL = 4,
  ENGINE_ERROR = 5,
  RUNTIME_EXCEPTION = 6,
  INVALID_PROTOBUF = 7,
  MODEL_LOADED = 8,
  NOT_IMPLEMENTED = 9,
  INVALID_GRAPH = 10,
  EP_FAIL = 11
};

class Status {
public:
  Status() noexcept = default;
  Status(StatusCategory category, int code, const std::string &msg)
      : state_(new State{category, code, msg}) {}
  Status(StatusCategory category, int code, const char *msg)
      : state_(new State{category, code, msg ? msg : ""}) {}
  Status(StatusCategory category, int code) : Status(category, code, "") {}
  Status(const Status &other)
      : state_(other.state_ ? new State(*other.state_) : nullptr) {}
  Status &operator=(const Status &other) {
    if (this != &other)
      state_.reset(other.state_ ? new State(*other.state_) : nullptr);
    return *this;
  }
  Status(Status &&) noexcept = default;
  Status &operator=(Status &&) noexcept = default;

  bool IsOK() const noexcept { return state_ == nullptr; }
  int Code() const noexcept { return state_ ? state_->code : static_cast<int>(common::OK); }
  StatusCategory Category() const noexcept { return state_ ? state_->category : common::NONE; }
  const std::string &ErrorMessage() const noexcept {
    static const std::string empty;
    return state_ ? state_->msg : empty;
  }
  std::string ToString() const;

  bool operator==(const Status &o) const {
    return IsOK() == o.IsOK() && Code() == o.Code() && Category() == o.Category();
  }
  bool operator!=(const Status &o) const { return !(*this == o); }

  static Status OK() { return Status(); }

private:
  struct State {
    StatusCategory category;
    int code;
    std::string msg;
  };
  std::unique_ptr<State> state_;
};

inline std::ostream &operator<<(std::ostream &out, const Status &status) {
  return out << status.ToString();
}

} // namespace common
} // namespace brt

#define BRT_RETURN_IF_ERROR(expr)                                              \
  do {                                                                         \
    auto _status = (expr);                                                     \
    if (!_status.IsOK())                                                       \
      return _status;                                                          \
  } while (0)
