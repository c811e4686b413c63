// Host-side events fired around a plan run and around every op
// (runtime/include/brt/core/framework/event.h:27-74).
#pragma once

#include <functional>
#include <vector>

namespace brt {
class OpKernelInfo;

namespace Events {
struct BeforeExecutionPlanRun {};
struct AfterExecutionPlanRun {};
struct BeforeOpKernelRun {
  const OpKernelInfo &info;
};
struct AfterOpKernelRun {
  const OpKernelInfo &info;
};
template <typename T> using Listener = std::function<void(const T &)>;
} // namespace Events

class EventListenerManager {
public:
  template <typename T> void AddEventListener(Events::Listener<T> &&l) { Slot<T>().push_back(std::move(l)); }
  template <typename T> void SignalEvent(const T &e) {
    for (auto &l : Slot<T>())
      l(e);
  }

private:
  template <typename T> std::vector<Events::Listener<T>> &Slot();
  std::vector<Events::Listener<Events::BeforeExecutionPlanRun>> before_plan_;
  std::vector<Events::Listener<Events::AfterExecutionPlanRun>> after_plan_;
  std::vector<Events::Listener<Events::BeforeOpKernelRun>> before_op_;
  std::vector<Events::Listener<Events::AfterOpKernelRun>> after_op_;
};

template <>
inline std::vector<Events::Listener<Events::BeforeExecutionPlanRun>> &
EventListenerManager::Slot<Events::BeforeExecutionPlanRun>() { return before_plan_; }
template <>
inline std::vector<Events::Listener<Events::AfterExecutionPlanRun>> &
EventListenerManager::Slot<Events::AfterExecutionPlanRun>() { return after_plan_; }
template <>
inline std::vector<Events::Listener<Events::BeforeOpKernelRun>> &
EventListenerManager::Slot<Events::BeforeOpKernelRun>() { return before_op_; }
template <>
inline std::vector<Events::Listener<Events::AfterOpKernelRun>> &
EventListenerManager::Slot<Events::AfterOpKernelRun>() { return after_op_; }

} // namespace brt
