// WorkQueue: where op kernels enqueue their work
// (runtime/include/brt/core/context/work_queue.h).
#pragma once

#include "brt/core/common/status.h"
#include <functional>
#include <string>
#include <vector>

namespace brt {

class WorkQueue {
public:
  explicit WorkQueue(const std::string &name) : name_(name) {}
  virtual ~WorkQueue() = default;
  const std::string &name() const { return name_; }

  // enqueue a device task described by (task_type, func, args); see the CUDA queues
  virtual common::Status AddTask(int task_type, const void *func, void **args, int op_id,
                                 const std::vector<int> &dependency) = 0;
  // `task` points to a std::function<void(void)>
  virtual common::Status AddHostTask(const void *task, void **args, int op_id,
                                     const std::vector<int> &dependency) = 0;
  common::Status AddTask(std::function<common::Status()> enqueue_functor) { return enqueue_functor(); }
  virtual common::Status Sync() = 0;

private:
  const std::string name_;
  WorkQueue(const WorkQueue &) = delete;
  WorkQueue &operator=(const WorkQueue &) = delete;
};

} // namespace brt
