// Host work queue that runs every task inline
// (runtime/include/brt/backends/cpu/device/cpu_work_queue.h: CPUNaiveWorkQueue).
#pragma once

#include "brt/core/context/work_queue.h"

namespace brt {
namespace cpu {

class CPUNaiveWorkQueue : public WorkQueue {
public:
  explicit CPUNaiveWorkQueue(const std::string &name = "cpu_naive") : WorkQueue(name) {}
  common::Status AddTask(int, const void *func, void **, int, const std::vector<int> &) override {
    (*reinterpret_cast<const std::function<void(void)> *>(func))();
    return common::Status::OK();
  }
  common::Status AddHostTask(const void *task, void **, int, const std::vector<int> &) override {
    (*reinterpret_cast<const std::function<void(void)> *>(task))();
    return common::Status::OK();
  }
  common::Status Sync() override { return common::Status::OK(); }
};

} // namespace cpu
} // namespace brt
