// StaticBRTExecutionPlan: built once when a module is loaded.  It numbers the
// tensors, picks a kernel for every ByRE op, and lays the intermediates out
// (runtime/lib/core/framework/execution_plan.cc:62-691).
#pragma once

#include "brt/core/common/status.h"
#include "brt/core/context/execution_context.h"
#include "brt/core/context/execution_frame.h"
#include "brt/core/framework/op_kernel.h"
#include "brt/core/ir/ir.h"
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

namespace brt {
class ExecutionProvider;
class IAllocator;
class WorkQueue;

class ExecutionPlan {
public:
  virtual ~ExecutionPlan() = default;
  using AllocatorMap = std::unordered_map<std::string, std::unique_ptr<IAllocator>>;
  virtual common::Status ProloguePerSession(const AllocatorMap &allocators,
                                            const std::vector<std::unique_ptr<ExecutionProvider>> &providers) = 0;
  virtual common::Status EpiloguePerSession() = 0;
  virtual common::Status ProloguePerFrame(const ExecutionContext &) = 0;
  virtual common::Status EpiloguePerFrame(const ExecutionContext &) = 0;
  virtual common::Status Run(const ExecutionContext &) = 0;
  virtual void CreateExecutinFrame(std::unique_ptr<ExecutionFrame> *frame) = 0;
  virtual void CreateWorkQueue(std::unique_ptr<WorkQueue> *wq, int rank = 0) = 0;
};

class StaticBRTExecutionPlan final : public ExecutionPlan {
public:
  explicit StaticBRTExecutionPlan(const ir::ByREHandle &handle, const std::string &ir_path = "");
  ~StaticBRTExecutionPlan() override;

  common::Status ProloguePerSession(const AllocatorMap &allocators,
                                    const std::vector<std::unique_ptr<ExecutionProvider>> &providers) override;
  common::Status EpiloguePerSession() override;
  common::Status ProloguePerFrame(const ExecutionContext &) override;
  common::Status EpiloguePerFrame(const ExecutionContext &) override;
  common::Status Run(const ExecutionContext &) override;
  void CreateExecutinFrame(std::unique_ptr<ExecutionFrame> *frame) override;
  void CreateWorkQueue(std::unique_ptr<WorkQueue> *wq, int rank = 0) override;

  // graph metadata, by position in the entry function's argument list
  struct ArgInfo {
    std::string name;
    int argtype; // ir::ArgType bits
    ir::MemRefType type;
  };
  const std::vector<ArgInfo> &GetArgs() const { return args_; }
  const std::vector<std::shared_ptr<OpKernel>> &GetKernels() const { return kernels_; }
  void *GetWeight(size_t arg_offset) const { return frame_info_.weights[arg_offset]; }

private:
  const ir::ByREHandle &handle_;
  std::string ir_path_;
  std::vector<ArgInfo> args_;
  std::vector<std::shared_ptr<OpKernel>> kernels_;
  std::vector<std::unique_ptr<OpKernelInfo>> infos_;
  ExecutionFrame::ConstructInfo frame_info_;
  std::vector<AsyncValue> weights_;
  std::vector<std::pair<IAllocator *, void *>> owned_weights_;
  bool uses_cuda_ = false; // some value of the entry function lives in device memory
};

} // namespace brt
