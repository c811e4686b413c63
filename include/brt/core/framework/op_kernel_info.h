// Everything a kernel is built from: which op, whose provider, which allocators
// (runtime/include/brt/core/framework/op_kernel_info.h).  The operation is this
// runtime's own ir::Operation instead of an mlir::Operation.
#pragma once

#include "brt/core/framework/value.h"
#include "brt/core/ir/ir.h"
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

namespace brt {
class ExecutionProvider;
class IAllocator;

class OpKernelInfo {
public:
  using AllocatorMap = std::unordered_map<std::string, std::unique_ptr<IAllocator>>;

  OpKernelInfo(const ExecutionProvider &provider, const ir::ByREHandle &handle, const ir::Operation *op,
               int op_id, const AllocatorMap &allocators, IAllocator *last_allocator,
               const std::vector<AsyncValue> &weights, size_t intermediate_begin,
               const std::string &ir_path, const std::vector<int> &dependency)
      : provider_(provider), handle_(handle), op_(op), op_id_(op_id), allocators_(allocators),
        last_allocator_(last_allocator), weights_(weights), intermediate_begin_(intermediate_begin),
        ir_path_(ir_path), dependency_(dependency) {}
  OpKernelInfo(const OpKernelInfo &) = default;

  const ExecutionProvider &GetExecutionProvider() const { return provider_; }
  const ir::ByREHandle &GetIRHandle() const { return handle_; }
  const ir::Operation *GetOperation() const { return op_; }
  int GetOpId() const { return op_id_; }
  const std::vector<AsyncValue> &GetWeights() const { return weights_; }
  const std::vector<int> &GetDependency() const { return dependency_; }
  IAllocator *GetAllocator(const std::string &key) const {
    auto it = allocators_.find(key);
    return it == allocators_.end() ? nullptr : it->second.get();
  }
  // the allocator of the memory space of the op's last operand (execution_plan.cc:327-347)
  IAllocator *GetAllocator() const { return last_allocator_; }
  const std::string &GetIRPath() const { return ir_path_; }
  std::string GetByREOpName() const { return op_->callee; }
  bool IsIntermediateArg(size_t idx) const;

private:
  const ExecutionProvider &provider_;
  const ir::ByREHandle &handle_;
  const ir::Operation *op_;
  int op_id_;
  const AllocatorMap &allocators_;
  IAllocator *last_allocator_;
  const std::vector<AsyncValue> &weights_;
  size_t intermediate_begin_;
  const std::string &ir_path_;
  std::vector<int> dependency_;
  OpKernelInfo &operator=(const OpKernelInfo &) = delete;
};

// tensor index (= ir::Value id) of the op's i-th operand; results follow the operands
size_t GetTensorIndexFromOpArgIndex(const OpKernelInfo &, unsigned int i);
unsigned int GetOpArgNum(const OpKernelInfo &);
unsigned int GetOpResultNum(const OpKernelInfo &);

inline bool OpKernelInfo::IsIntermediateArg(size_t idx) const {
  return GetTensorIndexFromOpArgIndex(*this, (unsigned)idx) >= intermediate_begin_;
}

} // namespace brt
