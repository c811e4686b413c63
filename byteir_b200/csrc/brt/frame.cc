// ExecutionFrame (runtime/lib/core/context/execution_frame.cc).
#include "brt/core/common/common.h"
#include "brt/core/context/execution_frame.h"

namespace brt {

void *ExecutionFrame::StateInfo::CreateStateIfNotExist(const std::string &key, const std::function<void *()> &creator,
                                                      Deleter deleter) {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = states_.find(key);
  if (it != states_.end())
    return it->second.ptr;
  void *p = creator();
  states_[key] = Entry{p, std::move(deleter)};
  return p;
}
bool ExecutionFrame::StateInfo::HasState(const std::string &key) const {
  std::lock_guard<std::mutex> lock(mu_);
  return states_.count(key) != 0;
}
void *ExecutionFrame::StateInfo::GetState(const std::string &key) const {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = states_.find(key);
  return it == states_.end() ? nullptr : it->second.ptr;
}
void *ExecutionFrame::StateInfo::RemoveState(const std::string &key) {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = states_.find(key);
  if (it == states_.end())
    return nullptr;
  void *p = it->second.ptr;
  states_.erase(it);
  return p;
}
ExecutionFrame::StateInfo::~StateInfo() {
  for (auto &kv : states_)
    if (kv.second.deleter && kv.second.ptr)
      kv.second.deleter(kv.second.ptr);
}

ExecutionFrame::ExecutionFrame(const ConstructInfo &info)
    : info_(info), args_(info.args.size()), intermediates_(info.allocators.size(), nullptr) {}

ExecutionFrame::~ExecutionFrame() {
  for (size_t i = 0; i < args_.size(); ++i) {
    auto &a = args_[i];
    if (a.ptr && (a.owned || a.ownership == BrtOwnershipType::OwnedByRuntime)) {
      IAllocator *alloc = info_.allocators[info_.args[i].allocator];
      if (alloc)
        alloc->Free(a.ptr);
    }
  }
  for (size_t k = 0; k < intermediates_.size(); ++k)
    if (intermediates_[k])
      info_.allocators[k]->Free(intermediates_[k]);
}

common::Status ExecutionFrame::BindArg(size_t offset, const void *value, BrtOwnershipType ownership) {
  if (offset >= args_.size())
    return common::Status(common::BRT, common::INVALID_ARGUMENT, "BindArg: offset out of range");
  if (info_.args[offset].is_weight)
    return common::Status(common::BRT, common::INVALID_ARGUMENT, "BindArg: weights are bound by the session");
  if (ownership == BrtOwnershipType::CopiedByRuntime)
    return common::Status(common::BRT, common::NOT_IMPLEMENTED,
                          "BindArg: CopiedByRuntime needs a device copy; copy into GetArg(offset) instead");
  auto &a = args_[offset];
  if (a.ptr && (a.owned || a.ownership == BrtOwnershipType::OwnedByRuntime)) {
    info_.allocators[info_.args[offset].allocator]->Free(a.ptr);
  }
  a.ptr = const_cast<void *>(value);
  a.ownership = ownership;
  a.owned = false;
  return common::Status::OK();
}

void *ExecutionFrame::GetArg(size_t offset) {
  BRT_ENFORCE(offset < args_.size(), "GetArg: offset out of range");
  if (info_.args[offset].is_weight)
    return info_.weights[offset];
  auto &a = args_[offset];
  if (!a.ptr) {
    IAllocator *alloc = info_.allocators[info_.args[offset].allocator];
    BRT_ENFORCE(alloc, "no allocator for the memory space of arg ", offset);
    const size_t bytes = info_.args[offset].bytes;
    a.ptr = alloc->Alloc(bytes ? bytes : 1);
    BRT_ENFORCE(a.ptr, "allocation of arg ", offset, " (", bytes, " bytes) failed");
    a.owned = true;
  }
  return a.ptr;
}

void ExecutionFrame::FinishIOBinding() {
  for (size_t i = 0; i < args_.size(); ++i)
    (void)GetArg(i);
}

common::Status ExecutionFrame::AllocIntermediate() {
  if (intermediates_allocated_)
    return common::Status::OK();
  for (size_t k = 0; k < intermediates_.size(); ++k) {
    const size_t bytes = info_.intermediate_bytes[k];
    if (bytes == 0)
      continue;
    intermediates_[k] = info_.allocators[k]->Alloc(bytes);
    if (!intermediates_[k])
      return common::Status(common::BRT, common::FAIL, "allocation of the intermediates failed");
  }
  intermediates_allocated_ = true;
  return common::Status::OK();
}

AsyncValueRef ExecutionFrame::GetAsyncValueRef(size_t tensor_index) {
  BRT_ENFORCE(tensor_index < info_.tensors.size(), "tensor index out of range");
  const auto &loc = info_.tensors[tensor_index];
  switch (loc.kind) {
  case ConstructInfo::TensorLoc::kArg:
    return GetArg((size_t)loc.index);
  case ConstructInfo::TensorLoc::kIntermediate:
    BRT_ENFORCE(intermediates_allocated_, "intermediates are not allocated yet");
    return static_cast<char *>(intermediates_[loc.index]) + loc.offset;
  default:
    return static_cast<char *>(GetAsyncValueRef((size_t)loc.index)) + loc.offset;
  }
}

} // namespace brt
