// ExecutionFrame: the storage behind one RequestContext
// (runtime/include/brt/core/context/execution_frame.h).  It owns or borrows the
// buffers of the entry-function arguments, owns one block per allocator for the
// planned intermediates, and keeps per-frame kernel state (workspaces).
#pragma once

#include "brt/core/common/status.h"
#include "brt/core/framework/allocator.h"
#include "brt/core/framework/memory_info.h"
#include "brt/core/framework/value.h"
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace brt {

class ExecutionFrame {
public:
  // Per-frame state created by kernels (e.g. a workspace), keyed by the op's UID.
  // (execution_frame.h:99-159: StateInfo)
  class StateInfo {
  public:
    using Deleter = std::function<void(void *)>;
    // returns the existing state or creates it with `creator`
    void *CreateStateIfNotExist(const std::string &key, const std::function<void *()> &creator,
                                Deleter deleter = nullptr);
    bool HasState(const std::string &key) const;
    void *GetState(const std::string &key) const;
    // removes the entry and returns its pointer without running the deleter
    void *RemoveState(const std::string &key);
    ~StateInfo();

  private:
    struct Entry {
      void *ptr;
      Deleter deleter;
    };
    mutable std::mutex mu_;
    std::map<std::string, Entry> states_;
  };

  // what the execution plan computed for this model
  struct ConstructInfo {
    struct Arg {
      size_t bytes;
      int allocator;   // index into allocators
      bool is_weight;
    };
    std::vector<Arg> args;
    // tensor index -> (kind, index/base, byte offset)
    struct TensorLoc {
      enum Kind { kArg, kIntermediate, kAlias } kind;
      int index;      // arg index, allocator index, or aliased tensor index
      size_t offset;  // byte offset inside the allocator block / the aliased tensor
    };
    std::vector<TensorLoc> tensors;
    std::vector<size_t> intermediate_bytes; // per allocator
    std::vector<IAllocator *> allocators;
    std::vector<void *> weights;            // per arg: session-owned weight buffer or nullptr
  };

  explicit ExecutionFrame(const ConstructInfo &info);
  virtual ~ExecutionFrame();

  // bind the arg at `offset` (position in the entry function's argument list)
  common::Status BindArg(size_t offset, const void *value, BrtOwnershipType ownership);
  // address of the arg, allocating it from its allocator if nothing is bound yet
  void *GetArg(size_t offset);
  // allocate every arg that is still unbound
  void FinishIOBinding();
  // allocate the intermediates (once per frame)
  common::Status AllocIntermediate();

  AsyncValueRef GetAsyncValueRef(size_t tensor_index);
  AsyncValue GetAsyncValue(size_t tensor_index) { return GetAsyncValueRef(tensor_index); }

  StateInfo &GetStateInfo() { return state_info_; }
  const ConstructInfo &GetInfo() const { return info_; }
  bool IsPrologued() const { return prologued_; }
  void SetPrologued() { prologued_ = true; }

private:
  struct ArgSlot {
    void *ptr = nullptr;
    BrtOwnershipType ownership = BrtOwnershipType::OwnedByExternal;
    bool owned = false; // allocated by this frame
  };
  ConstructInfo info_;
  std::vector<ArgSlot> args_;
  std::vector<void *> intermediates_;
  bool intermediates_allocated_ = false;
  bool prologued_ = false;
  StateInfo state_info_;
};

using BRTInferenceExecutionFrame = ExecutionFrame;

} // namespace brt
