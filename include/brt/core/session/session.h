// Session: holds one loaded model, its providers and allocators
// (runtime/include/brt/core/session/session.h:50-163).
#pragma once

#include "brt/core/common/status.h"
#include "brt/core/framework/dtype.h"
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

namespace brt {

class ExecutionPlan;
class StaticBRTExecutionPlan;
class ExecutionProvider;
class IAllocator;
class RequestContext;
class WorkQueue;
class DistributedBackend;
namespace ir {
class ByREHandle;
}

class Session {
public:
  Session();
  virtual ~Session();

  // Load a ByRE model from a file.  fmt: "byre".
  common::Status Load(const std::string &url, const std::string &fmt);
  // Load a ByRE model from a NUL-terminated text buffer.  fmt: "byre".
  common::Status LoadFromMemory(const void *ptr, const std::string &fmt);
  // ByRE text or bytecode held in memory (the reference hands over an mlir::ModuleOp instead)
  common::Status LoadFromBuffer(const void *data, size_t size);

  void *GetWeightAsyncValue(size_t offset);
  common::Status LoadWeights(const std::string &url, const std::string &fmt);

  // request_ctx takes ownership of work_queue if it is not nullptr
  common::Status NewRequestContext(std::unique_ptr<RequestContext> *request_ctx, WorkQueue *work_queue = nullptr);

  int GetGraphArgOffset(const std::string &name);
  common::Status Run(RequestContext &request_ctx);
  void Cleanup(RequestContext &request_ctx) noexcept;

  size_t GetArgNum();
  size_t GetWeightNum();
  const std::vector<std::string> &GetWeightNames();
  const std::vector<std::string> &GetInputNames();
  const std::vector<std::string> &GetOutputNames();
  const std::vector<size_t> &GetWeightArgOffsets();
  const std::vector<size_t> &GetInputArgOffsets();
  const std::vector<size_t> &GetOutputArgOffsets();
  const std::vector<int64_t> GetStaticShape(size_t id);
  DTypeEnum GetDType(size_t id);
  std::string GetSpace(size_t id);

  common::Status AddExecutionProvider(std::unique_ptr<ExecutionProvider> provider);
  common::Status AddAllocator(std::unique_ptr<IAllocator> allocator);
  IAllocator *GetAllocator(const std::string &key);

protected:
  common::Status BuildPlan(const std::string &ir_path);

  std::vector<std::unique_ptr<ExecutionProvider>> exec_providers_;
  std::unordered_map<std::string, std::unique_ptr<IAllocator>> allocators_;
  std::unique_ptr<StaticBRTExecutionPlan> execution_plan_;
  std::unique_ptr<ir::ByREHandle> ir_handle_;

  // the communicator Run hands to the kernels; set by a DistributedSession, null otherwise
  DistributedBackend *distributed_backend_ = nullptr;

  std::vector<std::string> weight_names_, input_names_, output_names_;
  std::vector<size_t> weight_offsets_, input_offsets_, output_offsets_;
};

} // namespace brt
