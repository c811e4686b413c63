// What a collective runs on (runtime/include/brt/core/distributed/d_context.h:16-21): a CUDA stream for
// device buffers (CudaContext, brt/backends/nccl/device/d_context_nccl.h), nothing for host buffers.
#pragma once

#include <string>

namespace brt {

class DContext {
public:
  virtual std::string type() const = 0;
  virtual ~DContext() = default;
};

// buffers in host memory: the collective completes before the call returns
class HostContext final : public DContext {
public:
  std::string type() const override { return "BRT_CTX_HOST"; }
};

} // namespace brt
