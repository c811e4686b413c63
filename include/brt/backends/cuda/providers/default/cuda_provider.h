// The default CUDA execution provider
// (runtime/include/brt/backends/cuda/providers/default/cuda_provider.h;
// runtime/lib/backends/cuda/providers/default/cuda_provider.cc:46-74).
#pragma once

#include "brt/core/framework/execution_provider.h"

namespace brt {
class Session;

class CUDAExecutionProvider : public ExecutionProvider {
public:
  explicit CUDAExecutionProvider(const std::string &name);
};

common::Status DefaultCUDAExecutionProviderFactory(Session *session);

} // namespace brt
