// Host execution provider (runtime/include/brt/backends/cpu/providers/default/
// cpu_provider.h).  It carries only what kernels register for
// (DeviceKind::CPU, ProviderType::BRT) plus the built-in AliasOp; the reference's
// LLVM-JIT op is not part of this runtime.
#pragma once

#include "brt/core/framework/execution_provider.h"

namespace brt {
class Session;

class CPUExecutionProvider : public ExecutionProvider {
public:
  explicit CPUExecutionProvider(const std::string &name);
};

common::Status NaiveCPUExecutionProviderFactory(Session *session, int intra_op_num_threads = 1);

} // namespace brt
