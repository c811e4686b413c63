// ExecutionProvider: a named set of kernels for one device kind
// (runtime/include/brt/core/framework/execution_provider.h:29-116).
#pragma once

#include "brt/core/common/status.h"
#include "brt/core/framework/allocator.h"
#include "brt/core/framework/kernel_registry.h"
#include <string>

namespace brt {

struct ProviderOptions {};

class ExecutionProvider {
protected:
  ExecutionProvider(const std::string &deviceKind, const std::string &name)
      : deviceKind_{deviceKind}, name_{name} {
    kernel_registry_ = std::make_unique<KernelRegistry>();
    RegisterKernels(deviceKind_, name_, kernel_registry_.get());
  }

public:
  virtual ~ExecutionProvider() = default;
  void SetKernelRegistry(std::unique_ptr<KernelRegistry> kernels) { kernel_registry_ = std::move(kernels); }
  KernelRegistry *GetKernelRegistry() const { return kernel_registry_.get(); }
  const std::string &DeviceKind() const { return deviceKind_; }
  const std::string &Name() const { return name_; }

  // dlopen(RTLD_LAZY | RTLD_GLOBAL) a library whose static initialisers call
  // BRT_STATIC_KERNEL_REGISTRATION; must happen before the provider is created
  static common::Status StaticRegisterKernelsFromDynlib(const std::string &path);

protected:
  const std::string deviceKind_;
  const std::string name_;
  std::unique_ptr<KernelRegistry> kernel_registry_;

private:
  ExecutionProvider(const ExecutionProvider &) = delete;
  ExecutionProvider &operator=(const ExecutionProvider &) = delete;
};

} // namespace brt
