// KernelRegistry and static registration
// (runtime/include/brt/core/framework/kernel_registry.h:27-94).
#pragma once

#include "brt/core/common/common.h"
#include "brt/core/framework/op_kernel.h"
#include "brt/core/framework/op_kernel_info.h"
#include <memory>
#include <unordered_map>

namespace brt {

using KernelCreateFn = std::function<std::shared_ptr<brt::OpKernel>(const brt::OpKernelInfo &)>;

class KernelRegistry {
public:
  KernelRegistry() = default;
  // the first registration of a key wins
  common::Status Register(const std::string &key, KernelCreateFn func) {
    kernel_creator_fn_map_.emplace(key, func);
    return common::Status::OK();
  }
  bool HasKernel(const std::string &key) { return kernel_creator_fn_map_.count(key) != 0; }
  std::shared_ptr<OpKernel> operator()(const std::string &key, const OpKernelInfo &info) {
    auto it = kernel_creator_fn_map_.find(key);
    return it == kernel_creator_fn_map_.end() ? nullptr : (it->second)(info);
  }
  const std::unordered_map<std::string, KernelCreateFn> &GetInternalMap() { return kernel_creator_fn_map_; }

private:
  std::unordered_map<std::string, KernelCreateFn> kernel_creator_fn_map_;
};

using KernelRegistration = std::function<void(KernelRegistry *)>;

// replays every registration recorded for (deviceKind, providerName) into kernelReg
void RegisterKernels(const std::string &deviceKind, const std::string &providerName, KernelRegistry *kernelReg);
void AddKernelRegistration(const std::string &deviceKind, const std::string &providerName,
                           KernelRegistration registration);
// AliasOp and friends that every provider carries (kernel_registry.cc:77-96)
void RegisterCommonBuiltinOps(KernelRegistry *registry);

} // namespace brt

#define BRT_STATIC_KERNEL_REGISTRATION(KIND, PROVIDER, FUNC)                   \
  BRT_STATIC_KERNEL_REGISTRATION_(KIND, PROVIDER, FUNC, __COUNTER__)
#define BRT_STATIC_KERNEL_REGISTRATION_(KIND, PROVIDER, FUNC, N)               \
  BRT_STATIC_KERNEL_REGISTRATION__(KIND, PROVIDER, FUNC, N)
#define BRT_STATIC_KERNEL_REGISTRATION__(KIND, PROVIDER, FUNC, N)              \
  [[gnu::unused]] static bool __kernel_registration_##N = [] {                 \
    ::brt::AddKernelRegistration(KIND, PROVIDER, FUNC);                        \
    return true;                                                               \
  }();
