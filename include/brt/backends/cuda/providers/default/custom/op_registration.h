// runtime/include/brt/backends/cuda/providers/default/custom/op_registration.h
#pragma once
namespace brt {
class KernelRegistry;
namespace cuda {
void RegisterCustomOps(KernelRegistry *registry);
} // namespace cuda
} // namespace brt
