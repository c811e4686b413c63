// runtime/include/brt/backends/cuda/providers/default/reduction/op_registration.h
#pragma once
namespace brt {
class KernelRegistry;
namespace cuda {
void RegisterReductionOps(KernelRegistry *registry);
} // namespace cuda
} // namespace brt
