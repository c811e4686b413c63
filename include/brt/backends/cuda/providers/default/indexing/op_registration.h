// runtime/include/brt/backends/cuda/providers/default/indexing/op_registration.h
#pragma once
namespace brt {
class KernelRegistry;
namespace cuda {
void RegisterIndexingOps(KernelRegistry *registry);
} // namespace cuda
} // namespace brt
