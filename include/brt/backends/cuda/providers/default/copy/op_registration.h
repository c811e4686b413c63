// runtime/include/brt/backends/cuda/providers/default/copy/op_registration.h
#pragma once
namespace brt {
class KernelRegistry;
namespace cuda {
void RegisterCopyOps(KernelRegistry *registry); // cpu2cuda, cuda2cpu, cuda2cuda
} // namespace cuda
} // namespace brt
