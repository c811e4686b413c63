// runtime/include/brt/backends/cuda/providers/default/tensor_manipulate/op_registration.h
#pragma once
namespace brt {
class KernelRegistry;
namespace cuda {
void RegisterTensorManipulateOps(KernelRegistry *registry);
} // namespace cuda
} // namespace brt
