// runtime/include/brt/backends/cuda/providers/default/tensor_generate/op_registration.h
#pragma once
namespace brt {
class KernelRegistry;
namespace cuda {
void RegisterTensorGenerateOps(KernelRegistry *registry); // FillOp (the rng ops are not part of this provider)
} // namespace cuda
} // namespace brt
