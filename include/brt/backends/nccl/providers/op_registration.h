// runtime/include/brt/backends/nccl/providers/op_registration.h
#pragma once

namespace brt {
class KernelRegistry;
namespace cuda {
// "nccl.AllReduce" (the collective of the hot path; the reference also registers nccl.Send / Recv /
// AllGather / Broadcast, runtime/lib/backends/nccl/providers/op_registration.cc:31-56)
void RegisterNCCLOps(KernelRegistry *registry);
} // namespace cuda
} // namespace brt
