// A kernel plug-in as a maintainer of the reference would write it: an Impl class with the contract of
// reduction/reduce_impl.h, wrapped by CudaOpKernelWithWorkspace, registered with
// BRT_STATIC_KERNEL_REGISTRATION, and calling the C ABI of libb200_kernels.so.  It is registered under a key
// of its own ("PluginReduceSumOp_f16_f16"), since KernelRegistry::Register is first-wins and the built-in
// key is taken in this runtime.
#include "b200_kernels.h"
#include "brt/backends/common.h"
#include "brt/backends/cuda/device/utils/op_kernel_impl_helpers.h"
#include "brt/core/framework/kernel_registry.h"

#include <algorithm>
#include <cuda_fp16.h>

namespace {
class B200ReduceSumF16 {
public:
  explicit B200ReduceSumF16(const brt::OpAccessor &a) {
    auto shape = a.GetArgShape(0);
    std::vector<int64_t> dims = a.GetAttrAsIntArray("dimensions");
    std::sort(dims.begin(), dims.end());
    BRT_ENFORCE(!dims.empty(), "dimensions must not be empty");
    for (size_t i = 1; i < dims.size(); ++i)
      BRT_ENFORCE(dims[i] == dims[i - 1] + 1, "Only consecutive dimensions reduction is supported");
    A = B = C = 1;
    for (int64_t i = 0; i < dims.front(); ++i)
      A *= shape[i];
    for (int64_t d : dims)
      B *= shape[d];
    for (size_t i = dims.back() + 1; i < shape.size(); ++i)
      C *= shape[i];
  }
  brt::common::Status Execute(const __half *in, __half *out, void *workspace, cudaStream_t stream) {
    const int rc = b200_reduce(B200_REDUCE_SUM, B200_F16, in, out, A, B, C, workspace,
                               b200_reduce_workspace_bytes(B200_REDUCE_SUM, B200_F16, A, B, C), stream);
    if (rc != B200_OK)
      return brt::common::Status(brt::common::StatusCategory::BRT, brt::common::StatusCode::FAIL, b200_error_string(rc));
    return brt::common::Status::OK();
  }
  size_t GetWorkspaceSize(const brt::ExecutionContext &) const {
    return b200_reduce_workspace_bytes(B200_REDUCE_SUM, B200_F16, A, B, C);
  }
  int64_t A, B, C;
};
using Kernel = brt::cuda::CudaOpKernelWithWorkspace<B200ReduceSumF16, brt::TypedOperand<const __half *, 0>,
                                                    brt::TypedOperand<__half *, 1>>;
} // namespace

BRT_STATIC_KERNEL_REGISTRATION(brt::DeviceKind::CUDA, brt::ProviderType::BRT, [](brt::KernelRegistry *r) {
  r->Register("PluginReduceSumOp_f16_f16", [](const brt::OpKernelInfo &info) -> std::shared_ptr<brt::OpKernel> {
    return std::make_shared<Kernel>(info);
  });
});
