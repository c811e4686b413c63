// Wrappers that turn an Impl class into a CUDA OpKernel
// (runtime/include/brt/backends/cuda/device/utils/op_kernel_impl_helpers.h:29-218).
//
//   struct Impl {
//     explicit Impl(const OpAccessor &);                 // shapes / attributes, may throw
//     Status-or-void Execute(operands..., [void *workspace,] cudaStream_t);
//     size_t GetWorkspaceSize(const ExecutionContext &); // WithWorkspace only
//   };
//   using MyOp = CudaOpKernel<Impl, TypedOperand<const float *, 0>, TypedOperand<float *, 1>>;
//
// The wrapper makes the queue's device current, fetches the operand addresses
// from the frame, passes the queue's compute stream, and checks
// cudaGetLastError() after Execute.  A workspace is allocated once per frame
// from the allocator of the op's last operand, kept in the frame state under the
// op's UID, and freed when the frame goes away.
#pragma once

#include "brt/backends/cuda/device/common/cuda_call.h"
#include "brt/backends/cuda/device/cuda_work_queue.h"
#include "brt/core/context/execution_frame.h"
#include "brt/core/framework/op_accessor.h"
#include "brt/core/framework/op_kernel.h"
#include "brt/core/framework/op_kernel_impl_base.h"
#include <type_traits>

namespace brt {
namespace cuda {

namespace detail {
template <typename F> common::Status CallToStatus(F &&f) {
  if constexpr (std::is_void_v<decltype(f())>) {
    f();
    return common::Status::OK();
  } else {
    return f();
  }
}
inline cudaStream_t StreamOf(const ExecutionContext &ctx) {
  auto *wq = dynamic_cast<CUDAWorkQueue *>(ctx.work_queue);
  BRT_ENFORCE(wq, "a CUDA op needs a CUDA work queue on the request");
  wq->GetCudaEnv().Activate();
  return reinterpret_cast<cudaStream_t>(wq->GetComputeStream());
}
} // namespace detail

template <typename Impl, typename... Operands> class CudaOpKernel final : public OpKernel {
public:
  explicit CudaOpKernel(const OpKernelInfo &info) : OpKernel(info), impl_(OpAccessor(info_)) {}

  common::Status RunImpl(const ExecutionContext &ctx) override {
    OpAccessor accessor(info_, ctx.exec_frame);
    cudaStream_t stream = detail::StreamOf(ctx);
    BRT_RETURN_IF_ERROR(detail::CallToStatus([&] { return impl_.Execute(Operands::Get(accessor)..., stream); }));
    return BRT_CUDA_CALL(cudaGetLastError());
  }

private:
  Impl impl_;
};

template <typename Impl, typename... Operands> class CudaOpKernelWithWorkspace final : public OpKernel {
public:
  explicit CudaOpKernelWithWorkspace(const OpKernelInfo &info)
      : OpKernel(info, false, false, /*prologue_per_frame=*/true, /*epilogue_per_frame=*/true),
        impl_(OpAccessor(info_)), uid_(OpAccessor(info_).GetUID()) {}

  common::Status ProloguePerFrame(const ExecutionContext &ctx) override {
    const size_t bytes = impl_.GetWorkspaceSize(ctx);
    IAllocator *allocator = info_.GetAllocator();
    auto *states = static_cast<ExecutionFrame::StateInfo *>(ctx.frame_state_info);
    bool failed = false;
    states->CreateStateIfNotExist(
        uid_,
        [&]() -> void * {
          auto *ws = new ::brt::detail::WorkspaceState();
          ws->bytes = bytes;
          ws->allocator = allocator;
          if (bytes > 0) {
            ws->ptr = allocator ? allocator->Alloc(bytes) : nullptr;
            failed = ws->ptr == nullptr;
          }
          return ws;
        },
        [](void *p) {
          auto *ws = static_cast<::brt::detail::WorkspaceState *>(p);
          if (ws->ptr && ws->allocator)
            ws->allocator->Free(ws->ptr);
          delete ws;
        });
    if (failed)
      return common::Status(common::StatusCategory::BRT, common::StatusCode::FAIL,
                            "workspace allocation failed for " + uid_);
    return common::Status::OK();
  }

  common::Status EpiloguePerFrame(const ExecutionContext &ctx) override {
    auto *states = static_cast<ExecutionFrame::StateInfo *>(ctx.frame_state_info);
    if (void *p = states->RemoveState(uid_)) {
      auto *ws = static_cast<::brt::detail::WorkspaceState *>(p);
      if (ws->ptr && ws->allocator)
        ws->allocator->Free(ws->ptr);
      delete ws;
    }
    return common::Status::OK();
  }

  common::Status RunImpl(const ExecutionContext &ctx) override {
    OpAccessor accessor(info_, ctx.exec_frame);
    auto *states = static_cast<ExecutionFrame::StateInfo *>(ctx.frame_state_info);
    auto *ws = static_cast<::brt::detail::WorkspaceState *>(states->GetState(uid_));
    if (!ws)
      return common::Status(common::StatusCategory::BRT, common::StatusCode::FAIL,
                            "no workspace state for " + uid_ + " (ProloguePerFrame did not run)");
    cudaStream_t stream = detail::StreamOf(ctx);
    BRT_RETURN_IF_ERROR(
        detail::CallToStatus([&] { return impl_.Execute(Operands::Get(accessor)..., ws->ptr, stream); }));
    return BRT_CUDA_CALL(cudaGetLastError());
  }

private:
  Impl impl_;
  std::string uid_;
};

} // namespace cuda
} // namespace brt
