// The exchange step of the hot path through the plug-in boundary: the nccl.AllReduce op kernel, the two
// communicators it can run on, and the per-rank session.
#include "brt/backends/common.h"
#include "brt/backends/cuda/device/common/cuda_call.h"
#include "brt/backends/cuda/device/cuda_work_queue.h"
#include "brt/backends/nccl/device/d_context_nccl.h"
#include "brt/backends/nccl/device/distributed_backend_b200.h"
#include "brt/backends/nccl/providers/op_registration.h"
#include "brt/core/common/common.h"
#include "brt/core/context/execution_frame.h"
#include "brt/core/distributed/distributed_session.h"
#include "brt/core/framework/kernel_registry.h"
#include "brt/core/framework/op_accessor.h"
#include "brt/core/framework/op_kernel.h"
#include "brt/core/framework/op_kernel_impl_base.h"

#include "b200_kernels.h"

#include <cuda_runtime.h>

namespace brt {

using common::Status;

namespace {
Status Fail(const std::string &msg) { return Status(common::StatusCategory::BRT, common::StatusCode::FAIL, msg); }

int KernelDType(DTypeEnum dt) {
  switch (dt) {
  case DTypeEnum::Float32: return B200_F32;
  case DTypeEnum::Float16: return B200_F16;
  case DTypeEnum::BFloat16: return B200_BF16;
  default: return -1;
  }
}

bool IsWholeWorld(const std::set<int64_t> &group, uint32_t nranks) {
  if (group.empty())
    return true;
  if (group.size() != nranks)
    return false;
  int64_t want = 0;
  for (int64_t r : group) // a set iterates in ascending order
    if (r != want++)
      return false;
  return true;
}

CUstream_st *StreamOf(const std::shared_ptr<DContext> &ctx) {
  auto *cuda = dynamic_cast<CudaContext *>(ctx.get());
  return cuda ? cuda->get_stream() : nullptr;
}
} // namespace

// ---- communicators ----------------------------------------------------------------------------------
Status DistributedBackendCallback::all_reduce(const void *sendbuff, void *recvbuff, size_t len, DTypeEnum dtype,
                                              ReduceOp op, std::set<int64_t> replica_group,
                                              std::shared_ptr<DContext> ctx) {
  if (!fn_)
    return Fail("the all-reduce callback is not set");
  std::vector<int64_t> group(replica_group.begin(), replica_group.end());
  const int rc = fn_(user_, sendbuff, recvbuff, (uint64_t)len, (int)dtype, (int)op, group.data(),
                     (uint64_t)group.size(), StreamOf(ctx));
  if (rc != 0)
    return Fail("the all-reduce callback failed with code " + std::to_string(rc));
  return Status::OK();
}

Status DistributedBackendPeer::Launch(const float *send, void *recv, size_t len, DTypeEnum out_dtype,
                                      const std::set<int64_t> &group, const std::shared_ptr<DContext> &ctx) {
  if (!IsWholeWorld(group, m_nranks))
    return Fail("the peer-memory all-reduce runs over all ranks: replica_group must name every rank");
  if (len != capacity_)
    return Fail("the peer-memory all-reduce was set up for " + std::to_string(capacity_) + " elements, got " +
                std::to_string(len));
  const int kdt = KernelDType(out_dtype);
  if (kdt < 0)
    return Fail(std::string("the peer-memory all-reduce delivers f32, f16 or bf16, not ") + DTypeName(out_dtype));
  auto *cuda = dynamic_cast<CudaContext *>(ctx.get());
  if (!cuda)
    return Fail("the peer-memory all-reduce needs a CUDA stream");
  const int rc = b200_sharded_sum_finish(kdt, send, inbox_.data(), flags_.data(), (int)m_rank, (int)m_nranks,
                                         (int64_t)len, epoch_counter_, recv, status_,
                                         reinterpret_cast<cudaStream_t>(cuda->get_stream()));
  if (rc != B200_OK)
    return Fail(std::string("b200_sharded_sum_finish: ") + b200_error_string(rc));
  return Status::OK();
}

Status DistributedBackendPeer::all_reduce(const void *sendbuff, void *recvbuff, size_t len, DTypeEnum dtype,
                                          ReduceOp op, std::set<int64_t> replica_group,
                                          std::shared_ptr<DContext> ctx) {
  if (dtype != DTypeEnum::Float32 || op != BRT_SUM)
    return Fail("the peer-memory all-reduce sums f32 vectors");
  return Launch(static_cast<const float *>(sendbuff), recvbuff, len, DTypeEnum::Float32, replica_group, ctx);
}

Status DistributedBackendPeer::all_reduce_sum_f32_rounded(const float *sendbuff, void *recvbuff, size_t len,
                                                          DTypeEnum out_dtype, std::set<int64_t> replica_group,
                                                          std::shared_ptr<DContext> ctx) {
  return Launch(sendbuff, recvbuff, len, out_dtype, replica_group, ctx);
}

// ---- per-rank session ---------------------------------------------------------------------------------
DistributedSession::DistributedSession(int rank, int nranks, const std::string &host, int port)
    : Session(), rank_(rank), nranks_(nranks), host_(host), port_(port) {
  BRT_ENFORCE(nranks > 0 && rank >= 0 && rank < nranks, "rank ", rank, " is not one of ", nranks, " ranks");
}

DistributedSession::~DistributedSession() = default;

Status DistributedSession::LoadConfig(const std::vector<std::string> &config, std::string &ir_url) {
  if ((size_t)rank_ >= config.size())
    return Status(common::StatusCategory::BRT, common::StatusCode::INVALID_ARGUMENT,
                  "no module for rank " + std::to_string(rank_) + " in a config of " + std::to_string(config.size()));
  ir_url = config[rank_];
  return Status::OK();
}

// ---- byre.compute @nccl.AllReduce ------------------------------------------------------------------------
// (runtime/lib/backends/nccl/providers/all_reduce.cc:44-69)  operand 0 -> operand 1, attributes `reduction`
// ("sum" / "max" / "min") and `replica_group` (ranks).  Source and target have the same shape and, as in
// the reference, the same element type; in addition an f32 source may go to an f16 / bf16 target, which is
// rounded once after the sum (the all-reduce of unrounded partial sums followed by the cast, as one op).
// The op runs wherever its buffers live: on the request's CUDA stream for "cuda" memrefs, at once for
// "cpu" memrefs.
namespace cuda {
namespace {
class AllReduce final : public OpKernel {
public:
  explicit AllReduce(const OpKernelInfo &info)
      : OpKernel(info, false, false, /*prologue_per_frame=*/true, /*epilogue_per_frame=*/true) {
    OpAccessor accessor(info_);
    BRT_ENFORCE(accessor.GetNumArgs() == 2, "nccl.AllReduce takes a source and a target");
    len_ = (size_t)OpAccessor::GetNumElementsOfShape(accessor.GetArgShape(0));
    BRT_ENFORCE((size_t)OpAccessor::GetNumElementsOfShape(accessor.GetArgShape(1)) == len_,
                "nccl.AllReduce: source and target differ in size");
    src_dtype_ = accessor.GetArgDTypeEnum(0);
    dst_dtype_ = accessor.GetArgDTypeEnum(1);
    const std::string reduction = accessor.GetAttrAsString("reduction");
    op_ = GetReduceOp(reduction);
    BRT_ENFORCE(op_ != BRT_REDUCEOP_COUNT, "nccl.AllReduce: unknown reduction '", reduction, "'");
    for (int64_t r : accessor.GetAttrAsIntArray("replica_group"))
      group_.insert(r);
    rounded_ = src_dtype_ != dst_dtype_;
    if (rounded_)
      BRT_ENFORCE(src_dtype_ == DTypeEnum::Float32 && op_ == BRT_SUM &&
                      (dst_dtype_ == DTypeEnum::Float16 || dst_dtype_ == DTypeEnum::BFloat16),
                  "nccl.AllReduce: source and target element types differ (only an f32 sum may be "
                  "delivered as f16 or bf16)");
    on_device_ = accessor.GetArgSpace(0) != "cpu";
    BRT_ENFORCE((accessor.GetArgSpace(1) != "cpu") == on_device_, "nccl.AllReduce: source and target live in different spaces");
    uid_ = accessor.GetUID();
  }

  // an f32 scratch vector for the rounded form on a backend that cannot fuse the cast
  Status ProloguePerFrame(const ExecutionContext &ctx) override {
    if (!rounded_ || !on_device_)
      return Status::OK();
    IAllocator *allocator = info_.GetAllocator();
    auto *states = static_cast<ExecutionFrame::StateInfo *>(ctx.frame_state_info);
    bool failed = false;
    states->CreateStateIfNotExist(
        uid_,
        [&]() -> void * {
          auto *ws = new ::brt::detail::WorkspaceState();
          ws->bytes = len_ * sizeof(float);
          ws->allocator = allocator;
          ws->ptr = allocator ? allocator->Alloc(ws->bytes) : nullptr;
          failed = ws->ptr == nullptr;
          return ws;
        },
        [](void *p) {
          auto *ws = static_cast<::brt::detail::WorkspaceState *>(p);
          if (ws->ptr && ws->allocator)
            ws->allocator->Free(ws->ptr);
          delete ws;
        });
    return failed ? Fail("workspace allocation failed for " + uid_) : Status::OK();
  }

  Status EpiloguePerFrame(const ExecutionContext &ctx) override {
    auto *states = static_cast<ExecutionFrame::StateInfo *>(ctx.frame_state_info);
    if (void *p = states->RemoveState(uid_)) {
      auto *ws = static_cast<::brt::detail::WorkspaceState *>(p);
      if (ws->ptr && ws->allocator)
        ws->allocator->Free(ws->ptr);
      delete ws;
    }
    return Status::OK();
  }

  Status RunImpl(const ExecutionContext &ctx) override {
    DistributedBackend *backend = ctx.distributed_backend;
    if (!backend)
      return Fail("nccl.AllReduce needs a communicator: run the module in a DistributedSession with "
                  "SetDistributedBackend");
    OpAccessor accessor(info_, ctx.exec_frame);
    const void *src = accessor.GetArgAsyncValueRef(0);
    void *dst = accessor.GetArgAsyncValueRef(1);
    std::shared_ptr<DContext> dctx;
    cudaStream_t stream = nullptr;
    if (on_device_) {
      auto *wq = dynamic_cast<CUDAWorkQueue *>(ctx.work_queue);
      if (!wq)
        return Fail("nccl.AllReduce on device memory needs a CUDA work queue on the request");
      wq->GetCudaEnv().Activate();
      stream = reinterpret_cast<cudaStream_t>(wq->GetComputeStream());
      dctx = std::make_shared<CudaContext>(wq->GetComputeStream());
    } else {
      dctx = std::make_shared<HostContext>();
    }
    if (!rounded_)
      return backend->all_reduce(src, dst, len_, src_dtype_, op_, group_, dctx);
    if (!on_device_)
      return Status(common::StatusCategory::BRT, common::StatusCode::NOT_IMPLEMENTED,
                    "nccl.AllReduce with a narrower target is implemented for device memory only");
    Status fused = backend->all_reduce_sum_f32_rounded(static_cast<const float *>(src), dst, len_, dst_dtype_, group_, dctx);
    if (fused.IsOK() || fused.Code() != common::StatusCode::NOT_IMPLEMENTED)
      return fused;
    auto *states = static_cast<ExecutionFrame::StateInfo *>(ctx.frame_state_info);
    auto *ws = static_cast<::brt::detail::WorkspaceState *>(states->GetState(uid_));
    if (!ws || !ws->ptr)
      return Fail("no workspace state for " + uid_ + " (ProloguePerFrame did not run)");
    BRT_RETURN_IF_ERROR(backend->all_reduce(src, ws->ptr, len_, DTypeEnum::Float32, BRT_SUM, group_, dctx));
    const int rc = b200_cast_from_f32(KernelDType(dst_dtype_), static_cast<const float *>(ws->ptr), dst, (int64_t)len_, stream);
    return rc == B200_OK ? Status::OK() : Fail(std::string("b200_cast_from_f32: ") + b200_error_string(rc));
  }

private:
  size_t len_;
  DTypeEnum src_dtype_, dst_dtype_;
  ReduceOp op_;
  std::set<int64_t> group_;
  bool rounded_, on_device_;
  std::string uid_;
};
} // namespace

void RegisterNCCLOps(KernelRegistry *registry) {
  registry->Register("nccl.AllReduce", [](const OpKernelInfo &info) -> std::shared_ptr<OpKernel> {
    return std::make_shared<AllReduce>(info);
  });
}
} // namespace cuda

namespace {
// the collective is an op of the CUDA provider and, for host-space memrefs, of the host provider
BRT_STATIC_KERNEL_REGISTRATION(DeviceKind::CUDA, ProviderType::BRT,
                               [](KernelRegistry *registry) { cuda::RegisterNCCLOps(registry); })
BRT_STATIC_KERNEL_REGISTRATION(DeviceKind::CPU, ProviderType::BRT,
                               [](KernelRegistry *registry) { cuda::RegisterNCCLOps(registry); })
} // namespace

} // namespace brt
