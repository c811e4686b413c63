// Device layers: host allocator / provider, CUDA allocators, CUDA work queues.
#include "brt/backends/common.h"
#include "brt/backends/cpu/providers/default/cpu_provider.h"
#include "brt/backends/cuda/device/common/cuda_call.h"
#include "brt/backends/cuda/device/cuda_allocator.h"
#include "brt/backends/cuda/device/cuda_env.h"
#include "brt/backends/cuda/device/cuda_work_queue.h"
#include "brt/core/common/common.h"
#include "brt/core/session/session.h"

#include <cstdlib>

namespace brt {

// ---- host ------------------------------------------------------------------------
void *CPUAllocator::Alloc(size_t size) {
  void *p = nullptr;
  if (posix_memalign(&p, kAllocAlignment, size ? size : 1) != 0)
    return nullptr;
  return p;
}
void CPUAllocator::Free(void *p) { std::free(p); }

common::Status CPUAllocatorFactory(Session *session) {
  return session->AddAllocator(std::make_unique<CPUAllocator>());
}

CPUExecutionProvider::CPUExecutionProvider(const std::string &name) : ExecutionProvider(DeviceKind::CPU, name) {
  RegisterCommonBuiltinOps(kernel_registry_.get());
}

common::Status NaiveCPUExecutionProviderFactory(Session *session, int) {
  BRT_RETURN_IF_ERROR(CPUAllocatorFactory(session));
  return session->AddExecutionProvider(std::make_unique<CPUExecutionProvider>(ProviderType::BRT));
}

// ---- CUDA env / allocators ----------------------------------------------------------
namespace cuda {
void CudaEnv::Activate() const { BRT_CUDA_CHECK(cudaSetDevice(device_id_)); }
} // namespace cuda

void CUDAAllocator::SetDevice(bool throw_when_fail) const {
  cudaError_t e = cudaSetDevice(Info().id);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    if (throw_when_fail)
      BRT_THROW("cudaSetDevice(", Info().id, ") failed: ", cudaGetErrorString(e));
  }
}

void *CUDAAllocator::Alloc(size_t size) {
  SetDevice(true);
  void *p = nullptr;
  if (size > 0)
    BRT_CUDA_CHECK(cudaMalloc(&p, size));
  return p;
}

void CUDAAllocator::Free(void *p) {
  SetDevice(false);
  if (p)
    (void)cudaFree(p); // never throws: runs from destructors
}

void *CUDAPinnedAllocator::Alloc(size_t size) {
  void *p = nullptr;
  if (size > 0)
    BRT_CUDA_CHECK(cudaMallocHost(&p, size));
  return p;
}
void CUDAPinnedAllocator::Free(void *p) {
  if (p)
    (void)cudaFreeHost(p);
}

common::Status CUDAAllocatorFactory(Session *session, int device_id, bool /*use_arena*/, size_t /*size*/) {
  BRT_RETURN_IF_ERROR(session->AddAllocator(std::make_unique<CUDAAllocator>(device_id, CUDA)));
  return session->AddAllocator(std::make_unique<CUDAPinnedAllocator>(device_id, CUDA_PINNED));
}

common::Status CUDAExternalAllocatorFactory(Session *session, int device_id, void *alloc, void *free) {
  if (!alloc || !free)
    return common::Status(common::BRT, common::INVALID_ARGUMENT, "external allocator needs both functions");
  BRT_RETURN_IF_ERROR(session->AddAllocator(std::make_unique<CUDAExternalAllocator>(device_id, CUDA, alloc, free)));
  return session->AddAllocator(std::make_unique<CUDAPinnedAllocator>(device_id, CUDA_PINNED));
}

// ---- CUDA work queues ------------------------------------------------------------------
common::Status CUDAWorkQueue::AddTask(int task_type, const void *, void **args, int, const std::vector<int> &) {
  cudaMemcpyKind kind;
  switch (task_type) {
  case kH2D: kind = cudaMemcpyHostToDevice; break;
  case kD2H: kind = cudaMemcpyDeviceToHost; break;
  case kD2D: kind = cudaMemcpyDeviceToDevice; break;
  default:
    return common::Status(common::BRT, common::NOT_IMPLEMENTED,
                          "CUDAWorkQueue::AddTask: only copy tasks are routed through the queue; "
                          "kernels launch on GetComputeStream()");
  }
  env_.Activate();
  // the reference's convention (cuda_work_queue.cc:36-58): args = {&dst, &src, &bytes}
  void *dst = *static_cast<void **>(args[0]);
  void *src = *static_cast<void **>(args[1]);
  const size_t bytes = *static_cast<size_t *>(args[2]);
  return BRT_CUDA_CALL(cudaMemcpyAsync(dst, src, bytes, kind, reinterpret_cast<cudaStream_t>(GetComputeStream())));
}

common::Status CUDAWorkQueue::Sync() {
  env_.Activate();
  return BRT_CUDA_CALL(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(GetComputeStream())));
}

CUDASingleStreamWorkQueue::CUDASingleStreamWorkQueue(int device_id) : CUDAWorkQueue(cuda::CudaEnv(device_id)) {
  GetCudaEnv().Activate();
  cudaStream_t s;
  BRT_CUDA_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  stream_ = reinterpret_cast<CUstream_st *>(s);
}

CUDASingleStreamWorkQueue::~CUDASingleStreamWorkQueue() {
  if (stream_) {
    (void)cudaSetDevice(GetCudaEnv().GetDeviceID());
    (void)cudaStreamDestroy(reinterpret_cast<cudaStream_t>(stream_));
  }
}

namespace {
int CurrentDeviceOr(int device_id) {
  if (device_id >= 0)
    return device_id;
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess)
    (void)cudaGetLastError();
  return d;
}
} // namespace

CUDAExternalStreamWorkQueue::CUDAExternalStreamWorkQueue(CUstream_st *stream, int device_id)
    : CUDAWorkQueue(cuda::CudaEnv(CurrentDeviceOr(device_id)), "cuda_external_stream"), stream_(stream) {}

} // namespace brt
