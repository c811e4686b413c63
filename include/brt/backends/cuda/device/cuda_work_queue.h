// CUDA work queues (runtime/include/brt/backends/cuda/device/cuda_work_queue.h).
// The kernels of this provider launch directly on GetComputeStream().
#pragma once

#include "brt/backends/cuda/device/cuda_env.h"
#include "brt/core/context/work_queue.h"

struct CUstream_st;

namespace brt {

// task types AddTask understands (cuda_work_queue.h: CUDATaskType)
enum CUDATaskType : int { kCompute = 0, kH2D = 1, kD2H = 2, kRecordEvent = 3, kWaitEvent = 4, kComputeDrv = 5, kD2D = 6 };

class CUDAWorkQueue : public WorkQueue {
public:
  explicit CUDAWorkQueue(cuda::CudaEnv env, const std::string &name = "cuda_default_stream")
      : WorkQueue(name), env_(env) {}
  // kH2D / kD2H / kD2D: args = {&dst, &src, &bytes} (void **, void **, size_t *); other types are not
  // used by this provider's kernels and return NOT_IMPLEMENTED
  common::Status AddTask(int task_type, const void *func, void **args, int op_id,
                         const std::vector<int> &dependency) override;
  common::Status AddHostTask(const void *task, void **, int, const std::vector<int> &) override {
    (*reinterpret_cast<const std::function<void(void)> *>(task))();
    return common::Status::OK();
  }
  common::Status Sync() override;
  virtual CUstream_st *GetComputeStream() { return nullptr; }
  cuda::CudaEnv &GetCudaEnv() { return env_; }

private:
  cuda::CudaEnv env_;
};

class CUDASingleStreamWorkQueue final : public CUDAWorkQueue {
public:
  explicit CUDASingleStreamWorkQueue(int device_id);
  ~CUDASingleStreamWorkQueue() override;
  CUstream_st *GetComputeStream() override { return stream_; }

private:
  CUstream_st *stream_ = nullptr;
};

// runs on a stream the caller owns (e.g. a framework's current stream)
class CUDAExternalStreamWorkQueue final : public CUDAWorkQueue {
public:
  explicit CUDAExternalStreamWorkQueue(CUstream_st *stream, int device_id = -1);
  CUstream_st *GetComputeStream() override { return stream_; }

private:
  CUstream_st *stream_;
};

} // namespace brt
