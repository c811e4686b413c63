// CUDA error checking (runtime/include/brt/backends/cuda/device/common/cuda_call.h):
// BRT_CUDA_CHECK throws, BRT_CUDA_CALL gives a Status.
#pragma once

#include "brt/core/common/exceptions.h"
#include "brt/core/common/status.h"
#include <cuda_runtime.h>

#define BRT_CUDA_CHECK(expr)                                                   \
  do {                                                                         \
    cudaError_t _e = (expr);                                                   \
    if (_e != cudaSuccess) {                                                   \
      (void)cudaGetLastError();                                                \
      BRT_THROW("CUDA failure ", (int)_e, ": ", cudaGetErrorString(_e), " ; expr=" #expr); \
    }                                                                          \
  } while (0)

namespace brt {
inline common::Status CudaCallStatus(cudaError_t e, const char *expr) {
  if (e == cudaSuccess)
    return common::Status::OK();
  (void)cudaGetLastError();
  return common::Status(common::StatusCategory::BRT, common::StatusCode::FAIL,
                        std::string("CUDA failure: ") + cudaGetErrorString(e) + " ; expr=" + expr);
}
} // namespace brt

#define BRT_CUDA_CALL(expr) ::brt::CudaCallStatus((expr), #expr)
