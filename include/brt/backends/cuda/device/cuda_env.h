// CudaEnv: which device a queue or kernel works on
// (runtime/include/brt/backends/cuda/device/cuda_env.h; cuda_env.cc:69-79).
#pragma once

namespace brt {
namespace cuda {

class CudaEnv {
public:
  explicit CudaEnv(int device_id = 0) : device_id_(device_id) {}
  // make this env's device current for the calling thread (throws on failure)
  void Activate() const;
  int GetDeviceID() const { return device_id_; }

private:
  int device_id_;
};

} // namespace cuda
} // namespace brt
