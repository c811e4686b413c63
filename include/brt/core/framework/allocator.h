// Allocator interface (runtime/include/brt/core/framework/allocator.h:40-190).
#pragma once

#include "brt/core/common/status.h"
#include "brt/core/framework/memory_info.h"
#include <cstddef>

namespace brt {
class Session;

constexpr const char *CPU = "Cpu";
constexpr const char *CUDA = "Cuda";
constexpr const char *CUDA_PINNED = "CudaPinned";

// every planned intermediate and every workspace starts on this boundary
constexpr size_t kAllocAlignment = 256;

class IAllocator {
public:
  explicit IAllocator(const BrtMemoryInfo &info) : memory_info_(info) {}
  virtual ~IAllocator() = default;
  virtual void *Alloc(size_t size) = 0;
  virtual void Free(void *p) = 0;
  virtual void SetDevice(bool /*throw_when_fail*/) const {}
  const BrtMemoryInfo &Info() const { return memory_info_; }

private:
  BrtMemoryInfo memory_info_;
};

class CPUAllocator : public IAllocator {
public:
  CPUAllocator()
      : IAllocator(BrtMemoryInfo(CPU, "cpu", BrtAllocatorType::DeviceAllocator, 0, BrtMemType::CPU)) {}
  void *Alloc(size_t size) override;
  void Free(void *p) override;
};

// registers the "cpu" allocator (runtime/lib/backends/cpu/device/cpu_device_api.cc)
common::Status CPUAllocatorFactory(Session *session);

} // namespace brt
