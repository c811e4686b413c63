// CUDA allocators (runtime/include/brt/backends/cuda/device/cuda_allocator.h).
#pragma once

#include "brt/core/framework/allocator.h"

namespace brt {
class Session;

class CUDAAllocator : public IAllocator {
public:
  CUDAAllocator(int device_id, const char *name)
      : IAllocator(BrtMemoryInfo(name, "cuda", BrtAllocatorType::DeviceAllocator, device_id, BrtMemType::Default)) {}
  void *Alloc(size_t size) override;
  void Free(void *p) override;
  void SetDevice(bool throw_when_fail) const override;
};

// takes its memory from caller-supplied functions (e.g. a framework's caching allocator)
class CUDAExternalAllocator : public CUDAAllocator {
  typedef void *(*ExternalAlloc)(size_t size);
  typedef void (*ExternalFree)(void *p);

public:
  CUDAExternalAllocator(int device_id, const char *name, void *alloc, void *free)
      : CUDAAllocator(device_id, name), alloc_(reinterpret_cast<ExternalAlloc>(alloc)),
        free_(reinterpret_cast<ExternalFree>(free)) {}
  void *Alloc(size_t size) override { return alloc_(size); }
  void Free(void *p) override { free_(p); }

private:
  ExternalAlloc alloc_;
  ExternalFree free_;
};

class CUDAPinnedAllocator : public IAllocator {
public:
  CUDAPinnedAllocator(int device_id, const char *name)
      : IAllocator(BrtMemoryInfo(name, "cudaPinned", BrtAllocatorType::DeviceAllocator, device_id,
                                 BrtMemType::CPUOutput)) {}
  void *Alloc(size_t size) override;
  void Free(void *p) override;
};

// registers allocators for the memory spaces "cuda" and "cudaPinned"
// (runtime/lib/backends/cuda/device/cuda_allocator.cc:88-110); use_arena and
// size are accepted for source compatibility (no arena here: intermediates are
// planned statically and allocated once per frame)
common::Status CUDAAllocatorFactory(Session *session, int device_id = 0, bool use_arena = false,
                                    size_t size = 1 << 30);
common::Status CUDAExternalAllocatorFactory(Session *session, int device_id, void *alloc, void *free);

} // namespace brt
