// Memory descriptors (runtime/include/brt/core/framework/memory_info.h).
#pragma once

#include <string>

namespace brt {

enum class BrtMemType { CPUInput = -2, CPUOutput = -1, CPU = CPUOutput, Default = 0 };

enum class BrtAllocatorType { Invalid = -1, DeviceAllocator = 0, ArenaAllocator = 1, CustomAllocator = 2 };

// who owns the buffer behind a bound argument (execution_frame.cc:208-247)
enum class BrtOwnershipType { OwnedByExternal = 0, CopiedByRuntime = 1, OwnedByRuntime = 2 };

struct BrtMemoryInfo {
  BrtMemoryInfo() = default;
  BrtMemoryInfo(const char *name_, const char *key_, BrtAllocatorType type_, int id_ = 0,
                BrtMemType mem_type_ = BrtMemType::Default)
      : name(name_), key(key_), id(id_), mem_type(mem_type_), alloc_type(type_) {}
  BrtMemoryInfo(const char *name_, BrtAllocatorType type_, int id_ = 0,
                BrtMemType mem_type_ = BrtMemType::Default)
      : BrtMemoryInfo(name_, name_, type_, id_, mem_type_) {}

  std::string name;
  std::string key; // the memref memory-space string that selects this allocator
  int id = -1;
  BrtMemType mem_type = BrtMemType::Default;
  BrtAllocatorType alloc_type = BrtAllocatorType::Invalid;
};

} // namespace brt
