#pragma once
#include <cstdint>
#include <vector>
namespace brt {
// device or host address of a tensor; kernels only enqueue work on it
using AsyncValue = void *;
using AsyncValueRef = void *;
using Shape = std::vector<int64_t>;
} // namespace brt
