// Kernel-implementation helpers: write an Impl class with a constructor from
// OpAccessor and an Execute(...) taking typed operand pointers, and wrap it as an
// OpKernel.  Same usage as the reference's op_kernel_impl_base.h, reduced to the
// pieces the CUDA provider's ops use (TypedOperand, workspace in frame state).
#pragma once

#include "brt/core/context/execution_frame.h"
#include "brt/core/framework/op_accessor.h"
#include "brt/core/framework/op_kernel.h"
#include <tuple>
#include <type_traits>

namespace brt {

// operand N of the op, as a T (a pointer type)
template <typename T, size_t N> struct TypedOperand {
  using type = T;
  static T Get(const OpAccessor &accessor) {
    return static_cast<T>(accessor.GetArgAsyncValueRef(N));
  }
};

namespace detail {
struct WorkspaceState {
  void *ptr = nullptr;
  size_t bytes = 0;
  IAllocator *allocator = nullptr;
};
} // namespace detail

} // namespace brt
