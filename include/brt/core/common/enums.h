// Reduction named by the `reduction` attribute of a collective op
// (runtime/include/brt/core/common/enums.h:24-42).
#pragma once

#include <string>

namespace brt {

typedef enum {
  BRT_SUM = 0,
  BRT_MAX = 1,
  BRT_MIN = 2,
  BRT_REDUCEOP_COUNT = 3,
} ReduceOp;

// "sum" / "max" / "min"; anything else gives BRT_REDUCEOP_COUNT
inline ReduceOp GetReduceOp(const std::string &name) {
  return name == "sum" ? BRT_SUM : name == "max" ? BRT_MAX : name == "min" ? BRT_MIN : BRT_REDUCEOP_COUNT;
}

} // namespace brt
