// Element types, numbered as the reference numbers them
// (runtime/include/brt/core/framework/dtype.h:28-47).
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>

namespace brt {

enum class DTypeEnum : uint32_t {
  Invalid = 0,
  Float32 = 1,
  Int32 = 2,
  Int64 = 3,
  UInt8 = 4,
  UInt32 = 5,
  Float16 = 6,
  BFloat16 = 7,
  Float64 = 8,
  Bool = 9,
  StringView = 10,
  Int8 = 11,
  Int16 = 12,
  UInt16 = 13,
  UInt64 = 14,
  TF32 = 15,
  LastDType,
  Unsupported = LastDType,
};

inline size_t GetDTypeByte(DTypeEnum dtype) {
  switch (dtype) {
  case DTypeEnum::Float32:
  case DTypeEnum::Int32:
  case DTypeEnum::UInt32:
  case DTypeEnum::TF32:
    return 4;
  case DTypeEnum::Int64:
  case DTypeEnum::UInt64:
  case DTypeEnum::Float64:
    return 8;
  case DTypeEnum::Float16:
  case DTypeEnum::BFloat16:
  case DTypeEnum::Int16:
  case DTypeEnum::UInt16:
    return 2;
  case DTypeEnum::UInt8:
  case DTypeEnum::Int8:
  case DTypeEnum::Bool:
    return 1;
  case DTypeEnum::StringView:
    return 16;
  default:
    return 0;
  }
}

// the spelling the compiler uses in ByRE op keys and MLIR element types
// (compiler/lib/Dialect/Byre/IR/Common.cpp:35-99)
inline const char *DTypeName(DTypeEnum dtype) {
  switch (dtype) {
  case DTypeEnum::Float32: return "f32";
  case DTypeEnum::Int32: return "i32";
  case DTypeEnum::Int64: return "i64";
  case DTypeEnum::UInt8: return "ui8";
  case DTypeEnum::UInt32: return "ui32";
  case DTypeEnum::Float16: return "f16";
  case DTypeEnum::BFloat16: return "bf16";
  case DTypeEnum::Float64: return "f64";
  case DTypeEnum::Bool: return "i1";
  case DTypeEnum::StringView: return "!ace.string";
  case DTypeEnum::Int8: return "i8";
  case DTypeEnum::Int16: return "i16";
  case DTypeEnum::UInt16: return "ui16";
  case DTypeEnum::UInt64: return "ui64";
  case DTypeEnum::TF32: return "tf32";
  default: return "invalid";
  }
}

DTypeEnum DTypeFromName(const std::string &name); // "index" maps to Int64

} // namespace brt
