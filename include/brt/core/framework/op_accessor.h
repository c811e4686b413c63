// OpAccessor: how a kernel reads its op's operands and attributes
// (runtime/include/brt/core/framework/op_accessor.h:36-97, lib: op_accessor.cc).
#pragma once

#include "brt/core/common/common.h"
#include "brt/core/framework/dtype.h"
#include "brt/core/framework/value.h"
#include <string>

namespace brt {
class OpKernelInfo;
class ExecutionFrame;

class OpAccessor {
public:
  OpAccessor(const OpKernelInfo &info) : info_(info), frame_(nullptr) {}
  OpAccessor(const OpKernelInfo &info, ExecutionFrame *frame) : info_(info), frame_(frame) {}

  /****** ExecutionFrame-free API ******/
  size_t GetNumArgs() const;
  size_t GetNumResults() const;
  Shape GetArgShape(size_t arg_idx) const;
  DTypeEnum GetArgDTypeEnum(size_t arg_idx) const;
  std::string GetArgSpace(size_t arg_idx) const;
  bool HasAttr(const std::string &name) const;
  bool GetAttrAsBool(const std::string &name) const;
  int64_t GetAttrAsInt(const std::string &name) const;
  float GetAttrAsFloat(const std::string &name) const;
  std::string GetAttrAsString(const std::string &name) const;
  // accepts an array of integer attrs, array<i64: ...> and dense<...> : tensor<..xi64>
  std::vector<int64_t> GetAttrAsIntArray(const std::string &name) const;
  template <typename T> bool HasAttrOfSplatValue(const std::string &name) const;
  template <typename T> T GetAttrAsSplatValue(const std::string &name) const;
  template <typename T> std::vector<T> GetAttrAsVector(const std::string &name) const;
  // Packs an array attribute into a malloc'd blob the caller frees: each integer
  // element as int64 (8 bytes), each float element as float (4 bytes), in order,
  // unaligned (op_accessor.cc:212-242).  *size gets the byte count if not null.
  void *GetAttrAsVoidPtr(const std::string &name, size_t *size = nullptr) const;
  std::string GetUID() const;
  static int64_t GetNumElementsOfShape(const Shape &shape);

  /****** Need attached ExecutionFrame ******/
  AsyncValueRef GetArgAsyncValueRef(size_t arg_idx) const;

private:
  void EnsureFrame(const std::string &where) const {
    BRT_ENFORCE(frame_, "need active execution frame by: " + where);
  }
  const OpKernelInfo &info_;
  ExecutionFrame *frame_;
};

} // namespace brt
