// Status, element-type names, the ByRE handle, the kernel registry, the provider
// base, OpKernelInfo helpers and OpAccessor.
#include "brt/core/common/common.h"
#include "brt/core/context/execution_frame.h"
#include "brt/core/framework/execution_provider.h"
#include "brt/core/framework/kernel_registry.h"
#include "brt/core/framework/op_accessor.h"
#include "brt/core/framework/op_kernel_info.h"
#include "brt/core/ir/ir.h"

#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <fstream>
#include <mutex>
#include <sstream>

namespace brt {

// ---- Status -------------------------------------------------------------------
namespace common {
std::string Status::ToString() const {
  if (IsOK())
    return "OK";
  std::ostringstream ss;
  ss << (Category() == SYSTEM ? "[SystemError] " : Category() == BRT ? "[BRTError] " : "[Error] ");
  ss << Code() << " : ";
  switch (Code()) {
  case FAIL: ss << "FAIL"; break;
  case INVALID_ARGUMENT: ss << "INVALID_ARGUMENT"; break;
  case NO_SUCHFILE: ss << "NO_SUCHFILE"; break;
  case NO_MODEL: ss << "NO_MODEL"; break;
  case NOT_IMPLEMENTED: ss << "NOT_IMPLEMENTED"; break;
  case INVALID_GRAPH: ss << "INVALID_GRAPH"; break;
  case EP_FAIL: ss << "EP_FAIL"; break;
  default: ss << "GENERAL ERROR"; break;
  }
  ss << " : " << ErrorMessage();
  return ss.str();
}
} // namespace common

// ---- dtype ----------------------------------------------------------------------
DTypeEnum DTypeFromName(const std::string &n) {
  static const std::pair<const char *, DTypeEnum> table[] = {
      {"f32", DTypeEnum::Float32}, {"i32", DTypeEnum::Int32},   {"si32", DTypeEnum::Int32},
      {"i64", DTypeEnum::Int64},   {"si64", DTypeEnum::Int64},  {"index", DTypeEnum::Int64},
      {"ui8", DTypeEnum::UInt8},   {"ui32", DTypeEnum::UInt32}, {"f16", DTypeEnum::Float16},
      {"bf16", DTypeEnum::BFloat16}, {"f64", DTypeEnum::Float64}, {"i1", DTypeEnum::Bool},
      {"i8", DTypeEnum::Int8},     {"si8", DTypeEnum::Int8},    {"i16", DTypeEnum::Int16},
      {"si16", DTypeEnum::Int16},  {"ui16", DTypeEnum::UInt16}, {"ui64", DTypeEnum::UInt64},
      {"tf32", DTypeEnum::TF32},   {"!ace.string", DTypeEnum::StringView}};
  for (auto &e : table)
    if (n == e.first)
      return e.second;
  return DTypeEnum::Invalid;
}

// ---- ByREHandle -------------------------------------------------------------------
namespace ir {

common::Status ByREHandle::Adopt(std::unique_ptr<Module> m) {
  const Function *entry = nullptr;
  for (auto &f : m->functions) {
    if (f.IsEntryPoint()) {
      if (entry)
        return common::Status(common::BRT, common::INVALID_GRAPH, "more than one byre.entry_point function");
      entry = &f;
    }
  }
  if (!entry)
    return common::Status(common::BRT, common::INVALID_GRAPH, "no function carries byre.entry_point");
  module_ = std::move(m);
  entry_ = entry;
  return common::Status::OK();
}

common::Status ByREHandle::Load(const std::string &url, const std::string &fmt) {
  if (fmt != "byre")
    return common::Status(common::BRT, common::INVALID_ARGUMENT, "unknown model format: " + fmt);
  std::ifstream in(url, std::ios::binary);
  if (!in)
    return common::Status(common::BRT, common::NO_SUCHFILE, "cannot open " + url);
  std::stringstream ss;
  ss << in.rdbuf();
  const std::string text = ss.str();
  std::string err;
  if (IsByREBytecode(text.data(), text.size())) {
    auto bc = ParseByREBytecode(text.data(), text.size(), &err);
    if (!bc)
      return common::Status(common::BRT, common::INVALID_GRAPH, url + ": " + err);
    return Adopt(std::move(bc));
  }
  auto m = ParseByRE(text, &err);
  if (!m)
    return common::Status(common::BRT, common::INVALID_GRAPH, url + ": " + err);
  return Adopt(std::move(m));
}

common::Status ByREHandle::LoadFromBuffer(const void *data, size_t size) {
  if (!data)
    return common::Status(common::BRT, common::INVALID_ARGUMENT, "null module buffer");
  std::string err;
  auto m = IsByREBytecode(data, size) ? ParseByREBytecode(data, size, &err)
                                      : ParseByRE(std::string(static_cast<const char *>(data), size), &err);
  if (!m)
    return common::Status(common::BRT, common::INVALID_GRAPH, err);
  return Adopt(std::move(m));
}

common::Status ByREHandle::LoadFromMemory(const void *ptr, const std::string &fmt) {
  if (fmt != "byre")
    return common::Status(common::BRT, common::INVALID_ARGUMENT, "unknown model format: " + fmt);
  if (!ptr)
    return common::Status(common::BRT, common::INVALID_ARGUMENT, "null module text");
  std::string err;
  auto m = ParseByRE(static_cast<const char *>(ptr), &err);
  if (!m)
    return common::Status(common::BRT, common::INVALID_GRAPH, err);
  return Adopt(std::move(m));
}

} // namespace ir

// ---- kernel registration -----------------------------------------------------------
namespace {
struct RegistrationTable {
  std::mutex mu;
  std::vector<std::tuple<std::string, std::string, KernelRegistration>> entries;
};
RegistrationTable &Table() {
  static RegistrationTable *t = new RegistrationTable(); // never destroyed: used from static initialisers
  return *t;
}
} // namespace

void AddKernelRegistration(const std::string &deviceKind, const std::string &providerName,
                           KernelRegistration registration) {
  auto &t = Table();
  std::lock_guard<std::mutex> lock(t.mu);
  t.entries.emplace_back(deviceKind, providerName, std::move(registration));
}

void RegisterKernels(const std::string &deviceKind, const std::string &providerName, KernelRegistry *kernelReg) {
  std::vector<KernelRegistration> todo;
  {
    auto &t = Table();
    std::lock_guard<std::mutex> lock(t.mu);
    for (auto &e : t.entries)
      if (std::get<0>(e) == deviceKind && std::get<1>(e) == providerName)
        todo.push_back(std::get<2>(e));
  }
  for (auto &f : todo)
    f(kernelReg);
}

namespace {
// byre.alias: the plan resolves the address; nothing runs (kernel_registry.cc:77-96)
class AliasOpKernel final : public OpKernel {
public:
  explicit AliasOpKernel(const OpKernelInfo &info) : OpKernel(info) {}
  common::Status RunImpl(const ExecutionContext &) override { return common::Status::OK(); }
};
} // namespace

void RegisterCommonBuiltinOps(KernelRegistry *registry) {
  registry->Register("AliasOp", [](const OpKernelInfo &info) -> std::shared_ptr<OpKernel> {
    return std::make_shared<AliasOpKernel>(info);
  });
}

common::Status ExecutionProvider::StaticRegisterKernelsFromDynlib(const std::string &path) {
  void *h = dlopen(path.c_str(), RTLD_LAZY | RTLD_GLOBAL);
  if (!h)
    return common::Status(common::BRT, common::FAIL, std::string("dlopen failed: ") + dlerror());
  return common::Status::OK();
}

// ---- OpKernelInfo helpers --------------------------------------------------------------
size_t GetTensorIndexFromOpArgIndex(const OpKernelInfo &info, unsigned int i) {
  const ir::Operation *op = info.GetOperation();
  if (i < op->operands.size())
    return (size_t)op->operands[i];
  i -= (unsigned)op->operands.size();
  BRT_ENFORCE(i < op->results.size(), "operand index out of range for ", op->callee);
  return (size_t)op->results[i];
}
unsigned int GetOpArgNum(const OpKernelInfo &info) { return (unsigned)info.GetOperation()->operands.size(); }
unsigned int GetOpResultNum(const OpKernelInfo &info) { return (unsigned)info.GetOperation()->results.size(); }

// ---- OpAccessor ----------------------------------------------------------------------------
namespace {
const ir::Value &ArgValue(const OpKernelInfo &info, size_t arg_idx) {
  const auto &fn = info.GetIRHandle().GetEntryFunc();
  return fn.values[GetTensorIndexFromOpArgIndex(info, (unsigned)arg_idx)];
}
const ir::Attribute &Attr(const OpKernelInfo &info, const std::string &name) {
  const auto &attrs = info.GetOperation()->attrs;
  auto it = attrs.find(name);
  BRT_ENFORCE(it != attrs.end(), "op ", info.GetOperation()->callee, " has no attribute '", name, "'");
  return it->second;
}
} // namespace

size_t OpAccessor::GetNumArgs() const { return GetOpArgNum(info_); }
size_t OpAccessor::GetNumResults() const { return GetOpResultNum(info_); }
Shape OpAccessor::GetArgShape(size_t arg_idx) const { return ArgValue(info_, arg_idx).type.shape; }
DTypeEnum OpAccessor::GetArgDTypeEnum(size_t arg_idx) const { return ArgValue(info_, arg_idx).type.dtype; }
std::string OpAccessor::GetArgSpace(size_t arg_idx) const { return ArgValue(info_, arg_idx).type.space; }
bool OpAccessor::HasAttr(const std::string &name) const { return info_.GetOperation()->attrs.count(name) != 0; }

bool OpAccessor::GetAttrAsBool(const std::string &name) const {
  const auto &a = Attr(info_, name);
  BRT_ENFORCE(a.kind == ir::Attribute::kBool || a.kind == ir::Attribute::kInt, "attribute ", name, " is not a bool");
  return a.i != 0;
}
int64_t OpAccessor::GetAttrAsInt(const std::string &name) const {
  const auto &a = Attr(info_, name);
  BRT_ENFORCE(a.kind == ir::Attribute::kInt || a.kind == ir::Attribute::kBool, "attribute ", name,
              " is not an integer");
  return a.i;
}
float OpAccessor::GetAttrAsFloat(const std::string &name) const {
  const auto &a = Attr(info_, name);
  BRT_ENFORCE(a.kind == ir::Attribute::kFloat, "attribute ", name, " is not a float");
  return (float)a.f;
}
std::string OpAccessor::GetAttrAsString(const std::string &name) const {
  const auto &a = Attr(info_, name);
  BRT_ENFORCE(a.kind == ir::Attribute::kString, "attribute ", name, " is not a string");
  return a.s;
}
std::vector<int64_t> OpAccessor::GetAttrAsIntArray(const std::string &name) const {
  const auto &a = Attr(info_, name);
  std::vector<int64_t> out;
  if (a.kind == ir::Attribute::kArray) {
    for (auto &e : a.array) {
      BRT_ENFORCE(e.kind == ir::Attribute::kInt || e.kind == ir::Attribute::kBool, "attribute ", name,
                  " holds a non-integer element");
      out.push_back(e.i);
    }
  } else if (a.kind == ir::Attribute::kDenseInt) {
    if (a.splat && !a.dense_shape.empty()) {
      int64_t n = 1;
      for (auto d : a.dense_shape)
        n *= d;
      out.assign((size_t)n, a.dense_i.empty() ? 0 : a.dense_i[0]);
    } else {
      out = a.dense_i;
    }
  } else if (a.kind == ir::Attribute::kInt) {
    out.push_back(a.i);
  } else {
    BRT_THROW("attribute ", name, " is not an integer array");
  }
  return out;
}

template <typename T> bool OpAccessor::HasAttrOfSplatValue(const std::string &name) const {
  if (!HasAttr(name))
    return false;
  const auto &a = Attr(info_, name);
  return (a.kind == ir::Attribute::kDenseInt || a.kind == ir::Attribute::kDenseFloat) && a.splat;
}
template <typename T> T OpAccessor::GetAttrAsSplatValue(const std::string &name) const {
  const auto &a = Attr(info_, name);
  BRT_ENFORCE((a.kind == ir::Attribute::kDenseInt || a.kind == ir::Attribute::kDenseFloat) && a.splat,
              "attribute ", name, " is not a splat");
  return a.kind == ir::Attribute::kDenseFloat ? (T)a.dense_f[0] : (T)a.dense_i[0];
}
template <typename T> std::vector<T> OpAccessor::GetAttrAsVector(const std::string &name) const {
  const auto &a = Attr(info_, name);
  std::vector<T> out;
  if (a.kind == ir::Attribute::kDenseFloat) {
    for (double v : a.dense_f)
      out.push_back((T)v);
  } else {
    for (int64_t v : GetAttrAsIntArray(name))
      out.push_back((T)v);
  }
  return out;
}
#define BRT_INST(T)                                                            \
  template bool OpAccessor::HasAttrOfSplatValue<T>(const std::string &) const; \
  template T OpAccessor::GetAttrAsSplatValue<T>(const std::string &) const;    \
  template std::vector<T> OpAccessor::GetAttrAsVector<T>(const std::string &) const;
BRT_INST(float)
BRT_INST(double)
BRT_INST(int64_t)
BRT_INST(int32_t)
#undef BRT_INST

void *OpAccessor::GetAttrAsVoidPtr(const std::string &name, size_t *size) const {
  const auto &a = Attr(info_, name);
  BRT_ENFORCE(a.kind == ir::Attribute::kArray, "attribute ", name, " is not an array");
  size_t total = 0;
  for (auto &e : a.array) {
    if (e.kind == ir::Attribute::kInt || e.kind == ir::Attribute::kBool)
      total += sizeof(int64_t);
    else if (e.kind == ir::Attribute::kFloat)
      total += sizeof(float);
    else
      BRT_THROW("attribute ", name, " holds an element that is neither integer nor float");
  }
  char *blob = static_cast<char *>(std::malloc(total ? total : 1));
  size_t pos = 0;
  for (auto &e : a.array) {
    if (e.kind == ir::Attribute::kFloat) {
      float f = (float)e.f;
      std::memcpy(blob + pos, &f, sizeof(f));
      pos += sizeof(f);
    } else {
      int64_t v = e.i;
      std::memcpy(blob + pos, &v, sizeof(v));
      pos += sizeof(v);
    }
  }
  if (size)
    *size = total;
  return blob;
}

std::string OpAccessor::GetUID() const {
  // callee + position in the entry function: unique per op instance (ir.cc:243-247)
  return info_.GetOperation()->callee + "#" + std::to_string(info_.GetOperation()->index);
}

int64_t OpAccessor::GetNumElementsOfShape(const Shape &shape) {
  int64_t n = 1;
  for (auto d : shape)
    n *= d;
  return n;
}

AsyncValueRef OpAccessor::GetArgAsyncValueRef(size_t arg_idx) const {
  EnsureFrame("GetArgAsyncValueRef");
  return frame_->GetAsyncValueRef(GetTensorIndexFromOpArgIndex(info_, (unsigned)arg_idx));
}

} // namespace brt
