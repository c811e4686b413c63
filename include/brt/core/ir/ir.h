// ByRE module handle without MLIR.
//
// The reference parses ByRE with the MLIR parser and walks mlir::Operation
// (runtime/lib/core/ir/ir.cc:22-300).  This runtime carries its own small
// object model and a hand-written parser for the textual ByRE subset that
// byteir-opt emits: a module with one func.func marked byre.entry_point whose
// body is a flat list of byre.compute / byre.copy / byre.alias / byre.custom /
// memref.alloc ops; and a reader of the same modules in ByRE bytecode (bytecode.cc).
#pragma once

#include "brt/core/common/status.h"
#include "brt/core/framework/dtype.h"
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace brt {
namespace ir {

// byre.argtype bit mask (compiler/include/byteir/Dialect/Byre/ByreBase.td:93-96)
enum ArgType : int { kInput = 1, kOutput = 2, kWeight = 4 };

struct MemRefType {
  DTypeEnum dtype = DTypeEnum::Invalid;
  std::vector<int64_t> shape; // -1 for a dynamic dim
  std::string space;          // "cuda", "cpu", "" ...
  int64_t NumElements() const;
  size_t SizeInBytes() const;
};

struct Attribute {
  enum Kind { kUnit, kInt, kFloat, kString, kBool, kArray, kDenseInt, kDenseFloat, kType } kind = kUnit;
  int64_t i = 0;
  double f = 0;
  std::string s;
  DTypeEnum elt_type = DTypeEnum::Invalid; // of an int/float attr or a dense attr's elements
  std::vector<Attribute> array;            // kArray
  std::vector<int64_t> dense_i;            // kDenseInt: values (a single value if splat)
  std::vector<double> dense_f;             // kDenseFloat
  bool splat = false;
  std::vector<int64_t> dense_shape;        // tensor<...> shape of a dense attr
};

using AttrDict = std::map<std::string, Attribute>;

struct Value {
  int id = -1;       // dense numbering over the entry function: args first
  std::string name;  // "%arg0", "%alloc", "%0"
  MemRefType type;
  int arg_index = -1;      // >= 0 for entry-function arguments
  int defining_op = -1;    // index into Function::ops, -1 for arguments
};

struct Operation {
  std::string name;   // "byre.compute", "byre.custom", "byre.copy", "byre.alias", "memref.alloc", ...
  std::string callee; // the registry key: @Callee of byre.compute, or the callee attr
  std::vector<int> operands; // Value ids
  std::vector<int> results;  // Value ids
  AttrDict attrs;
  int index = -1;
  int line = 0;
};

struct Function {
  std::string name;
  std::vector<int> args; // Value ids
  std::vector<AttrDict> arg_attrs;
  AttrDict attrs;
  std::vector<Operation> ops;
  std::vector<Value> values;
  bool IsEntryPoint() const { return attrs.count("byre.entry_point") != 0; }
};

struct Module {
  std::string name;
  AttrDict attrs;
  std::vector<Function> functions;
};

// Parses ByRE text.  On a syntax error returns nullptr and sets *error to
// "line N: message".
std::unique_ptr<Module> ParseByRE(const std::string &text, std::string *error);

// Reads ByRE bytecode: MLIR bytecode (container version 5) of the `byre_serial` dialect,
// version 1.0.0.  On failure returns nullptr and sets *error.
bool IsByREBytecode(const void *data, size_t size);
std::unique_ptr<Module> ParseByREBytecode(const void *data, size_t size, std::string *error);

class IRHandle {
public:
  virtual ~IRHandle() = default;
  virtual common::Status Load(const std::string &url, const std::string &fmt) = 0;
  virtual common::Status LoadFromMemory(const void *ptr, const std::string &fmt) = 0;
};

// Holds one loaded ByRE module and its entry function.
class ByREHandle : public IRHandle {
public:
  // fmt "byre": `url` names a text file (.mlir) or a bytecode file (.mlirbc, told apart by
  // its magic).
  common::Status Load(const std::string &url, const std::string &fmt) override;
  // fmt "byre": `ptr` is a NUL-terminated ByRE text buffer.  (The reference takes an
  // mlir::ModuleOp here, runtime/lib/core/ir/ir.cc:171-184.)
  common::Status LoadFromMemory(const void *ptr, const std::string &fmt) override;
  // `size` bytes of ByRE text or ByRE bytecode (a module a host already holds in memory)
  common::Status LoadFromBuffer(const void *data, size_t size);

  const Module &GetModule() const { return *module_; }
  const Function &GetEntryFunc() const { return *entry_; }
  bool IsLoaded() const { return entry_ != nullptr; }

private:
  common::Status Adopt(std::unique_ptr<Module> m);
  std::unique_ptr<Module> module_;
  const Function *entry_ = nullptr;
};

} // namespace ir
} // namespace brt
