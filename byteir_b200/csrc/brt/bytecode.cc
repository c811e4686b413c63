// ByRE bytecode reader: MLIR bytecode (container version 5, as MLIR 17 writes it) whose only
// payload dialect is `byre_serial` version 1.0.0, the form `byteir-translate -emit-byre-bytecode`
// writes and the reference loads with the MLIR parser (runtime/lib/core/ir/ir.cc:86-118).
//
// What the reference's dialect defines, and this file decodes without MLIR:
//   ops      module_v1, func_v1, return_v1, alloc_v1, compute_v1, copy_v1, group_copy_v1, alias
//            (compiler/include/byteir/Dialect/Byre/Serialization/ByreSerial.td:355-424); their
//            attributes are native properties, written in the alphabetical order of their names,
//            optional ones as (index << 1 | 1) or 0;
//   types    kinds 0..24 (compiler/lib/Dialect/Byre/IR/Serialization/Bytecode.cpp:34-60);
//   attrs    kinds 0..12 (Bytecode.cpp:62-76) with the encodings of Bytecode.cpp:199-330;
//   back to ByRE as compiler/lib/Dialect/Byre/IR/Serialization.cpp:466-545 does: the entries of
//            compute_v1's `extra_args` dictionary become the op's attributes, byre_arg_names /
//            byre_arg_types become argument attributes.
// The container: magic "ML\xefR", version, producer, then sections (string 0, dialect 1, attr/type
// 2, their offsets 3, IR 4, resources 5/6, dialect versions 7, properties 8).  Integers are
// prefix varints: the number of trailing zero bits of the first byte is the number of bytes
// that follow.  Locations are read past, use-list orders and resources are not supported.
#include "brt/core/ir/ir.h"

#include <cstring>
#include <stdexcept>

namespace brt {
namespace ir {
namespace {

struct Fail : std::runtime_error {
  using std::runtime_error::runtime_error;
};

class Reader {
public:
  Reader() = default;
  Reader(const uint8_t *base, size_t begin, size_t end) : b_(base), p_(begin), e_(end) {}
  bool Done() const { return p_ >= e_; }
  size_t Pos() const { return p_; }
  uint8_t Byte() {
    Need(1);
    return b_[p_++];
  }
  uint64_t VarInt() {
    const uint8_t b0 = Byte();
    if (b0 & 1)
      return b0 >> 1;
    if (b0 == 0) {
      Need(8);
      uint64_t v;
      std::memcpy(&v, b_ + p_, 8);
      p_ += 8;
      return v;
    }
    const int n = __builtin_ctz(b0);
    Need((size_t)n);
    uint64_t v = b0;
    for (int i = 0; i < n; ++i)
      v |= (uint64_t)b_[p_ + i] << (8 * (i + 1));
    p_ += n;
    return v >> (n + 1);
  }
  int64_t SignedVarInt() {
    const uint64_t v = VarInt();
    return (int64_t)(v >> 1) ^ -(int64_t)(v & 1);
  }
  uint64_t Flagged(bool *flag) {
    const uint64_t v = VarInt();
    *flag = v & 1;
    return v >> 1;
  }
  const uint8_t *Bytes(size_t n) {
    Need(n);
    const uint8_t *r = b_ + p_;
    p_ += n;
    return r;
  }
  // a nested section: id byte (high bit: aligned), length, optional alignment and 0xCB padding
  Reader Section(int *id) {
    const uint8_t idb = Byte();
    *id = idb & 0x7f;
    const uint64_t len = VarInt();
    if (idb & 0x80) {
      const uint64_t align = VarInt();
      if (align == 0 || (align & (align - 1)))
        throw Fail("section alignment is not a power of two");
      while (p_ % align)
        if (Byte() != 0xCB)
          throw Fail("bad section padding");
    }
    Need(len);
    Reader r(b_, p_, p_ + len);
    p_ += len;
    return r;
  }

private:
  void Need(size_t n) const {
    if (n > e_ - p_ || p_ > e_)
      throw Fail("truncated bytecode at byte " + std::to_string(p_));
  }
  const uint8_t *b_ = nullptr;
  size_t p_ = 0, e_ = 0;
};

// a decoded byre_serial type
struct SerialType {
  enum Kind { kScalar, kString, kMemref, kTensor, kFunction } kind = kScalar;
  DTypeEnum dtype = DTypeEnum::Invalid; // scalar, or element type
  std::vector<int64_t> shape;
  std::string space;
};

// a decoded attribute: an ir::Attribute, or one of the two shapes that have no ir:: form
struct SerialAttr {
  Attribute value;
  bool is_dict = false;
  std::vector<std::pair<std::string, int>> dict; // name, attribute index
  bool is_symbol = false;                        // value.s holds the root reference
  bool is_location = false;
};

struct Entry {
  int dialect;
  size_t begin, size;
  bool custom;
};

class Decoder {
public:
  Decoder(const uint8_t *data, size_t size) : d_(data), n_(size) {}

  std::unique_ptr<Module> Run() {
    Reader top(d_, 0, n_);
    if (n_ < 4 || std::memcmp(d_, "ML\xefR", 4) != 0)
      throw Fail("not MLIR bytecode");
    top.Bytes(4);
    const uint64_t version = top.VarInt();
    if (version != 5)
      throw Fail("bytecode container version " + std::to_string(version) + " (this reader knows version 5, MLIR 17)");
    while (top.Byte() != 0) { // producer string
    }
    Reader sections[9];
    bool have[9] = {};
    while (!top.Done()) {
      int id;
      Reader r = top.Section(&id);
      if (id > 8)
        throw Fail("unknown section " + std::to_string(id));
      sections[id] = r;
      have[id] = true;
    }
    for (int need : {0, 1, 2, 3, 4})
      if (!have[need])
        throw Fail("section " + std::to_string(need) + " is missing");
    ReadStrings(sections[0]);
    ReadDialects(sections[1]);
    ReadOffsets(sections[3], sections[2].Pos());
    if (have[8])
      ReadProperties(sections[8]);
    module_ = std::make_unique<Module>();
    ReadTopLevel(sections[4]);
    if (module_->functions.empty())
      throw Fail("the module holds no function");
    return std::move(module_);
  }

private:
  // ---- tables -------------------------------------------------------------------------
  void ReadStrings(Reader r) {
    const uint64_t count = r.VarInt();
    std::vector<uint64_t> sizes(count);
    uint64_t total = 0;
    for (auto &s : sizes) // sizes (with the NUL) are stored last string first
      total += (s = r.VarInt());
    const uint8_t *data = r.Bytes(total);
    strings_.resize(count);
    for (uint64_t i = 0; i < count; ++i) {
      const uint64_t sz = sizes[count - 1 - i];
      if (sz == 0)
        throw Fail("empty string entry");
      strings_[i].assign(reinterpret_cast<const char *>(data), sz - 1);
      data += sz;
    }
  }
  const std::string &Str(uint64_t i) const {
    if (i >= strings_.size())
      throw Fail("string index out of range");
    return strings_[i];
  }

  void ReadDialects(Reader r) {
    const uint64_t count = r.VarInt();
    for (uint64_t i = 0; i < count; ++i) {
      bool versioned;
      dialects_.push_back(Str(r.Flagged(&versioned)));
      if (versioned) {
        int id;
        Reader v = r.Section(&id);
        if (id != 7)
          throw Fail("expected a dialect version section");
        // the dialect writes one number and its reader ignores it (Bytecode.cpp:582-589): the op,
        // type and attribute names carry their own version suffix
        v.VarInt();
      }
    }
    r.VarInt(); // number of op names
    while (!r.Done()) {
      const uint64_t dialect = r.VarInt(), n = r.VarInt();
      if (dialect >= dialects_.size())
        throw Fail("dialect index out of range");
      for (uint64_t i = 0; i < n; ++i) {
        bool registered;
        op_names_.push_back({(int)dialect, Str(r.Flagged(&registered))});
      }
    }
  }

  void ReadOffsets(Reader r, size_t data_begin) {
    const uint64_t n_attrs = r.VarInt(), n_types = r.VarInt();
    size_t at = data_begin;
    std::vector<Entry> all;
    while (!r.Done()) {
      const uint64_t dialect = r.VarInt(), n = r.VarInt();
      for (uint64_t i = 0; i < n; ++i) {
        bool custom;
        const uint64_t size = r.Flagged(&custom);
        all.push_back({(int)dialect, at, (size_t)size, custom});
        at += size;
      }
    }
    if (all.size() != n_attrs + n_types)
      throw Fail("attribute/type table size mismatch");
    attr_entries_.assign(all.begin(), all.begin() + n_attrs);
    type_entries_.assign(all.begin() + n_attrs, all.end());
    attrs_.resize(n_attrs);
    attr_done_.assign(n_attrs, 0);
    types_.resize(n_types);
    type_done_.assign(n_types, 0);
  }

  void ReadProperties(Reader r) {
    const uint64_t count = r.VarInt();
    for (uint64_t i = 0; i < count; ++i) {
      const uint64_t size = r.VarInt();
      const size_t begin = r.Pos();
      r.Bytes(size);
      props_.push_back({begin, begin + (size_t)size});
    }
  }

  // ---- types --------------------------------------------------------------------------
  const SerialType &Type(uint64_t i) {
    if (i >= types_.size())
      throw Fail("type index out of range");
    if (type_done_[i] == 1)
      throw Fail("a type refers to itself");
    if (type_done_[i] == 0) {
      type_done_[i] = 1;
      const Entry &e = type_entries_[i];
      if (!e.custom || dialects_[e.dialect] != "byre_serial")
        throw Fail("type " + std::to_string(i) + " is not a byre_serial type");
      Reader r(d_, e.begin, e.begin + e.size);
      types_[i] = DecodeType(r);
      type_done_[i] = 2;
    }
    return types_[i];
  }

  SerialType DecodeType(Reader &r) {
    static const DTypeEnum scalar[] = {
        DTypeEnum::Bool,    DTypeEnum::BFloat16, DTypeEnum::Float16, DTypeEnum::Float32, DTypeEnum::Float64,
        DTypeEnum::Invalid, DTypeEnum::Invalid,  DTypeEnum::Invalid, DTypeEnum::Invalid, DTypeEnum::Invalid, // f8 kinds
        DTypeEnum::Int64 /* index */, DTypeEnum::Invalid /* i4 */, DTypeEnum::Int8, DTypeEnum::Int16, DTypeEnum::Int32,
        DTypeEnum::Int64,   DTypeEnum::Invalid /* ui4 */, DTypeEnum::UInt8, DTypeEnum::UInt16, DTypeEnum::UInt32,
        DTypeEnum::UInt64};
    const uint64_t kind = r.VarInt();
    SerialType t;
    if (kind <= 20) {
      t.dtype = scalar[kind];
      if (t.dtype == DTypeEnum::Invalid)
        throw Fail("element type kind " + std::to_string(kind) + " has no runtime dtype");
      return t;
    }
    if (kind == 21) {
      t.kind = SerialType::kString;
      t.dtype = DTypeEnum::StringView;
      return t;
    }
    if (kind == 22 || kind == 23) { // shape, element type, optional memory space / encoding
      t.kind = kind == 22 ? SerialType::kMemref : SerialType::kTensor;
      const uint64_t rank = r.VarInt();
      for (uint64_t i = 0; i < rank; ++i) {
        const int64_t dim = r.SignedVarInt();
        t.shape.push_back(dim < 0 ? -1 : dim);
      }
      const SerialType &elt = Type(r.VarInt());
      if (elt.kind != SerialType::kScalar && elt.kind != SerialType::kString)
        throw Fail("shaped type with a shaped element type");
      t.dtype = elt.dtype;
      bool present;
      const uint64_t extra = r.Flagged(&present);
      if (present && kind == 22) {
        const SerialAttr &space = Attr(extra);
        if (space.value.kind != Attribute::kString)
          throw Fail("memory space is not a string");
        t.space = space.value.s;
      }
      return t;
    }
    if (kind == 24) {
      t.kind = SerialType::kFunction;
      return t; // inputs and outputs repeat the block arguments
    }
    throw Fail("unknown byre_serial type kind " + std::to_string(kind));
  }

  // ---- attributes ---------------------------------------------------------------------
  const SerialAttr &Attr(uint64_t i) {
    if (i >= attrs_.size())
      throw Fail("attribute index out of range");
    if (attr_done_[i] == 1)
      throw Fail("an attribute refers to itself");
    if (attr_done_[i] == 0) {
      attr_done_[i] = 1;
      const Entry &e = attr_entries_[i];
      if (dialects_[e.dialect] == "builtin") {
        attrs_[i].is_location = true; // only locations come from the builtin dialect here
      } else {
        if (!e.custom || dialects_[e.dialect] != "byre_serial")
          throw Fail("attribute " + std::to_string(i) + " is not a byre_serial attribute");
        Reader r(d_, e.begin, e.begin + e.size);
        attrs_[i] = DecodeAttr(r);
      }
      attr_done_[i] = 2;
    }
    return attrs_[i];
  }

  // APInt of a known width (BytecodeReader's readAPIntWithKnownWidth): one byte up to 8 bits,
  // a signed varint up to 64
  static int64_t ReadAPInt(Reader &r, unsigned bits) {
    if (bits <= 8)
      return (int64_t)(int8_t)r.Byte();
    if (bits <= 64)
      return r.SignedVarInt();
    throw Fail("integers wider than 64 bits are not supported");
  }

  static double FloatFromBits(DTypeEnum t, uint64_t bits) {
    if (t == DTypeEnum::Float64) {
      double v;
      std::memcpy(&v, &bits, 8);
      return v;
    }
    uint32_t w;
    if (t == DTypeEnum::Float32) {
      w = (uint32_t)bits;
    } else if (t == DTypeEnum::BFloat16) {
      w = (uint32_t)(bits & 0xffff) << 16;
    } else { // f16
      const uint32_t h = (uint32_t)bits & 0xffff, sign = (h & 0x8000u) << 16;
      uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff;
      if (exp == 0x1f) {
        w = sign | 0x7f800000u | (man << 13);
      } else if (exp == 0) {
        if (man == 0) {
          w = sign;
        } else {
          int e = -1;
          do {
            ++e;
            man <<= 1;
          } while (!(man & 0x400));
          w = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13);
        }
      } else {
        w = sign | ((exp + 112) << 23) | (man << 13);
      }
    }
    float f;
    std::memcpy(&f, &w, 4);
    return f;
  }

  static bool IsFloat(DTypeEnum t) {
    return t == DTypeEnum::Float16 || t == DTypeEnum::BFloat16 || t == DTypeEnum::Float32 || t == DTypeEnum::Float64;
  }

  // raw little-endian element data of a dense attribute; i1 is bit-packed, a single element
  // (or a single 0x00 / 0xff byte for i1) is a splat
  void DenseFromBlob(const SerialType &t, const uint8_t *blob, size_t size, int64_t count, Attribute *a) {
    a->elt_type = t.dtype;
    a->dense_shape = t.shape;
    const bool is_float = IsFloat(t.dtype);
    a->kind = is_float ? Attribute::kDenseFloat : Attribute::kDenseInt;
    auto push = [&](int64_t i, double f) {
      a->dense_i.push_back(is_float ? (int64_t)f : i);
      a->dense_f.push_back(is_float ? f : (double)i);
    };
    if (t.dtype == DTypeEnum::Bool) {
      if (size == 1 && (blob[0] == 0x00 || blob[0] == 0xff) && count != 8) {
        a->splat = true;
        push(blob[0] ? 1 : 0, 0);
        return;
      }
      if ((int64_t)size * 8 < count)
        throw Fail("dense i1 data is too short");
      for (int64_t i = 0; i < count; ++i)
        push((blob[i / 8] >> (i % 8)) & 1, 0);
      return;
    }
    const size_t w = GetDTypeByte(t.dtype);
    if (w == 0 || size % w != 0)
      throw Fail("dense data size does not match its element type");
    const int64_t have = (int64_t)(size / w);
    if (have != count && have != 1)
      throw Fail("dense data holds " + std::to_string(have) + " elements for a tensor of " + std::to_string(count));
    a->splat = have == 1;
    for (int64_t i = 0; i < have; ++i) {
      uint64_t bits = 0;
      std::memcpy(&bits, blob + i * w, w);
      if (is_float) {
        push(0, FloatFromBits(t.dtype, bits));
      } else {
        const bool is_signed = t.dtype == DTypeEnum::Int8 || t.dtype == DTypeEnum::Int16 || t.dtype == DTypeEnum::Int32 ||
                               t.dtype == DTypeEnum::Int64;
        int64_t v = (int64_t)bits;
        if (is_signed && w < 8) {
          const int shift = 64 - 8 * (int)w;
          v = (int64_t)(bits << shift) >> shift;
        }
        push(v, 0);
      }
    }
  }

  SerialAttr DecodeAttr(Reader &r) {
    SerialAttr out;
    Attribute &a = out.value;
    const uint64_t kind = r.VarInt();
    switch (kind) {
    case 0: { // IntegerV1: type, value
      const SerialType &t = Type(r.VarInt());
      a.elt_type = t.dtype;
      if (t.dtype == DTypeEnum::Bool) {
        a.kind = Attribute::kBool;
        a.i = ReadAPInt(r, 1) & 1;
      } else {
        a.kind = Attribute::kInt;
        const unsigned bits = (unsigned)GetDTypeByte(t.dtype) * 8;
        a.i = ReadAPInt(r, bits); // the writer stores the zero-extended pattern
        const bool is_unsigned = t.dtype == DTypeEnum::UInt8 || t.dtype == DTypeEnum::UInt16 ||
                                 t.dtype == DTypeEnum::UInt32 || t.dtype == DTypeEnum::UInt64;
        if (bits < 64) {
          const uint64_t mask = (1ull << bits) - 1;
          const uint64_t u = (uint64_t)a.i & mask;
          a.i = is_unsigned || !(u >> (bits - 1)) ? (int64_t)u : (int64_t)(u | ~mask);
        }
      }
      a.f = (double)a.i;
      break;
    }
    case 1: { // FloatV1: type, bit pattern
      const SerialType &t = Type(r.VarInt());
      if (!IsFloat(t.dtype))
        throw Fail("float attribute of a non-float type");
      a.kind = Attribute::kFloat;
      a.elt_type = t.dtype;
      a.f = FloatFromBits(t.dtype, (uint64_t)ReadAPInt(r, (unsigned)GetDTypeByte(t.dtype) * 8));
      a.i = (int64_t)a.f;
      break;
    }
    case 2:
      a.kind = Attribute::kUnit;
      break;
    case 3: { // ArrayV1
      a.kind = Attribute::kArray;
      const uint64_t n = r.VarInt();
      for (uint64_t i = 0; i < n; ++i)
        a.array.push_back(Plain(r.VarInt()));
      break;
    }
    case 4: { // DictionaryV1: (name, value) pairs
      out.is_dict = true;
      const uint64_t n = r.VarInt();
      for (uint64_t i = 0; i < n; ++i) {
        const SerialAttr &name = Attr(r.VarInt());
        if (name.value.kind != Attribute::kString)
          throw Fail("dictionary key is not a string");
        out.dict.push_back({name.value.s, (int)r.VarInt()});
      }
      break;
    }
    case 5:
      a.kind = Attribute::kString;
      a.s = Str(r.VarInt());
      break;
    case 6: { // TypeV1
      a.kind = Attribute::kType;
      const SerialType &t = Type(r.VarInt());
      a.elt_type = t.dtype;
      a.dense_shape = t.shape;
      break;
    }
    case 7: { // SymbolRefV1: root, nested
      out.is_symbol = true;
      const SerialAttr &root = Attr(r.VarInt());
      if (root.value.kind != Attribute::kString)
        throw Fail("symbol reference without a name");
      a.kind = Attribute::kString;
      a.s = root.value.s;
      const uint64_t nested = r.VarInt();
      for (uint64_t i = 0; i < nested; ++i)
        r.VarInt();
      break;
    }
    case 8: { // DenseIntOrFPElementsV1: tensor type, blob
      const SerialType t = Type(r.VarInt());
      if (t.kind != SerialType::kTensor)
        throw Fail("dense attribute without a tensor type");
      int64_t count = 1;
      for (int64_t dim : t.shape)
        count *= dim;
      const uint64_t size = r.VarInt();
      DenseFromBlob(t, r.Bytes(size), size, count, &a);
      break;
    }
    case 10: { // DenseArrayV1: element type, size, blob
      const SerialType t = Type(r.VarInt());
      const int64_t count = r.SignedVarInt();
      const uint64_t size = r.VarInt();
      SerialType flat = t;
      flat.shape = {count};
      DenseFromBlob(flat, r.Bytes(size), size, count, &a);
      a.splat = false;
      break;
    }
    case 11: // ArgTypeV1
    case 12: // MemoryEffectV1
      a.kind = Attribute::kInt;
      a.elt_type = DTypeEnum::Int32;
      a.i = (int64_t)r.VarInt();
      a.f = (double)a.i;
      break;
    default:
      throw Fail("byre_serial attribute kind " + std::to_string(kind) + " is not supported");
    }
    return out;
  }

  // an attribute that has an ir::Attribute form
  Attribute Plain(uint64_t i) {
    const SerialAttr &a = Attr(i);
    if (a.is_dict || a.is_location)
      throw Fail("a dictionary or location where a value is expected");
    return a.value;
  }

  // ---- IR -----------------------------------------------------------------------------
  struct OpHeader {
    std::string name;
    int props = -1;
    std::vector<int> result_types, operands;
    int regions = 0;
    bool isolated = false;
  };

  OpHeader ReadOpHeader(Reader &r) {
    OpHeader h;
    const uint64_t name = r.VarInt();
    if (name >= op_names_.size())
      throw Fail("op name index out of range");
    if (dialects_[op_names_[name].first] != "byre_serial")
      throw Fail("op of dialect " + dialects_[op_names_[name].first] + " in a ByRE bytecode module");
    h.name = op_names_[name].second;
    const uint8_t mask = r.Byte();
    r.VarInt(); // location
    if (mask & 0x01)
      throw Fail("op " + h.name + " carries a discardable attribute dictionary");
    if (mask & 0x40)
      h.props = (int)r.VarInt();
    if (mask & 0x02) {
      const uint64_t n = r.VarInt();
      for (uint64_t i = 0; i < n; ++i)
        h.result_types.push_back((int)r.VarInt());
    }
    if (mask & 0x04) {
      const uint64_t n = r.VarInt();
      for (uint64_t i = 0; i < n; ++i)
        h.operands.push_back((int)r.VarInt());
    }
    if (mask & 0x08)
      throw Fail("op " + h.name + " has successors");
    if (mask & 0x20)
      throw Fail("use-list orders are not supported");
    if (mask & 0x10) {
      bool isolated;
      h.regions = (int)r.Flagged(&isolated);
      h.isolated = isolated;
    }
    return h;
  }

  // the properties of op `h`: one attribute index per declared attribute, alphabetical order
  std::vector<int> ReadProps(const OpHeader &h, const std::vector<bool> &optional) {
    if (h.props < 0 || (size_t)h.props >= props_.size())
      throw Fail("op " + h.name + " has no properties");
    Reader r(d_, props_[h.props].first, props_[h.props].second);
    std::vector<int> out;
    for (bool opt : optional) {
      if (opt) {
        bool present;
        const uint64_t idx = r.Flagged(&present);
        out.push_back(present ? (int)idx : -1);
      } else {
        out.push_back((int)r.VarInt());
      }
    }
    return out;
  }

  // region header of an op with one region: returns the reader to parse the region from
  Reader EnterRegion(Reader &r, const OpHeader &h, Reader *nested) {
    if (h.regions != 1)
      throw Fail("op " + h.name + " must have one region");
    if (!h.isolated)
      return r;
    int id;
    *nested = r.Section(&id); // lazily loadable regions sit in an IR section of their own
    if (id != 4)
      throw Fail("expected a nested IR section");
    return *nested;
  }

  void ReadTopLevel(Reader r) {
    bool has_args;
    if (r.Flagged(&has_args) != 1 || has_args)
      throw Fail("the top level must hold exactly one op");
    OpHeader mod = ReadOpHeader(r);
    if (mod.name != "module_v1")
      throw Fail("top-level op is " + mod.name + ", expected module_v1");
    // container_module, sym_name?, sym_visibility?
    const std::vector<int> p = ReadProps(mod, {false, true, true});
    module_->attrs["byre.container_module"] = Plain(p[0]);
    if (p[1] >= 0)
      module_->name = Plain(p[1]).s;
    Reader nested;
    Reader body = EnterRegion(r, mod, &nested);
    Reader &b = mod.isolated ? body : r;
    const uint64_t blocks = b.VarInt();
    if (blocks == 0)
      return;
    if (blocks != 1)
      throw Fail("the module body must be one block");
    b.VarInt(); // values defined in the region
    const uint64_t n_ops = b.Flagged(&has_args);
    if (has_args)
      throw Fail("the module body has block arguments");
    for (uint64_t i = 0; i < n_ops; ++i)
      ReadFunc(b);
  }

  void ReadFunc(Reader &r) {
    OpHeader f = ReadOpHeader(r);
    if (f.name != "func_v1")
      throw Fail("op " + f.name + " at module level, expected func_v1");
    // byre_arg_alias_indexs?, byre_arg_names, byre_arg_types, byre_entry_point, byteir_entry_point?,
    // function_type, sym_name, sym_visibility?, tf_original_input_names?
    const std::vector<int> p = ReadProps(f, {true, false, false, false, true, false, false, true, true});
    module_->functions.emplace_back();
    Function &fn = module_->functions.back();
    // regions that are not isolated number their values on from the enclosing scope
    value_base_ = f.isolated ? 0 : scope_values_;
    fn.name = Plain(p[6]).s;
    fn.attrs["byre.entry_point"] = Plain(p[3]);
    const Attribute names = Plain(p[1]), types = Plain(p[2]);
    Reader nested;
    Reader body = EnterRegion(r, f, &nested);
    Reader &b = f.isolated ? body : r;
    if (b.VarInt() != 1)
      throw Fail("a function body must be one block");
    const uint64_t region_values = b.VarInt();
    if (!f.isolated)
      scope_values_ += region_values;
    bool has_args;
    const uint64_t n_ops = b.Flagged(&has_args);
    if (has_args) {
      const uint64_t n = b.VarInt();
      for (uint64_t i = 0; i < n; ++i) {
        bool has_loc;
        const SerialType &t = Type(b.Flagged(&has_loc));
        if (has_loc)
          b.VarInt();
        if (t.kind != SerialType::kMemref)
          throw Fail("function argument " + std::to_string(i) + " is not a memref");
        Value v;
        v.id = (int)fn.values.size();
        v.name = "%arg" + std::to_string(i);
        v.type.dtype = t.dtype;
        v.type.shape = t.shape;
        v.type.space = t.space;
        v.arg_index = (int)i;
        fn.args.push_back(v.id);
        fn.values.push_back(v);
        AttrDict d;
        if (i < names.array.size())
          d["byre.argname"] = names.array[i];
        if (i < types.array.size())
          d["byre.argtype"] = types.array[i];
        fn.arg_attrs.push_back(d);
      }
      if (b.Byte() != 0)
        throw Fail("use-list orders are not supported");
    }
    if (names.array.size() != fn.args.size() || types.array.size() != fn.args.size())
      throw Fail("byre_arg_names / byre_arg_types do not match the arguments of " + fn.name);
    for (uint64_t i = 0; i < n_ops; ++i)
      ReadBodyOp(b, &fn);
  }

  void ReadBodyOp(Reader &r, Function *fn) {
    OpHeader h = ReadOpHeader(r);
    if (h.regions != 0)
      throw Fail("op " + h.name + " has a region");
    Operation op;
    op.index = (int)fn->ops.size();
    op.line = op.index + 1; // bytecode has no lines: the op's position stands in
    for (int v : h.operands) {
      v -= (int)value_base_;
      if (v < 0 || (size_t)v >= fn->values.size())
        throw Fail("operand of " + h.name + " refers to a value that is not defined yet");
      op.operands.push_back(v);
    }
    auto add_results = [&]() {
      for (int ti : h.result_types) {
        const SerialType &t = Type((uint64_t)ti);
        if (t.kind != SerialType::kMemref)
          throw Fail("result of " + h.name + " is not a memref");
        Value v;
        v.id = (int)fn->values.size();
        v.name = "%" + std::to_string(v.id - (int)fn->args.size());
        v.type.dtype = t.dtype;
        v.type.shape = t.shape;
        v.type.space = t.space;
        v.defining_op = op.index;
        op.results.push_back(v.id);
        fn->values.push_back(v);
      }
    };
    if (h.name == "return_v1") {
      op.name = "func.return";
      op.operands.clear();
    } else if (h.name == "compute_v1") { // callee, extra_args?, memory_effects?
      const std::vector<int> p = ReadProps(h, {false, true, true});
      op.name = "byre.compute";
      op.callee = Plain(p[0]).s;
      if (p[1] >= 0) {
        const SerialAttr &extra = Attr((uint64_t)p[1]);
        if (!extra.is_dict)
          throw Fail("extra_args of compute_v1 is not a dictionary");
        for (auto &kv : extra.dict)
          op.attrs[kv.first] = Plain((uint64_t)kv.second);
      }
      if (p[2] >= 0)
        op.attrs["memory_effects"] = Plain((uint64_t)p[2]);
      add_results();
    } else if (h.name == "alias") { // offset
      const std::vector<int> p = ReadProps(h, {false});
      op.name = "byre.alias";
      op.callee = "AliasOp";
      op.attrs["offset"] = Plain((uint64_t)p[0]);
      if (op.operands.size() != 1 || h.result_types.size() != 1)
        throw Fail("alias takes one operand and gives one result");
      add_results();
    } else if (h.name == "alloc_v1") { // alignment?, operand_segment_sizes
      const std::vector<int> p = ReadProps(h, {true, false});
      op.name = "memref.alloc";
      if (!op.operands.empty())
        throw Fail("dynamic shapes are not supported (alloc_v1 with operands)");
      if (p[0] >= 0)
        op.attrs["alignment"] = Plain((uint64_t)p[0]);
      if (h.result_types.size() != 1)
        throw Fail("alloc_v1 gives one result");
      add_results();
    } else if (h.name == "copy_v1") { // callee
      const std::vector<int> p = ReadProps(h, {false});
      op.name = "byre.copy";
      op.attrs["callee"] = Plain((uint64_t)p[0]);
      op.callee = op.attrs["callee"].s;
      if (op.operands.size() != 2)
        throw Fail("copy_v1 takes a source and a target");
    } else if (h.name == "group_copy_v1") { // callee; operands: the sources, then as many targets
      // (compiler/include/byteir/Dialect/Byre/Serialization/ByreSerial.td:407-413, SameVariadicOperandSize:
      // no segment sizes are stored).  A group copy is its copies, source i -> target i, in order.
      const std::vector<int> p = ReadProps(h, {false});
      const std::string callee = Plain((uint64_t)p[0]).s;
      if (op.operands.empty() || op.operands.size() % 2 != 0)
        throw Fail("group_copy_v1 takes as many targets as sources");
      const size_t pairs = op.operands.size() / 2;
      for (size_t i = 0; i < pairs; ++i) {
        Operation one;
        one.name = "byre.copy";
        one.index = (int)fn->ops.size();
        one.line = one.index + 1;
        one.operands = {op.operands[i], op.operands[pairs + i]};
        one.attrs["callee"] = Plain((uint64_t)p[0]);
        one.callee = callee;
        fn->ops.push_back(std::move(one));
      }
      return;
    } else {
      throw Fail("byre_serial op " + h.name + " is not supported");
    }
    fn->ops.push_back(std::move(op));
  }

  const uint8_t *d_;
  size_t n_;
  std::vector<std::string> strings_, dialects_;
  std::vector<std::pair<int, std::string>> op_names_;
  std::vector<Entry> attr_entries_, type_entries_;
  std::vector<SerialAttr> attrs_;
  std::vector<SerialType> types_;
  std::vector<char> attr_done_, type_done_;
  std::vector<std::pair<size_t, size_t>> props_;
  std::unique_ptr<Module> module_;
  size_t scope_values_ = 0, value_base_ = 0;
};

} // namespace

bool IsByREBytecode(const void *data, size_t size) {
  return size >= 4 && std::memcmp(data, "ML\xefR", 4) == 0;
}

std::unique_ptr<Module> ParseByREBytecode(const void *data, size_t size, std::string *error) {
  try {
    return Decoder(static_cast<const uint8_t *>(data), size).Run();
  } catch (const std::exception &e) {
    if (error)
      *error = std::string("bytecode: ") + e.what();
    return nullptr;
  }
}

} // namespace ir
} // namespace brt
