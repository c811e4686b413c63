// Hand-written parser for the textual ByRE subset.  It reads what byteir-opt's
// byre pipeline prints (and what the reference's hand-written test fixtures
// contain): generic and custom op forms, the attribute spellings
// `1 : i64`, `0.5 : f32`, "str", true, unit, [a, b], {k = v}, array<i64: 1, 2>,
// dense<1> : tensor<1xi64>, dense<[3, 2]> : tensor<2xi64>, and the `<{...}>`
// property dictionary.  Anything it does not understand inside an attribute
// (affine maps, dialect attributes) is kept as an opaque string.
#include "brt/core/ir/ir.h"

#include <cctype>
#include <cstdlib>
#include <map>
#include <stdexcept>

namespace brt {
namespace ir {

int64_t MemRefType::NumElements() const {
  int64_t n = 1;
  for (auto d : shape)
    n *= d;
  return n;
}

size_t MemRefType::SizeInBytes() const {
  int64_t n = NumElements();
  return n < 0 ? 0 : (size_t)n * GetDTypeByte(dtype);
}

namespace {

struct ParseError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

class Parser {
public:
  explicit Parser(const std::string &text) : s_(text) {}

  std::unique_ptr<Module> ParseModule() {
    auto m = std::make_unique<Module>();
    SkipWs();
    if (TryKeyword("module")) {
      SkipWs();
      if (Peek() == '@')
        m->name = ParseSymbol();
      SkipWs();
      if (TryKeyword("attributes")) {
        SkipWs();
        m->attrs = ParseAttrDict();
      }
      Expect('{');
      ParseFunctions(m.get(), /*until_brace=*/true);
      Expect('}');
    } else {
      ParseFunctions(m.get(), /*until_brace=*/false);
    }
    SkipWs();
    if (!AtEnd())
      Fail("unexpected text after the module");
    return m;
  }

private:
  const std::string &s_;
  size_t pos_ = 0;
  Function *fn_ = nullptr;
  std::map<std::string, int> value_ids_;

  // ---- character level -----------------------------------------------------
  bool AtEnd() const { return pos_ >= s_.size(); }
  char Peek(size_t k = 0) const { return pos_ + k < s_.size() ? s_[pos_ + k] : '\0'; }
  int Line() const {
    int line = 1;
    for (size_t i = 0; i < pos_ && i < s_.size(); ++i)
      if (s_[i] == '\n')
        ++line;
    return line;
  }
  [[noreturn]] void Fail(const std::string &msg) const {
    throw ParseError("line " + std::to_string(Line()) + ": " + msg);
  }
  void SkipWs() {
    for (;;) {
      while (!AtEnd() && std::isspace((unsigned char)Peek()))
        ++pos_;
      if (Peek() == '/' && Peek(1) == '/') {
        while (!AtEnd() && Peek() != '\n')
          ++pos_;
        continue;
      }
      break;
    }
  }
  bool TryChar(char c) {
    SkipWs();
    if (Peek() == c) {
      ++pos_;
      return true;
    }
    return false;
  }
  void Expect(char c) {
    if (!TryChar(c))
      Fail(std::string("expected '") + c + "' but found '" + (AtEnd() ? std::string("<eof>") : std::string(1, Peek())) + "'");
  }
  static bool IsIdentChar(char c) {
    return std::isalnum((unsigned char)c) || c == '_' || c == '.' || c == '$' || c == '-';
  }
  bool TryKeyword(const char *kw) {
    SkipWs();
    size_t n = std::char_traits<char>::length(kw);
    if (s_.compare(pos_, n, kw) == 0 && !(IsIdentChar(Peek(n)) && Peek(n) != '-')) {
      pos_ += n;
      return true;
    }
    return false;
  }
  std::string ParseBareIdent() {
    SkipWs();
    size_t b = pos_;
    while (!AtEnd() && (std::isalnum((unsigned char)Peek()) || Peek() == '_' || Peek() == '.' || Peek() == '$'))
      ++pos_;
    if (b == pos_)
      Fail("expected an identifier");
    return s_.substr(b, pos_ - b);
  }
  std::string ParseString() {
    SkipWs();
    if (Peek() != '"')
      Fail("expected a string");
    ++pos_;
    std::string out;
    while (!AtEnd() && Peek() != '"') {
      if (Peek() == '\\' && pos_ + 1 < s_.size()) {
        char n = s_[pos_ + 1];
        if (n == 'n')
          out += '\n';
        else if (n == 't')
          out += '\t';
        else if (std::isxdigit((unsigned char)n) && pos_ + 2 < s_.size() && std::isxdigit((unsigned char)s_[pos_ + 2])) {
          out += (char)std::strtol(s_.substr(pos_ + 1, 2).c_str(), nullptr, 16);
          ++pos_;
        } else
          out += n;
        pos_ += 2;
      } else {
        out += s_[pos_++];
      }
    }
    if (AtEnd())
      Fail("unterminated string");
    ++pos_;
    return out;
  }
  std::string ParseSymbol() { // @name or @"name"
    SkipWs();
    if (Peek() != '@')
      Fail("expected a symbol name");
    ++pos_;
    if (Peek() == '"')
      return ParseString();
    return ParseBareIdent();
  }
  std::string ParseValueName() { // %name, %0, %arg0#1 is not used by ByRE
    SkipWs();
    if (Peek() != '%')
      Fail("expected an SSA value");
    size_t b = pos_++;
    while (!AtEnd() && (std::isalnum((unsigned char)Peek()) || Peek() == '_' || Peek() == '.' || Peek() == '$' || Peek() == '-'))
      ++pos_;
    return s_.substr(b, pos_ - b);
  }
  // text between balanced brackets starting at the current opening bracket
  std::string ParseBalanced() {
    SkipWs();
    size_t b = pos_;
    int depth = 0;
    do {
      if (AtEnd())
        Fail("unbalanced brackets");
      char c = s_[pos_];
      if (c == '"') {
        ParseString();
        continue;
      }
      if (c == '<' || c == '(' || c == '[' || c == '{')
        ++depth;
      else if (c == '>' || c == ')' || c == ']' || c == '}') {
        if (c == '>' && pos_ > 0 && s_[pos_ - 1] == '-') { // "->" inside a map
          ++pos_;
          continue;
        }
        --depth;
      }
      ++pos_;
    } while (depth > 0);
    return s_.substr(b, pos_ - b);
  }

  // ---- types -----------------------------------------------------------------
  static bool IsShapedKeyword(const std::string &w) { return w == "memref" || w == "tensor" || w == "vector"; }

  // returns true and fills `out` for memref/tensor types; other types are skipped
  bool ParseType(MemRefType *out, std::string *spelled = nullptr) {
    SkipWs();
    size_t b = pos_;
    if (Peek() == '(') { // function type
      ParseBalanced();
      SkipWs();
      if (Peek() == '-' && Peek(1) == '>') {
        pos_ += 2;
        MemRefType dummy;
        ParseType(&dummy);
      }
      if (spelled)
        *spelled = s_.substr(b, pos_ - b);
      return false;
    }
    if (Peek() == '!') { // dialect type such as !ace.string
      ++pos_;
      ParseBareIdent();
      SkipWs();
      if (Peek() == '<')
        ParseBalanced();
      if (spelled)
        *spelled = s_.substr(b, pos_ - b);
      return false;
    }
    std::string word = ParseBareIdent();
    if (IsShapedKeyword(word)) {
      Expect('<');
      *out = ParseShapedBody();
      if (spelled)
        *spelled = s_.substr(b, pos_ - b);
      return true;
    }
    SkipWs();
    if (Peek() == '<')
      ParseBalanced();
    out->dtype = DTypeFromName(word);
    out->shape.clear();
    if (spelled)
      *spelled = s_.substr(b, pos_ - b);
    return false;
  }

  // after "memref<": dims 'x' element-type [, layout] [, memory space] '>'
  MemRefType ParseShapedBody() {
    MemRefType t;
    for (;;) {
      SkipWs();
      if (Peek() == '?') {
        ++pos_;
        t.shape.push_back(-1);
      } else if (std::isdigit((unsigned char)Peek())) {
        size_t b = pos_;
        while (std::isdigit((unsigned char)Peek()))
          ++pos_;
        t.shape.push_back(std::strtoll(s_.substr(b, pos_ - b).c_str(), nullptr, 10));
      } else if (Peek() == '*') { // unranked
        ++pos_;
      } else {
        break;
      }
      if (Peek() != 'x')
        Fail("expected 'x' after a dimension");
      ++pos_;
    }
    SkipWs();
    if (Peek() == '!') {
      ++pos_;
      std::string w = ParseBareIdent();
      t.dtype = DTypeFromName("!" + w);
    } else {
      std::string w = ParseBareIdent();
      t.dtype = DTypeFromName(w);
      if (t.dtype == DTypeEnum::Invalid)
        Fail("unknown element type '" + w + "'");
    }
    while (TryChar(',')) {
      SkipWs();
      if (Peek() == '"') {
        t.space = ParseString();
      } else if (std::isdigit((unsigned char)Peek())) { // integer memory space
        size_t b = pos_;
        while (std::isdigit((unsigned char)Peek()))
          ++pos_;
        t.space = s_.substr(b, pos_ - b);
      } else { // layout: affine_map<...>, strided<...>, #map
        if (Peek() == '#')
          ++pos_;
        ParseBareIdent();
        SkipWs();
        if (Peek() == '<')
          ParseBalanced();
      }
    }
    Expect('>');
    return t;
  }

  // ---- attributes ------------------------------------------------------------
  AttrDict ParseAttrDict() {
    AttrDict d;
    Expect('{');
    SkipWs();
    if (TryChar('}'))
      return d;
    for (;;) {
      SkipWs();
      std::string key = Peek() == '"' ? ParseString() : ParseBareIdent();
      Attribute a;
      if (TryChar('='))
        a = ParseAttr();
      d[key] = a;
      if (TryChar(','))
        continue;
      Expect('}');
      break;
    }
    return d;
  }

  bool LooksLikeNumber() {
    SkipWs();
    char c = Peek();
    if (std::isdigit((unsigned char)c))
      return true;
    if ((c == '-' || c == '+') && (std::isdigit((unsigned char)Peek(1)) || Peek(1) == '.'))
      return true;
    return false;
  }

  // number with optional ": type" suffix
  Attribute ParseNumberAttr() {
    SkipWs();
    size_t b = pos_;
    if (Peek() == '-' || Peek() == '+')
      ++pos_;
    bool is_float = false, is_hex = false;
    if (Peek() == '0' && (Peek(1) == 'x' || Peek(1) == 'X')) {
      is_hex = true;
      pos_ += 2;
      while (std::isxdigit((unsigned char)Peek()))
        ++pos_;
    } else {
      while (std::isdigit((unsigned char)Peek()))
        ++pos_;
      if (Peek() == '.') {
        is_float = true;
        ++pos_;
        while (std::isdigit((unsigned char)Peek()))
          ++pos_;
      }
      if (Peek() == 'e' || Peek() == 'E') {
        size_t save = pos_;
        ++pos_;
        if (Peek() == '-' || Peek() == '+')
          ++pos_;
        if (std::isdigit((unsigned char)Peek())) {
          is_float = true;
          while (std::isdigit((unsigned char)Peek()))
            ++pos_;
        } else {
          pos_ = save;
        }
      }
    }
    std::string tok = s_.substr(b, pos_ - b);
    Attribute a;
    DTypeEnum ty = DTypeEnum::Invalid;
    size_t save = pos_;
    if (TryChar(':')) {
      MemRefType t;
      SkipWs();
      if (std::isalpha((unsigned char)Peek()) || Peek() == '!') {
        ParseType(&t);
        ty = t.dtype;
      } else {
        pos_ = save;
      }
    }
    const bool float_type = ty == DTypeEnum::Float32 || ty == DTypeEnum::Float64 || ty == DTypeEnum::Float16 ||
                            ty == DTypeEnum::BFloat16;
    if (is_float || (float_type && !is_hex)) {
      a.kind = Attribute::kFloat;
      a.f = std::strtod(tok.c_str(), nullptr);
      a.i = (int64_t)a.f;
      a.elt_type = ty == DTypeEnum::Invalid ? DTypeEnum::Float64 : ty;
    } else if (is_hex && float_type) { // bit pattern of a float
      a.kind = Attribute::kFloat;
      uint64_t bits = std::strtoull(tok.c_str(), nullptr, 16);
      if (ty == DTypeEnum::Float32) {
        uint32_t b32 = (uint32_t)bits;
        float f;
        __builtin_memcpy(&f, &b32, 4);
        a.f = f;
      } else {
        double d;
        __builtin_memcpy(&d, &bits, 8);
        a.f = d;
      }
      a.elt_type = ty;
    } else {
      a.kind = ty == DTypeEnum::Bool ? Attribute::kBool : Attribute::kInt;
      a.i = is_hex ? (int64_t)std::strtoull(tok.c_str(), nullptr, 16) : std::strtoll(tok.c_str(), nullptr, 10);
      a.f = (double)a.i;
      a.elt_type = ty == DTypeEnum::Invalid ? DTypeEnum::Int64 : ty;
    }
    return a;
  }

  void ParseDenseValues(Attribute *a, int depth, bool *any_float) {
    SkipWs();
    if (TryChar('[')) {
      SkipWs();
      if (TryChar(']'))
        return;
      for (;;) {
        ParseDenseValues(a, depth + 1, any_float);
        if (TryChar(','))
          continue;
        Expect(']');
        break;
      }
      return;
    }
    if (TryKeyword("true")) {
      a->dense_i.push_back(1);
      a->dense_f.push_back(1);
      a->splat = a->splat || depth == 0;
      return;
    }
    if (TryKeyword("false")) {
      a->dense_i.push_back(0);
      a->dense_f.push_back(0);
      a->splat = a->splat || depth == 0;
      return;
    }
    if (Peek() == '"') { // hex blob: keep the text, values unavailable
      a->s = ParseString();
      return;
    }
    if (!LooksLikeNumber())
      Fail("expected a number in dense<...>");
    size_t b = pos_;
    if (Peek() == '-' || Peek() == '+')
      ++pos_;
    bool fl = false;
    while (std::isdigit((unsigned char)Peek()) || Peek() == '.' || Peek() == 'e' || Peek() == 'E' ||
           ((Peek() == '-' || Peek() == '+') && (s_[pos_ - 1] == 'e' || s_[pos_ - 1] == 'E'))) {
      if (Peek() == '.' || Peek() == 'e' || Peek() == 'E')
        fl = true;
      ++pos_;
    }
    std::string tok = s_.substr(b, pos_ - b);
    double d = std::strtod(tok.c_str(), nullptr);
    a->dense_f.push_back(d);
    a->dense_i.push_back(fl ? (int64_t)d : std::strtoll(tok.c_str(), nullptr, 10));
    if (fl)
      *any_float = true;
    if (depth == 0)
      a->splat = true;
  }

  Attribute ParseAttr() {
    SkipWs();
    Attribute a;
    char c = Peek();
    if (c == '"') {
      a.kind = Attribute::kString;
      a.s = ParseString();
      size_t save = pos_;
      if (TryChar(':')) { // typed string attr
        MemRefType t;
        SkipWs();
        if (std::isalpha((unsigned char)Peek()) || Peek() == '!')
          ParseType(&t);
        else
          pos_ = save;
      }
      return a;
    }
    if (c == '[') {
      a.kind = Attribute::kArray;
      ++pos_;
      SkipWs();
      if (TryChar(']'))
        return a;
      for (;;) {
        a.array.push_back(ParseAttr());
        if (TryChar(','))
          continue;
        Expect(']');
        break;
      }
      return a;
    }
    if (c == '{') { // nested dictionary: keep as opaque text
      a.kind = Attribute::kString;
      a.s = ParseBalanced();
      return a;
    }
    if (LooksLikeNumber())
      return ParseNumberAttr();
    if (c == '#' || c == '@') { // dialect attribute alias or symbol reference
      size_t b = pos_++;
      if (Peek() == '"')
        ParseString();
      else
        ParseBareIdent();
      SkipWs();
      if (Peek() == '<')
        ParseBalanced();
      a.kind = Attribute::kString;
      a.s = s_.substr(b, pos_ - b);
      return a;
    }
    if (TryKeyword("true")) {
      a.kind = Attribute::kBool;
      a.i = 1;
      return a;
    }
    if (TryKeyword("false")) {
      a.kind = Attribute::kBool;
      a.i = 0;
      return a;
    }
    if (TryKeyword("unit")) {
      a.kind = Attribute::kUnit;
      return a;
    }
    if (TryKeyword("dense")) {
      Expect('<');
      bool any_float = false;
      SkipWs();
      if (Peek() != '>')
        ParseDenseValues(&a, 0, &any_float);
      Expect('>');
      MemRefType t;
      if (TryChar(':')) {
        ParseType(&t);
        a.dense_shape = t.shape;
        a.elt_type = t.dtype;
      }
      const bool float_type = a.elt_type == DTypeEnum::Float32 || a.elt_type == DTypeEnum::Float64 ||
                              a.elt_type == DTypeEnum::Float16 || a.elt_type == DTypeEnum::BFloat16;
      a.kind = (any_float || float_type) ? Attribute::kDenseFloat : Attribute::kDenseInt;
      return a;
    }
    if (TryKeyword("array")) { // array<i64: 1, 2> or array<i64>
      Expect('<');
      MemRefType t;
      ParseType(&t);
      a.elt_type = t.dtype;
      a.kind = Attribute::kDenseInt;
      if (TryChar(':')) {
        bool any_float = false;
        for (;;) {
          ParseDenseValues(&a, 1, &any_float);
          if (!TryChar(','))
            break;
        }
        if (any_float)
          a.kind = Attribute::kDenseFloat;
      }
      a.splat = false;
      a.dense_shape = {(int64_t)a.dense_i.size()};
      Expect('>');
      return a;
    }
    // a type used as an attribute, or a dialect keyword attribute such as affine_map<...>
    size_t b = pos_;
    MemRefType t;
    std::string spelled;
    ParseType(&t, &spelled);
    (void)b;
    a.kind = Attribute::kType;
    a.s = spelled;
    a.elt_type = t.dtype;
    return a;
  }

  // ---- functions and ops -------------------------------------------------------
  void ParseFunctions(Module *m, bool until_brace) {
    for (;;) {
      SkipWs();
      if (AtEnd() || (until_brace && Peek() == '}'))
        return;
      if (TryKeyword("func.func") || TryKeyword("func")) {
        m->functions.emplace_back();
        ParseFunction(&m->functions.back());
      } else if (TryKeyword("gpu.module") || TryKeyword("memref.global")) {
        // device code and globals ride along in some modules: skip to the end of the item
        SkipItem();
      } else {
        Fail("expected func.func");
      }
    }
  }

  void SkipItem() {
    // skip to the first '{' at depth 0 and past its matching '}', or to end of line
    while (!AtEnd() && Peek() != '{' && Peek() != '\n') {
      if (Peek() == '"')
        ParseString();
      else
        ++pos_;
    }
    if (Peek() == '{')
      ParseBalanced();
  }

  int NewValue(const std::string &name, const MemRefType &type, int arg_index, int def_op) {
    Value v;
    v.id = (int)fn_->values.size();
    v.name = name;
    v.type = type;
    v.arg_index = arg_index;
    v.defining_op = def_op;
    fn_->values.push_back(v);
    value_ids_[name] = v.id;
    return v.id;
  }

  int LookupValue(const std::string &name) {
    auto it = value_ids_.find(name);
    if (it == value_ids_.end())
      Fail("use of undefined value " + name);
    return it->second;
  }

  void ParseFunction(Function *f) {
    fn_ = f;
    value_ids_.clear();
    SkipWs();
    if (TryKeyword("private") || TryKeyword("public")) {
    }
    f->name = ParseSymbol();
    Expect('(');
    SkipWs();
    if (!TryChar(')')) {
      for (;;) {
        std::string name = ParseValueName();
        Expect(':');
        MemRefType t;
        ParseType(&t);
        AttrDict attrs;
        SkipWs();
        if (Peek() == '{')
          attrs = ParseAttrDict();
        int id = NewValue(name, t, (int)f->args.size(), -1);
        f->args.push_back(id);
        f->arg_attrs.push_back(attrs);
        if (TryChar(','))
          continue;
        Expect(')');
        break;
      }
    }
    SkipWs();
    if (Peek() == '-' && Peek(1) == '>') {
      pos_ += 2;
      SkipWs();
      if (Peek() == '(')
        ParseBalanced();
      else {
        MemRefType t;
        ParseType(&t);
      }
    }
    if (TryKeyword("attributes"))
      f->attrs = ParseAttrDict();
    SkipWs();
    if (Peek() != '{')
      return; // declaration only
    Expect('{');
    for (;;) {
      SkipWs();
      if (TryChar('}'))
        break;
      if (AtEnd())
        Fail("unterminated function body");
      ParseOperation();
    }
    fn_ = nullptr;
  }

  void ParseTypeListInto(std::vector<MemRefType> *types) {
    // either "(t, t)" or "t, t" or "()"
    SkipWs();
    if (Peek() == '(') {
      ++pos_;
      SkipWs();
      if (TryChar(')'))
        return;
      for (;;) {
        MemRefType t;
        ParseType(&t);
        types->push_back(t);
        if (TryChar(','))
          continue;
        Expect(')');
        break;
      }
      return;
    }
    for (;;) {
      MemRefType t;
      ParseType(&t);
      types->push_back(t);
      if (!TryChar(','))
        break;
    }
  }

  void MergeProps(Operation *op) {
    // `<{...}>` property dictionary right after the operand list
    SkipWs();
    if (Peek() == '<' && Peek(1) == '{') {
      ++pos_;
      AttrDict props = ParseAttrDict();
      Expect('>');
      for (auto &kv : props)
        op->attrs[kv.first] = kv.second;
    }
  }

  void ParseOperation() {
    Operation op;
    op.line = Line();
    std::vector<std::string> result_names;
    SkipWs();
    if (Peek() == '%') {
      for (;;) {
        result_names.push_back(ParseValueName());
        SkipWs();
        if (Peek() == ':') { // %r:2 packs are not used by ByRE
          Fail("multi-result packs are not supported");
        }
        if (TryChar(','))
          continue;
        break;
      }
      Expect('=');
    }
    SkipWs();
    bool generic = Peek() == '"';
    op.name = generic ? ParseString() : ParseBareIdent();
    std::vector<MemRefType> operand_types, result_types;

    auto parse_operands_paren = [&]() {
      Expect('(');
      SkipWs();
      if (TryChar(')'))
        return;
      for (;;) {
        op.operands.push_back(LookupValue(ParseValueName()));
        if (TryChar(','))
          continue;
        Expect(')');
        break;
      }
    };

    if (generic) {
      parse_operands_paren();
      MergeProps(&op);
      SkipWs();
      if (Peek() == '(') // regions are not part of ByRE entry functions
        Fail("ops with regions are not supported");
      if (Peek() == '{') {
        AttrDict d = ParseAttrDict();
        for (auto &kv : d)
          op.attrs[kv.first] = kv.second;
      }
      Expect(':');
      ParseTypeListInto(&operand_types);
      SkipWs();
      if (Peek() == '-' && Peek(1) == '>') {
        pos_ += 2;
        ParseTypeListInto(&result_types);
      }
    } else if (op.name == "return" || op.name == "func.return") {
      SkipWs();
      if (Peek() == '%') { // ByRE entry functions return nothing; tolerate and ignore operands
        while (Peek() != '\n' && !AtEnd())
          ++pos_;
      }
      op.name = "func.return";
    } else if (op.name == "byre.compute") {
      op.callee = ParseSymbol();
      parse_operands_paren();
      MergeProps(&op);
      SkipWs();
      if (Peek() == '{') {
        AttrDict d = ParseAttrDict();
        for (auto &kv : d)
          op.attrs[kv.first] = kv.second;
      }
      if (TryChar(':'))
        ParseTypeListInto(&operand_types);
    } else if (op.name == "byre.copy") {
      parse_operands_paren();
      SkipWs();
      if (Peek() == '{') {
        AttrDict d = ParseAttrDict();
        for (auto &kv : d)
          op.attrs[kv.first] = kv.second;
      }
      if (TryChar(':'))
        ParseTypeListInto(&operand_types);
    } else if (op.name == "memref.alloc" || op.name == "memref.alloca") {
      Expect('(');
      Expect(')');
      SkipWs();
      if (Peek() == '{') {
        AttrDict d = ParseAttrDict();
        for (auto &kv : d)
          op.attrs[kv.first] = kv.second;
      }
      Expect(':');
      MemRefType t;
      if (!ParseType(&t))
        Fail("memref.alloc needs a memref type");
      result_types.push_back(t);
    } else if (op.name == "byre.alias") {
      // custom form: byre.alias %src {offset = N : i64} : memref<..> to memref<..>
      SkipWs();
      if (Peek() == '(')
        parse_operands_paren();
      else
        op.operands.push_back(LookupValue(ParseValueName()));
      MergeProps(&op);
      SkipWs();
      if (Peek() == '{') {
        AttrDict d = ParseAttrDict();
        for (auto &kv : d)
          op.attrs[kv.first] = kv.second;
      }
      Expect(':');
      ParseTypeListInto(&operand_types);
      SkipWs();
      if (TryKeyword("to") || (Peek() == '-' && Peek(1) == '>' && (pos_ += 2))) {
        ParseTypeListInto(&result_types);
      }
    } else {
      Fail("unsupported op '" + op.name + "' (only the ByRE op set is understood)");
    }

    // callee: the registry key
    if (op.callee.empty()) {
      auto it = op.attrs.find("callee");
      if (it != op.attrs.end() && it->second.kind == Attribute::kString)
        op.callee = it->second.s;
      else if (op.name == "byre.alias")
        op.callee = "AliasOp";
    }
    if (op.name == "byre.compute" && op.attrs.count("callee") == 0 && generic) {
      Fail("generic byre.compute without a callee attribute");
    }

    if (!operand_types.empty() && operand_types.size() != op.operands.size())
      Fail("operand count and type count differ for " + op.name);
    if (result_names.size() != result_types.size() && !result_names.empty())
      Fail("result count and result type count differ for " + op.name);
    op.index = (int)fn_->ops.size();
    for (size_t i = 0; i < result_names.size(); ++i)
      op.results.push_back(NewValue(result_names[i], result_types[i], -1, op.index));
    fn_->ops.push_back(std::move(op));
  }
};

} // namespace

std::unique_ptr<Module> ParseByRE(const std::string &text, std::string *error) {
  try {
    Parser p(text);
    return p.ParseModule();
  } catch (const ParseError &e) {
    if (error)
      *error = e.what();
    return nullptr;
  }
}

} // namespace ir
} // namespace brt
