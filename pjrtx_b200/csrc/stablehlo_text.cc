// StableHLO text -> ExecutablePlan for the subset of operations the backend executes.
//
// The reference imports StableHLO through MLIR (src/compiler/stablehlo_module_import.zig:241-264,
// stablehlo_operation_import.zig:22-456, stablehlo_operation_attrs.zig:222-246 for the reduce body rule,
// stablehlo_sharding.zig:40-93 for sdy shardings); neither MLIR nor the bytecode reader is available here, so this is
// a reader of the textual form only: `func.func @main`, tensor types with static shapes, the pretty and the generic
// operation syntax, dense constants, integer-list / array / dot / gather attributes, `sdy.sharding` and donation
// attributes on arguments. Anything outside the subset stops the import with one diagnostic line in the reference's
// format (stablehlo_decode.zig:117-140):
//   unsupported op: op=<name> loc=L:C dtype=<t> rank=<r|unknown> sharding=<...> feature=stablehlo-op
// Malformed text is reported as
//   invalid module: loc=L:C detail="..." feature=stablehlo-text
#include "stablehlo_text.h"

#include <cctype>
#include <cmath>
#include <cstring>
#include <map>

namespace pjrtx {

namespace {

struct Fail {
  std::string why;
};

struct Type {
  bool tensor = false;
  int dtype = kInvalid;
  std::vector<int64_t> dims;
  std::string text;  // for diagnostics
};

// Value of an attribute as far as the importer needs it.
struct Attr {
  std::vector<int64_t> ints;          // [1, 2] / array<i64: 1, 2> / dense<[1, 2]> : tensor<2xi64> / 3 : i64 / true
  std::vector<int64_t> ints2;         // second list of `[..] x [..]`
  std::string text;                   // string literal or bare word
  std::map<std::string, std::vector<int64_t>> fields;  // #stablehlo.dot<...> / #stablehlo.gather<...>
  bool has_ints = false;
};

uint16_t float_to_half_bits(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
  uint32_t man = x & 0x7fffffu;
  if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t h = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1))) h++;
    return (uint16_t)(sign | h);
  }
  uint32_t h = ((uint32_t)exp << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) h++;
  return (uint16_t)(sign | h);
}

uint16_t float_to_bf16_bits(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u);  // quiet NaN
  x += 0x7fffu + ((x >> 16) & 1);
  return (uint16_t)(x >> 16);
}

class Parser {
 public:
  explicit Parser(const std::string& text) : s_(text) {}

  Plan run() {
    plan_.num_replicas = 1;
    plan_.num_partitions = 1;
    skip();
    bool found = false;
    while (pos_ < s_.size()) {
      skip();
      if (pos_ >= s_.size()) break;
      if (try_word("module")) {
        // module [@name] [attributes {...}] {
        skip();
        if (peek() == '@') symbol();
        skip();
        if (try_word("attributes")) skip_balanced();
        expect('{');
        continue;
      }
      if (peek() == '}') {
        pos_++;
        continue;
      }
      if (try_word("sdy.mesh")) {
        parse_mesh();
        continue;
      }
      if (try_word("func.func")) {
        const bool is_main = parse_function(!found);
        found |= is_main;
        continue;
      }
      fail("expected module, func.func or sdy.mesh");
    }
    if (!found) fail("no func.func @main in the module");
    while ((int)plan_.device_assignment.size() < plan_.num_replicas * plan_.num_partitions)
      plan_.device_assignment.push_back((int32_t)plan_.device_assignment.size());
    return plan_;
  }

  std::string location() const {
    size_t line = 1, col = 1;
    for (size_t i = 0; i < pos_ && i < s_.size(); i++) {
      if (s_[i] == '\n') {
        line++;
        col = 1;
      } else {
        col++;
      }
    }
    return strfmt("%zu:%zu", line, col);
  }

 private:
  const std::string& s_;
  size_t pos_ = 0;
  Plan plan_;
  std::map<std::string, std::vector<uint32_t>> names_;  // %name -> value ids (several for multi-result operations)
  std::map<std::string, int64_t> mesh_size_;

  [[noreturn]] void fail(const std::string& why) { throw Fail{strfmt("invalid module: loc=%s detail=\"%s\" feature=stablehlo-text", location().c_str(), why.c_str())}; }
  [[noreturn]] void unsupported(const std::string& op, size_t at, const Type* t) {
    const size_t keep = pos_;
    pos_ = at;
    const std::string loc = location();
    pos_ = keep;
    throw Fail{strfmt("unsupported op: op=%s loc=%s dtype=%s rank=%s sharding=unspecified feature=stablehlo-op", op.c_str(), loc.c_str(),
                      t && t->tensor ? dtype_name(t->dtype) : "unknown",
                      t && t->tensor ? std::to_string(t->dims.size()).c_str() : "unknown")};
  }

  // ---- characters ---------------------------------------------------------------------------------------------
  void skip() {
    while (pos_ < s_.size()) {
      if (isspace((unsigned char)s_[pos_])) {
        pos_++;
      } else if (s_[pos_] == '/' && pos_ + 1 < s_.size() && s_[pos_ + 1] == '/') {
        while (pos_ < s_.size() && s_[pos_] != '\n') pos_++;
      } else {
        break;
      }
    }
  }
  char peek() {
    skip();
    return pos_ < s_.size() ? s_[pos_] : '\0';
  }
  bool try_eat(char c) {
    if (peek() == c) {
      pos_++;
      return true;
    }
    return false;
  }
  void expect(char c) {
    if (!try_eat(c)) fail(strfmt("expected '%c'", c));
  }
  bool try_str(const char* lit) {
    skip();
    const size_t n = strlen(lit);
    if (s_.compare(pos_, n, lit) == 0) {
      pos_ += n;
      return true;
    }
    return false;
  }
  static bool word_char(char c) { return isalnum((unsigned char)c) || c == '_' || c == '.' || c == '$'; }
  // A bare word that must end at a non-word character.
  bool try_word(const char* lit) {
    skip();
    const size_t n = strlen(lit);
    if (s_.compare(pos_, n, lit) == 0 && (pos_ + n >= s_.size() || !word_char(s_[pos_ + n]))) {
      pos_ += n;
      return true;
    }
    return false;
  }
  std::string word() {
    skip();
    size_t b = pos_;
    while (pos_ < s_.size() && word_char(s_[pos_])) pos_++;
    if (b == pos_) fail("expected an identifier");
    return s_.substr(b, pos_ - b);
  }
  std::string symbol() {  // @name
    expect('@');
    if (peek() == '"') return string_literal();
    return word();
  }
  std::string string_literal() {
    expect('"');
    std::string out;
    while (pos_ < s_.size() && s_[pos_] != '"') {
      if (s_[pos_] == '\\' && pos_ + 1 < s_.size()) pos_++;
      out += s_[pos_++];
    }
    if (pos_ >= s_.size()) fail("unterminated string");
    pos_++;
    return out;
  }
  int64_t integer() {
    skip();
    size_t b = pos_;
    if (pos_ < s_.size() && (s_[pos_] == '-' || s_[pos_] == '+')) pos_++;
    while (pos_ < s_.size() && isdigit((unsigned char)s_[pos_])) pos_++;
    if (b == pos_ || (pos_ == b + 1 && !isdigit((unsigned char)s_[b]))) fail("expected an integer");
    return strtoll(s_.substr(b, pos_ - b).c_str(), nullptr, 10);
  }
  // Skips one balanced group or token sequence up to (not including) a top-level ',' or closing bracket.
  void skip_balanced() {
    skip();
    int depth = 0;
    while (pos_ < s_.size()) {
      const char c = s_[pos_];
      if (c == '"') {
        string_literal();
        continue;
      }
      if (c == '(' || c == '[' || c == '{' || c == '<') depth++;
      if (c == ')' || c == ']' || c == '}' || c == '>') {
        if (c == '>' && pos_ > 0 && s_[pos_ - 1] == '-') {  // "->" is not a bracket
          pos_++;
          continue;
        }
        if (depth == 0) return;
        depth--;
        pos_++;
        if (depth == 0) {
          // a group just closed: a following group or suffix (": type") belongs to the same value only for attributes
          return;
        }
        continue;
      }
      if (depth == 0 && (c == ',' )) return;
      pos_++;
    }
  }

  // ---- types --------------------------------------------------------------------------------------------------
  static int element_type(const std::string& t) {
    static const std::map<std::string, int> kTypes = {
        {"f32", kF32}, {"f16", kF16}, {"bf16", kBF16}, {"f64", kF64}, {"i1", kPred},  {"i8", kS8},   {"si8", kS8},
        {"i16", kS16}, {"si16", kS16}, {"i32", kS32},  {"si32", kS32}, {"i64", kS64}, {"si64", kS64}, {"ui8", kU8},
        {"ui16", kU16}, {"ui32", kU32}, {"ui64", kU64}};
    auto it = kTypes.find(t);
    return it == kTypes.end() ? kInvalid : it->second;
  }
  Type parse_type() {
    skip();
    Type t;
    const size_t b = pos_;
    if (try_str("tensor<")) {
      t.tensor = true;
      // dims separated by 'x', then the element type
      while (true) {
        skip();
        if (isdigit((unsigned char)peek())) {
          size_t save = pos_;
          int64_t d = integer();
          if (pos_ < s_.size() && s_[pos_] == 'x') {
            pos_++;
            t.dims.push_back(d);
            continue;
          }
          pos_ = save;
          fail("malformed tensor shape");
        }
        if (peek() == '?') fail("dynamic dimensions are not supported");
        break;
      }
      const std::string et = word();
      if (et == "complex") {
        skip_balanced();
        t.dtype = kC64;
      } else {
        t.dtype = element_type(et);
        if (t.dtype == kInvalid) fail("unknown element type " + et);
      }
      skip();
      if (peek() == ',') {  // encoding attribute
        pos_++;
        skip_balanced();
      }
      expect('>');
    } else {
      // tuple<...>, !stablehlo.token, index ... : kept as text, refused where a tensor is needed
      word();
      if (peek() == '<') skip_balanced();
    }
    t.text = s_.substr(b, pos_ - b);
    return t;
  }
  std::vector<Type> parse_type_list_parens() {  // "(t, t)" or "()"
    std::vector<Type> out;
    expect('(');
    if (try_eat(')')) return out;
    do {
      out.push_back(parse_type());
      if (peek() == '{') skip_balanced();  // result attributes
    } while (try_eat(','));
    expect(')');
    return out;
  }

  // ---- attributes ---------------------------------------------------------------------------------------------
  std::vector<int64_t> int_list_brackets() {  // [1, 2, 3]
    std::vector<int64_t> out;
    expect('[');
    if (try_eat(']')) return out;
    do {
      out.push_back(integer());
    } while (try_eat(','));
    expect(']');
    return out;
  }
  Attr parse_attr_value() {
    Attr a;
    skip();
    const char c = peek();
    if (c == '[') {
      // integer list, or a list of words (precision configs)
      size_t save = pos_;
      pos_++;
      skip();
      if (peek() == ']' || isdigit((unsigned char)peek()) || peek() == '-') {
        pos_ = save;
        a.ints = int_list_brackets();
        a.has_ints = true;
        if (try_word("x")) a.ints2 = int_list_brackets();
      } else {
        pos_ = save;
        skip_group();
      }
      return a;
    }
    if (c == '"') {
      a.text = string_literal();
      return a;
    }
    if (c == '#' || c == '@' || c == '<') {
      if (try_str("#stablehlo.dot<") || try_str("#stablehlo.gather<") || try_str("#stablehlo.scatter<")) {
        while (!try_eat('>')) {
          const std::string key = word();
          expect('=');
          if (peek() == '[') a.fields[key] = int_list_brackets();
          else a.fields[key] = {integer()};
          try_eat(',');
        }
        return a;
      }
      if (try_str("#stablehlo<")) {  // #stablehlo<comparison_direction LT>
        word();
        a.text = word();
        expect('>');
        return a;
      }
      if (c == '@') {
        a.text = symbol();
        return a;
      }
      const size_t b = pos_;
      pos_++;
      while (pos_ < s_.size() && word_char(s_[pos_])) pos_++;
      if (peek() == '<') skip_group();
      a.text = s_.substr(b, pos_ - b);
      return a;
    }
    if (try_str("array<")) {
      word();  // element type
      if (try_eat(':')) {
        do {
          a.ints.push_back(integer());
        } while (try_eat(','));
      }
      expect('>');
      a.has_ints = true;
      return a;
    }
    if (try_str("dense<")) {
      // integer payloads only (shapes, dimension lists); tensor constants are parsed by parse_dense_literal
      if (peek() == '[') {
        a.ints = int_list_brackets();
      } else if (peek() != '>') {
        a.ints = {integer()};
      }
      expect('>');
      if (try_eat(':')) parse_type();
      a.has_ints = true;
      return a;
    }
    if (try_word("true")) {
      a.ints = {1};
      a.has_ints = true;
      return a;
    }
    if (try_word("false")) {
      a.ints = {0};
      a.has_ints = true;
      return a;
    }
    if (try_word("unit")) return a;
    if (c == '{') {  // nested dictionary (backend configs): not needed
      skip_group();
      return a;
    }
    if (isdigit((unsigned char)c) || c == '-') {
      size_t save = pos_;
      a.ints = {integer()};
      a.has_ints = true;
      if (pos_ < s_.size() && (s_[pos_] == '.' || s_[pos_] == 'e' || s_[pos_] == 'E')) {  // a float: keep as text
        pos_ = save;
        a.has_ints = false;
        a.ints.clear();
        size_t b = pos_;
        while (pos_ < s_.size() && (isalnum((unsigned char)s_[pos_]) || s_[pos_] == '.' || s_[pos_] == '-' || s_[pos_] == '+')) pos_++;
        a.text = s_.substr(b, pos_ - b);
      }
      // "2 : i64" carries its own type; "dim = 2 : tensor<...>" is followed by the operation's signature instead
      const size_t before_colon = pos_;
      if (try_eat(':')) {
        skip();
        if (s_.compare(pos_, 6, "tensor") == 0 || peek() == '(') pos_ = before_colon;
        else parse_type();
      }
      return a;
    }
    // bare word (enum value)
    a.text = word();
    if (peek() == '<') skip_group();
    return a;
  }
  // Skips one bracketed group including its brackets.
  void skip_group() {
    skip();
    int depth = 0;
    while (pos_ < s_.size()) {
      const char c = s_[pos_];
      if (c == '"') {
        string_literal();
        continue;
      }
      if (c == '(' || c == '[' || c == '{' || c == '<') depth++;
      if ((c == ')' || c == ']' || c == '}' || c == '>') && !(c == '>' && pos_ > 0 && s_[pos_ - 1] == '-')) {
        depth--;
        if (depth == 0) {
          pos_++;
          return;
        }
      }
      pos_++;
    }
    fail("unbalanced brackets");
  }
  // {a = 1 : i64, b = [..]}  or  <{...}>
  void parse_attr_dict(std::map<std::string, Attr>* out) {
    const bool props = try_str("<{");
    if (!props) expect('{');
    if (!try_eat('}')) {
      do {
        std::string key = peek() == '"' ? string_literal() : word();
        Attr a;
        if (try_eat('=')) a = parse_attr_value();
        (*out)[key] = a;
      } while (try_eat(','));
      expect('}');
    }
    if (props) expect('>');
  }

  // ---- dense constants ----------------------------------------------------------------------------------------
  void append_scalar(std::vector<uint8_t>* out, int dtype, const std::string& tok) {
    auto put = [&](const void* p, size_t n) { out->insert(out->end(), (const uint8_t*)p, (const uint8_t*)p + n); };
    if (dtype_is_float(dtype)) {
      double v;
      if (tok.size() > 2 && tok[0] == '0' && (tok[1] == 'x' || tok[1] == 'X')) {
        // bit pattern of the element type
        const uint64_t bits = strtoull(tok.c_str(), nullptr, 16);
        put(&bits, dtype_size(dtype));
        return;
      }
      v = strtod(tok.c_str(), nullptr);
      if (tok == "inf" || tok == "+inf") v = INFINITY;
      if (tok == "-inf") v = -INFINITY;
      if (tok == "nan" || tok == "-nan") v = NAN;
      if (dtype == kF64) {
        put(&v, 8);
      } else if (dtype == kF32) {
        float f = (float)v;
        put(&f, 4);
      } else if (dtype == kF16) {
        uint16_t h = float_to_half_bits((float)v);
        put(&h, 2);
      } else {
        uint16_t h = float_to_bf16_bits((float)v);
        put(&h, 2);
      }
      return;
    }
    int64_t v = tok == "true" ? 1 : tok == "false" ? 0 : (tok.size() > 2 && tok[1] == 'x') ? (int64_t)strtoull(tok.c_str(), nullptr, 16)
                                                                                         : strtoll(tok.c_str(), nullptr, 10);
    if (dtype == kU64) v = (int64_t)strtoull(tok.c_str(), nullptr, 0);
    put(&v, dtype_size(dtype));  // little endian
  }
  std::string scalar_token() {
    skip();
    size_t b = pos_;
    while (pos_ < s_.size() && (isalnum((unsigned char)s_[pos_]) || s_[pos_] == '.' || s_[pos_] == '-' || s_[pos_] == '+')) pos_++;
    if (b == pos_) fail("expected a number");
    return s_.substr(b, pos_ - b);
  }
  void parse_dense_elements(std::vector<uint8_t>* out, int dtype) {
    if (try_eat('[')) {
      if (try_eat(']')) return;
      do {
        parse_dense_elements(out, dtype);
      } while (try_eat(','));
      expect(']');
      return;
    }
    append_scalar(out, dtype, scalar_token());
  }
  // dense<...> : tensor<...>  ->  row-major bytes of the tensor
  std::vector<uint8_t> parse_dense_literal(Type* type_out) {
    if (!try_str("dense<")) fail("expected dense<...>");
    const size_t body = pos_;
    // find the type first (the payload cannot be encoded without the element type)
    int depth = 1;
    size_t p = pos_;
    while (p < s_.size() && depth > 0) {
      if (s_[p] == '"') {
        p++;
        while (p < s_.size() && s_[p] != '"') p++;
      } else if (s_[p] == '<') {
        depth++;
      } else if (s_[p] == '>') {
        depth--;
      }
      p++;
    }
    const size_t after = p;
    pos_ = after;
    expect(':');
    const Type t = parse_type();
    const size_t end = pos_;
    if (!t.tensor) fail("constant must be a tensor");
    *type_out = t;
    const uint64_t bytes = dense_byte_size(t.dtype, t.dims);
    std::vector<uint8_t> out;
    pos_ = body;
    skip();
    if (peek() == '"') {  // hex blob "0x..."
      const std::string hex = string_literal();
      if (hex.size() < 2 || hex[0] != '0' || (hex[1] != 'x' && hex[1] != 'X')) fail("expected a hex blob");
      for (size_t i = 2; i + 1 < hex.size(); i += 2) out.push_back((uint8_t)strtoul(hex.substr(i, 2).c_str(), nullptr, 16));
    } else {
      parse_dense_elements(&out, t.dtype);
    }
    const size_t esize = dtype_size(t.dtype);
    if (out.size() == esize && bytes > esize) {  // splat
      std::vector<uint8_t> one = out;
      out.clear();
      out.reserve(bytes);
      for (uint64_t i = 0; i < bytes / esize; i++) out.insert(out.end(), one.begin(), one.end());
    }
    if (out.size() != bytes) fail(strfmt("constant has %zu bytes, its type needs %llu", out.size(), (unsigned long long)bytes));
    pos_ = end;
    return out;
  }

  // ---- module level -------------------------------------------------------------------------------------------
  void parse_mesh() {  // sdy.mesh @mesh = <["x"=2, "y"=4]>
    const std::string name = symbol();
    expect('=');
    expect('<');
    int64_t size = 1;
    if (try_eat('[')) {
      if (!try_eat(']')) {
        do {
          string_literal();
          expect('=');
          size *= integer();
        } while (try_eat(','));
        expect(']');
      }
    }
    while (peek() != '>' && pos_ < s_.size()) pos_++;
    expect('>');
    mesh_size_[name] = size;
    plan_.num_partitions = (int32_t)std::max<int64_t>(plan_.num_partitions, size);
  }

  Sharding parse_sdy_sharding_text(const std::string& text) {
    // #sdy.sharding<@mesh, [{"x"}, {}]>: the first dimension with a named axis is the split dimension
    Sharding sh;
    const size_t at = text.find('@');
    if (at != std::string::npos) {
      size_t e = at + 1;
      while (e < text.size() && word_char(text[e])) e++;
      sh.mesh_name = text.substr(at + 1, e - at - 1);
    }
    const size_t lb = text.find('[');
    if (lb == std::string::npos) return sh;
    int64_t dim = -1, cur = 0;
    for (size_t i = lb + 1; i < text.size(); i++) {
      if (text[i] == '{') {
        size_t close = text.find('}', i);
        if (close == std::string::npos) break;
        if (text.find('"', i) < close && dim < 0) dim = cur;
        cur++;
        i = close;
      } else if (text[i] == ']') {
        break;
      }
    }
    if (dim >= 0) {
      sh.kind = ShardingKind::partitioned;
      sh.split_dim = dim;
    }
    return sh;
  }

  uint32_t add_value(ValueRole role, const Type& t) {
    Value v;
    v.id = (uint32_t)plan_.values.size();
    v.role = role;
    v.dtype = t.dtype;
    v.dims = t.dims;
    plan_.values.push_back(v);
    return v.id;
  }

  // Returns true when the function was imported as the entry point.
  bool parse_function(bool may_import) {
    skip();
    if (try_word("public") || try_word("private")) {
    }
    const std::string name = symbol();
    if (name != "main" || !may_import) {
      // another function (only @main is imported; a call to it is reported where it is used): skip it whole
      if (peek() != '(') fail("expected the argument list");
      skip_group();
      if (try_str("->")) {
        if (peek() == '(') skip_group();
        else {
          parse_type();
          if (peek() == '{' && result_attr_follows()) skip_group();
        }
      }
      if (try_word("attributes")) skip_group();
      if (peek() != '{') fail("expected a function body");
      skip_group();
      return false;
    }
    expect('(');
    std::vector<std::pair<uint32_t, uint32_t>> aliases;  // (output index, parameter index)
    if (!try_eat(')')) {
      do {
        skip();
        expect('%');
        const std::string arg = word();
        expect(':');
        const Type t = parse_type();
        if (!t.tensor) unsupported("func.func", pos_, &t);
        const uint32_t id = add_value(ValueRole::parameter, t);
        names_[arg] = {id};
        Sharding sh;
        const uint32_t pindex = (uint32_t)plan_.parameter_shardings.size();
        if (peek() == '{') {
          // argument attributes: raw scan for the ones that matter
          const size_t b = pos_;
          skip_group();
          const std::string attrs = s_.substr(b, pos_ - b);
          const size_t sd = attrs.find("#sdy.sharding<");
          if (sd != std::string::npos) sh = parse_sdy_sharding_text(attrs.substr(sd));
          if (attrs.find("jax.buffer_donor = true") != std::string::npos) plan_.donated_parameter_indices.push_back(pindex);
          const size_t al = attrs.find("tf.aliasing_output");
          if (al != std::string::npos) {
            size_t eq = attrs.find('=', al);
            if (eq != std::string::npos) {
              const uint32_t out_index = (uint32_t)strtoul(attrs.c_str() + eq + 1, nullptr, 10);
              plan_.donated_parameter_indices.push_back(pindex);
              aliases.push_back({out_index, pindex});
            }
          }
        }
        plan_.parameter_shardings.push_back(sh);
      } while (try_eat(','));
      expect(')');
    }
    if (try_str("->")) {
      if (peek() == '(') parse_type_list_parens();
      else {
        parse_type();
        if (peek() == '{' && result_attr_follows()) skip_group();
      }
    }
    if (try_word("attributes")) skip_group();
    expect('{');
    parse_body();
    for (auto& a : aliases)
      if (a.first < plan_.output_ids.size()) plan_.output_aliases.push_back(OutputAlias{a.first, a.second, 1});
    return true;
  }
  // After a single result type, "{...}" directly followed by "{" or "attributes" is a result attribute dictionary.
  bool result_attr_follows() {
    const size_t save = pos_;
    skip_group();
    skip();
    const bool yes = peek() == '{' || s_.compare(pos_, 10, "attributes") == 0;
    pos_ = save;
    return yes;
  }

  // ---- operations ---------------------------------------------------------------------------------------------
  uint32_t lookup(const std::string& ref) {
    // %name or %name#k
    std::string name = ref;
    size_t index = 0;
    const size_t hash = ref.find('#');
    if (hash != std::string::npos) {
      name = ref.substr(0, hash);
      index = (size_t)strtoul(ref.c_str() + hash + 1, nullptr, 10);
    }
    auto it = names_.find(name);
    if (it == names_.end() || index >= it->second.size()) fail("use of undefined value %" + ref);
    return it->second[index];
  }
  std::string value_ref() {
    skip();
    expect('%');
    size_t b = pos_;
    while (pos_ < s_.size() && (word_char(s_[pos_]) || s_[pos_] == '#')) pos_++;
    return s_.substr(b, pos_ - b);
  }

  static std::string plan_kind_name(const std::string& op) {
    static const std::map<std::string, std::string> kRename = {
        {"exponential", "exp"}, {"exponential_minus_one", "expm1"}, {"log_plus_one", "log1p"}, {"and", "and_"},
        {"or", "or_"}, {"xor", "xor_"}, {"not", "not_"}};
    auto it = kRename.find(op);
    return it == kRename.end() ? op : it->second;
  }

  void parse_body() {
    while (true) {
      skip();
      if (pos_ >= s_.size()) fail("unterminated function body");
      if (try_eat('}')) return;
      parse_operation();
    }
  }

  // Names of the operations inside the region(s) that follow, in order; the regions are consumed.
  std::vector<std::string> scan_region_ops() {
    std::vector<std::string> ops;
    const size_t b = pos_;
    skip_group();
    const std::string region = s_.substr(b, pos_ - b);
    size_t p = 0;
    while ((p = region.find("stablehlo.", p)) != std::string::npos) {
      size_t e = p + 10;
      while (e < region.size() && (isalnum((unsigned char)region[e]) || region[e] == '_')) e++;
      ops.push_back(region.substr(p + 10, e - p - 10));
      p = e;
    }
    return ops;
  }

  void parse_operation() {
    const size_t op_at = pos_;
    // results
    std::vector<std::string> result_names;
    std::vector<size_t> result_counts;
    if (peek() == '%') {
      do {
        skip();
        expect('%');
        std::string n = word();
        size_t count = 1;
        if (pos_ < s_.size() && s_[pos_] == ':') {
          pos_++;
          count = (size_t)integer();
        }
        result_names.push_back(n);
        result_counts.push_back(count);
      } while (try_eat(','));
      expect('=');
    }
    skip();
    bool generic = false;
    std::string full;
    if (peek() == '"') {
      generic = true;
      full = string_literal();
    } else {
      full = word();
    }
    if (full == "return" || full == "func.return" || full == "stablehlo.return") {
      std::vector<uint32_t> outs;
      if (peek() == '%') {
        do {
          outs.push_back(lookup(value_ref()));
        } while (try_eat(','));
        expect(':');
        do {
          parse_type();
        } while (try_eat(','));
      }
      plan_.output_ids = outs;
      plan_.output_shardings.assign(outs.size(), Sharding{});
      for (uint32_t o : outs)
        if (plan_.values[o].role == ValueRole::instruction_result) plan_.values[o].role = ValueRole::output;
      return;
    }
    std::string op = full;
    if (op.rfind("stablehlo.", 0) == 0) op = op.substr(10);
    else if (op.rfind("mhlo.", 0) == 0) op = op.substr(5);
    else if (op == "sdy.sharding_constraint" || op == "sdy.reshard") op = "sdy.alias";
    else unsupported(full, op_at, nullptr);

    std::vector<uint32_t> operands;
    std::map<std::string, Attr> attrs;
    std::vector<Type> in_types, out_types;
    std::vector<std::string> region_ops;
    std::vector<uint8_t> literal;
    std::string target;

    auto parse_signature = [&]() {
      expect(':');
      if (peek() == '(') {
        in_types = parse_type_list_parens();
        if (!try_str("->")) fail("expected '->'");
        if (peek() == '(') out_types = parse_type_list_parens();
        else out_types = {parse_type()};
      } else {
        std::vector<Type> list;
        do {
          list.push_back(parse_type());
        } while (try_eat(','));
        out_types = {list.back()};
      }
    };

    // Operations whose meaning lives in a region other than a reduce body, and the ones the plan cannot express.
    if (op == "while" || op == "case" || op == "if" || op == "sort" || op == "map" || op == "scatter" || op == "reduce_window" ||
        op == "select_and_scatter" || op == "convolution" || op == "all_reduce" || op == "all_gather" || op == "reduce_scatter" ||
        op == "collective_permute" || op == "all_to_all")
      unsupported("stablehlo." + op, op_at, nullptr);
    if (generic) {
      expect('(');
      if (!try_eat(')')) {
        do {
          operands.push_back(lookup(value_ref()));
        } while (try_eat(','));
        expect(')');
      }
      if (op == "constant") {
        // the value (a dense tensor, possibly floating point) lives in the property or attribute dictionary
        if (peek() != '<' && peek() != '{') fail("constant without a value");
        parse_constant_dict(&literal, &out_types);
      }
      if (peek() == '<') parse_attr_dict(&attrs);
      if (peek() == '(') region_ops = scan_region_ops();
      if (peek() == '{') parse_attr_dict(&attrs);
      const std::vector<Type> keep = out_types;
      parse_signature();
      if (!keep.empty()) out_types = keep;
    } else if (op == "constant") {
      Type t;
      literal = parse_dense_literal(&t);
      out_types = {t};
    } else if (op == "compare") {
      attrs["comparison_direction"].text = word();
      expect(',');
      operands.push_back(lookup(value_ref()));
      expect(',');
      operands.push_back(lookup(value_ref()));
      if (try_eat(',')) word();  // compare type
      parse_signature();
    } else if (op == "slice") {
      operands.push_back(lookup(value_ref()));
      expect('[');
      Attr start, limit, strides;
      do {
        start.ints.push_back(integer());
        expect(':');
        limit.ints.push_back(integer());
        strides.ints.push_back(try_eat(':') ? integer() : 1);
      } while (try_eat(','));
      expect(']');
      attrs["start_indices"] = start;
      attrs["limit_indices"] = limit;
      attrs["strides"] = strides;
      parse_signature();
    } else if (op == "reduce") {
      // stablehlo.reduce(%a init: %c), (%b init: %d) [applies stablehlo.add] across dimensions = [1] : sig [reducer...]
      std::vector<uint32_t> inits;
      do {
        expect('(');
        operands.push_back(lookup(value_ref()));
        if (!try_word("init")) fail("expected 'init:'");
        expect(':');
        inits.push_back(lookup(value_ref()));
        expect(')');
      } while (try_eat(','));
      operands.insert(operands.end(), inits.begin(), inits.end());
      if (try_word("applies")) {
        std::string body = word();
        if (body.rfind("stablehlo.", 0) == 0) body = body.substr(10);
        region_ops = {body};
      }
      if (!try_word("across")) fail("expected 'across dimensions'");
      if (!try_word("dimensions")) fail("expected 'dimensions'");
      expect('=');
      attrs["dimensions"].ints = int_list_brackets();
      parse_signature();
      if (try_word("reducer")) {
        while (peek() == '(') skip_group();
        region_ops = scan_region_ops();
      }
    } else if (op == "custom_call") {
      target = symbol();
      expect('(');
      if (!try_eat(')')) {
        do {
          operands.push_back(lookup(value_ref()));
        } while (try_eat(','));
        expect(')');
      }
      if (peek() == '{') parse_attr_dict(&attrs);
      parse_signature();
    } else {
      // operands, then `key = value` pairs, then an optional dictionary, then the types
      bool first = true;
      while (true) {
        skip();
        if (peek() == '%') {
          operands.push_back(lookup(value_ref()));
        } else if (peek() == ':' || peek() == '{') {
          break;
        } else {
          std::string key = word();
          expect('=');
          attrs[key] = parse_attr_value();
        }
        first = false;
        if (!try_eat(',')) break;
      }
      (void)first;
      if (peek() == '{') parse_attr_dict(&attrs);
      parse_signature();
    }
    if (generic && op == "custom_call" && attrs.count("call_target_name")) target = attrs["call_target_name"].text;

    emit(op, full, op_at, operands, attrs, out_types, region_ops, literal, target, result_names, result_counts);
  }

  // {value = dense<...> : tensor<...>} of a generic constant.
  void parse_constant_dict(std::vector<uint8_t>* literal, std::vector<Type>* out_types) {
    const bool props = try_str("<{");
    if (!props) expect('{');
    const std::string key = word();
    if (key != "value") fail("constant: expected 'value'");
    expect('=');
    Type t;
    *literal = parse_dense_literal(&t);
    *out_types = {t};
    expect('}');
    if (props) expect('>');
  }

  static std::vector<int64_t> list_of(const std::map<std::string, Attr>& attrs, std::initializer_list<const char*> keys) {
    for (const char* k : keys) {
      auto it = attrs.find(k);
      if (it != attrs.end()) return it->second.ints;
    }
    return {};
  }

  void emit(const std::string& op, const std::string& full, size_t op_at, std::vector<uint32_t> operands,
            std::map<std::string, Attr>& attrs, const std::vector<Type>& out_types, const std::vector<std::string>& region_ops,
            const std::vector<uint8_t>& literal, const std::string& target, const std::vector<std::string>& result_names,
            const std::vector<size_t>& result_counts) {
    for (const Type& t : out_types)
      if (!t.tensor) unsupported(full, op_at, &t);
    const Type* first_type = out_types.empty() ? nullptr : &out_types[0];
    auto bind_results = [&](const std::vector<uint32_t>& ids) {
      size_t k = 0;
      for (size_t r = 0; r < result_names.size(); r++) {
        std::vector<uint32_t> group;
        for (size_t c = 0; c < result_counts[r] && k < ids.size(); c++) group.push_back(ids[k++]);
        names_[result_names[r]] = group;
      }
    };
    if (op == "sdy.alias") {
      if (operands.size() != 1) fail("sharding constraint takes one operand");
      bind_results({operands[0]});
      return;
    }
    if (op == "optimization_barrier" && operands.size() > 1) {
      // one barrier per operand: the plan's barrier is a one-in one-out identity
      if (out_types.size() != operands.size()) fail("optimization_barrier: operand / result count mismatch");
      std::vector<uint32_t> ids;
      for (size_t k = 0; k < operands.size(); k++) {
        Instruction b;
        b.kind = Kind::optimization_barrier;
        b.inputs = {operands[k]};
        b.attrs["dims"] = out_types[k].dims;
        const uint32_t id = add_value(ValueRole::instruction_result, out_types[k]);
        b.outputs = {id};
        plan_.instructions.push_back(b);
        ids.push_back(id);
      }
      bind_results(ids);
      return;
    }
    Instruction ins;
    std::string kind = plan_kind_name(op);
    if (op == "constant") {
      ins.kind = Kind::constant;
      ins.literal = literal;
      const uint32_t id = add_value(ValueRole::constant, out_types.at(0));
      ins.outputs = {id};
      plan_.instructions.push_back(ins);
      bind_results({id});
      return;
    }
    auto set = [&](const char* name, const std::vector<int64_t>& v) { ins.attrs[name] = v; };
    const std::vector<int64_t> out_dims = first_type ? first_type->dims : std::vector<int64_t>{};
    if (op == "reduce") {
      const size_t n = operands.size() / 2;
      if (n == 0 || operands.size() != 2 * n || out_types.size() != n) fail("malformed reduce");
      operands.resize(n);  // the init values are the identities of the recognised bodies
      std::string body = region_ops.empty() ? "" : region_ops[0];
      if (n == 1) {
        static const std::map<std::string, std::string> kBody = {
            {"add", "reduce_sum"}, {"maximum", "reduce_max"}, {"minimum", "reduce_min"}, {"and", "reduce_and"}, {"or", "reduce_or"}};
        auto it = kBody.find(body);
        if (it == kBody.end()) unsupported("stablehlo.reduce(" + body + ")", op_at, first_type);
        kind = it->second;
      } else if (n == 2) {
        bool has_compare = false, has_select = false;
        for (const std::string& r : region_ops) {
          has_compare |= r == "compare";
          has_select |= r == "select";
        }
        if (!has_compare || !has_select) unsupported("stablehlo.reduce(variadic)", op_at, first_type);
        kind = "reduce_max";  // value / index pair (src/compiler/stablehlo_operation_attrs.zig:222-246)
      } else {
        unsupported("stablehlo.reduce(variadic)", op_at, first_type);
      }
      set("reduce_dimensions", list_of(attrs, {"dimensions"}));
      set("dims", out_dims);
    } else if (op == "compare") {
      static const std::map<std::string, int64_t> kDir = {{"EQ", 0}, {"NE", 1}, {"GE", 2}, {"GT", 3}, {"LE", 4}, {"LT", 5}};
      std::string d = attrs["comparison_direction"].text;
      auto it = kDir.find(d);
      if (it == kDir.end()) fail("unknown comparison direction " + d);
      set("compare_direction", {it->second});
    } else if (op == "reshape") {
      set("dims", out_dims);
    } else if (op == "transpose") {
      set("permutation", list_of(attrs, {"dims", "permutation"}));
      set("dims", out_dims);
    } else if (op == "broadcast_in_dim") {
      set("broadcast_dimensions", list_of(attrs, {"dims", "broadcast_dimensions"}));
      set("dims", out_dims);
    } else if (op == "broadcast") {
      // leading new dimensions: operand dimensions map to the trailing output dimensions
      kind = "broadcast_in_dim";
      const size_t orank = plan_.values[operands.at(0)].dims.size();
      std::vector<int64_t> bd;
      for (size_t d = 0; d < orank; d++) bd.push_back((int64_t)(out_dims.size() - orank + d));
      set("broadcast_dimensions", bd);
      set("dims", out_dims);
    } else if (op == "slice") {
      set("start_indices", list_of(attrs, {"start_indices"}));
      set("limit_indices", list_of(attrs, {"limit_indices"}));
      std::vector<int64_t> st = list_of(attrs, {"strides"});
      if (st.empty()) st.assign(out_dims.size(), 1);
      set("strides", st);
      set("dims", out_dims);
    } else if (op == "reverse") {
      set("dimensions", list_of(attrs, {"dims", "dimensions"}));
      set("dims", out_dims);
    } else if (op == "concatenate") {
      set("dimension", list_of(attrs, {"dim", "dimension"}));
      set("dims", out_dims);
    } else if (op == "iota") {
      set("iota_dimension", list_of(attrs, {"dim", "iota_dimension"}));
      set("dims", out_dims);
    } else if (op == "dynamic_slice") {
      set("slice_sizes", list_of(attrs, {"sizes", "slice_sizes"}));
      set("dims", out_dims);
    } else if (op == "dynamic_update_slice" || op == "optimization_barrier") {
      set("dims", out_dims);
    } else if (op == "pad") {
      set("edge_padding_low", list_of(attrs, {"low", "edge_padding_low"}));
      set("edge_padding_high", list_of(attrs, {"high", "edge_padding_high"}));
      set("interior_padding", list_of(attrs, {"interior", "interior_padding"}));
      set("dims", out_dims);
    } else if (op == "dot_general" || op == "dot") {
      kind = "dot_general";
      std::vector<int64_t> lb, rb, lc, rc;
      if (op == "dot") {
        lc = {(int64_t)plan_.values[operands.at(0)].dims.size() - 1};
        rc = {0};
      } else if (attrs.count("dot_dimension_numbers")) {
        auto& f = attrs["dot_dimension_numbers"].fields;
        lb = f["lhs_batching_dimensions"];
        rb = f["rhs_batching_dimensions"];
        lc = f["lhs_contracting_dimensions"];
        rc = f["rhs_contracting_dimensions"];
      } else {
        lb = attrs["batching_dims"].ints;
        rb = attrs["batching_dims"].ints2;
        lc = attrs["contracting_dims"].ints;
        rc = attrs["contracting_dims"].ints2;
      }
      set("lhs_batch_dimensions", lb);
      set("rhs_batch_dimensions", rb);
      set("lhs_contracting_dimensions", lc);
      set("rhs_contracting_dimensions", rc);
      set("dims", out_dims);
    } else if (op == "gather") {
      auto& f = attrs["dimension_numbers"].fields;
      set("offset_dims", f["offset_dims"]);
      set("collapsed_slice_dims", f["collapsed_slice_dims"]);
      set("start_index_map", f["start_index_map"]);
      set("operand_batching_dims", f["operand_batching_dims"]);
      set("start_indices_batching_dims", f["start_indices_batching_dims"]);
      set("index_vector_dim", f.count("index_vector_dim") ? f["index_vector_dim"] : std::vector<int64_t>{0});
      set("slice_sizes", list_of(attrs, {"slice_sizes"}));
      set("dims", out_dims);
    } else if (op == "custom_call") {
      ins.custom_call_target = target;
      set("dims", out_dims);
    }
    ins.kind = kind_from_name(kind);
    if (ins.kind == Kind::unsupported || ins.kind == Kind::all_reduce || ins.kind == Kind::all_gather) unsupported(full, op_at, first_type);
    ins.inputs = operands;
    std::vector<uint32_t> ids;
    for (const Type& t : out_types) ids.push_back(add_value(ValueRole::instruction_result, t));
    ins.outputs = ids;
    plan_.instructions.push_back(ins);
    bind_results(ids);
  }
};

}  // namespace

bool import_stablehlo_text(const std::string& text, Plan* plan, std::string* error) {
  try {
    Parser parser(text);
    *plan = parser.run();
    return true;
  } catch (const Fail& f) {
    if (error) *error = f.why;
    return false;
  }
}

}  // namespace pjrtx
